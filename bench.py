"""Benchmark of the attention hot path: forward + backward of one attention call per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Prints ONE JSON line (rank 0). At N=1 the workload is the Llama-3-8B-shaped causal bf16 config
(B=8, Hq=32, Hkv=8, S=4096, D=128); at N>1 every rank runs that same per-GPU workload on its own
batch slice of a global batch 8*N (independent (batch, kv-head) units, no collective on the
path: weak scaling). `value` is fwd+bwd attention TFLOP/s with inputs resident in HBM, timed with
CUDA events; `e2e` is the same metric through the host-buffer path (pinned host inputs copied in,
results copied out, inside the timed region). FLOPs: forward 4*B*Hq*Sq*Sk*D, halved for causal;
backward 2.5x forward.

Further records on the same line (skipped with --no-extras, e.g. under a profiler):
  sustained   the headline step repeated for >= 2 s, with the SM clock sampled meanwhile
  per_config  forward and forward+backward of the other benchmark configurations, a few steps each
  strong      the two configurations that are defined as sharded problems (long context over its
              key/value heads, head dim 256 over batch x heads), cut with the shard plan over the
              N ranks: time = slowest rank, plus a bitwise check of rank 0's shard against the
              same slice of the unsharded computation

`--impl reference` times the CPU restatement of the reference's blockwise JAX algorithm (the
reference itself needs jax, which is not installed) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "jax-flash-attn2_b200"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

import torch  # noqa: E402

METRIC = "attention TFLOP/s fwd & fwd+bwd per B200, % of bf16 tensor peak; 1/2/4/8 GPU"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# name -> (B, Sq, Sk, Hq, Hkv, D, dtype, causal, input scale)
WORKLOADS = {
    "llama3_8b_causal_bf16": (8, 4096, 4096, 32, 8, 128, torch.bfloat16, True, 1.0 / math.sqrt(128)),
    "readme_gqa_causal_fp16": (2, 512, 512, 16, 4, 64, torch.float16, True, 1.0),
    "long_context_causal_bf16": (1, 32768, 32768, 64, 8, 128, torch.bfloat16, True, 1.0 / math.sqrt(128)),
    "mha_bias_mask_dropout_bf16": (4, 2048, 2048, 16, 16, 64, torch.bfloat16, False, 1.0),
    "head_dim_256_causal_fp16": (4, 8192, 8192, 8, 8, 256, torch.float16, True, 1.0 / 16),
}
HEADLINE = "llama3_8b_causal_bf16"
# the configurations that are defined as sharded problems: (workload, what the plan splits)
STRONG = ("long_context_causal_bf16", "head_dim_256_causal_fp16")
# additive bias 1/(1+|i-j|), key-padding mask (valid length U[S/2, S] per batch element, finfo.min
# beyond it), dropout 0.1 with seed 42
WORKLOAD_EXTRAS = {"mha_bias_mask_dropout_bf16": {"bias": True, "mask": True, "dropout": 0.1, "seed": 42}}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the backward main kernel at the
# default workload, from the ncu capture summarised under profiles/ (--batch 2 capture: 365.7 MB
# read + 149.1 MB written; traffic grows with the batch, so x4 for the full launch).
BWD_MAIN_DRAM_TRAFFIC_BYTES = 2.06e9


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def flops_fwd(B, Sq, Sk, Hq, D, causal):
    f = 4.0 * B * Hq * Sq * Sk * D
    return 0.5 * f if causal else f


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.01):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:   # NVML missing: the clocks record says so
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksEventReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksEventReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksEventReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksEventReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        if self.ok:
            self.join(timeout=2)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


# ------------------------------------------------------------------------------------------------
# reference arm: CPU restatement of the reference's blockwise algorithm
# ------------------------------------------------------------------------------------------------
def cpu_sample(workload, seconds_budget=20.0):
    """Times forward + backward of (batch element, kv-head group) units of the workload with the
    CPU oracle on all host cores. Units are independent, so TFLOP/s of a sample of whole units is
    the throughput of the whole job. Returns (tflops, units_timed, seconds, cores)."""
    from oracle.block import BlockAttention
    import workloads as W
    B, Sq, Sk, Hq, Hkv, D, dtype, causal, scale = workload
    G = Hq // Hkv
    # very long sequences: time a prefix of the rows of one unit (still whole key range up to the diagonal)
    Sq_s, Sk_s = min(Sq, 4096), min(Sk, 4096)
    q, k, v, do = W.make_qkv(1, Sq_s, Sk_s, G, 1, D, dtype, scale)
    blk = BlockAttention(128, 128)
    unit_flops = 3.5 * flops_fwd(1, Sq_s, Sk_s, G, D, causal)
    t0 = time.perf_counter()
    units = 0
    while True:
        o, lse = blk.forward(q, k, v, causal=causal)
        blk.backward(do, q, k, v, o, lse, causal=causal)
        units += 1
        dt = time.perf_counter() - t0
        if dt > seconds_budget or units >= 4:
            break
    return unit_flops * units / dt / 1e12, units, dt, torch.get_num_threads(), (Sq_s, Sk_s, G)


def make_config(workload_name, workload, world, batch_override=0):
    """The `config` record of the JSON line: the same for the product arm and the reference arm."""
    B, Sq, Sk, Hq, Hkv, D, dtype, causal, _ = workload
    per_step = 2 * (2 * B * Sq * Hq * D + 2 * B * Sk * Hkv * D)      # q, dO, k, v in 16 bit
    return {
        "workload": workload_name + (f" (batch {batch_override})" if batch_override > 0 else ""),
        "shape_per_gpu": f"B={B} Sq={Sq} Sk={Sk} Hq={Hq} Hkv={Hkv} D={D} causal={causal}",
        "global_batch": B * world,
        "parallelism": f"{world} x independent (batch, kv-head) shards, no collective",
        "extras": WORKLOAD_EXTRAS.get(workload_name, {}),
        "l2": f"inputs ({per_step // (1 << 20)} MiB per step) vs the 126 MB L2; no explicit flush",
        "flops": "fwd 4*B*Hq*Sq*Sk*D (x0.5 causal), bwd 2.5x fwd",
    }


def run_reference(args, workload_name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = WORKLOADS[workload_name]
    if args.batch > 0:
        wl = (args.batch,) + wl[1:]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    B, Sq, Sk, Hq, Hkv, D, dtype, causal, _ = wl
    torch.set_num_threads(os.cpu_count() or 1)
    budget = max(2.0, 20.0 / max(1, args.steps + args.warmup))
    vals, ms = [], []
    sample_desc = ""
    for step in range(args.warmup + args.steps):
        tf, units, dt, cores, (sq_s, sk_s, g) = cpu_sample(wl, budget)
        sample_desc = (f"{units} unit(s) of (1 batch element x 1 kv head = {g} q heads), Sq={sq_s}, Sk={sk_s}, "
                       f"D={D}, fwd+bwd, block 128x128, torch CPU fp32")
        if step >= args.warmup:
            vals.append(tf)
            ms.append(dt * 1e3)
    v = statistics.mean(vals)
    line = {
        "impl": "reference",
        "metric": METRIC, "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": statistics.mean(ms), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 (cpu)", "data": "synthetic",
        "config": make_config(workload_name, wl, world, args.batch),
        "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample_desc},
        "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "reference JAX/CPU path cannot run (jax not installed); this is the CPU restatement of its blockwise algorithm",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# product arm
# ------------------------------------------------------------------------------------------------
class Inputs:
    """One attention problem on the current device (plus what its configuration adds)."""

    def __init__(self, name, workload, device_seed=None, host_seed=None, pinned=False):
        B, Sq, Sk, Hq, Hkv, D, dtype, causal, scale = workload
        self.name, self.shape, self.dtype, self.causal = name, (B, Sq, Sk, Hq, Hkv, D), dtype, causal
        self.host = None
        if host_seed is not None:
            # drawn on the host (the end-to-end leg copies these pinned buffers every step)
            g = torch.Generator().manual_seed(host_seed)
            draw = lambda shape, s: (torch.randn(shape, generator=g, dtype=torch.float32) * s).to(dtype)
            hq, hk, hv = draw((B, Sq, Hq, D), scale), draw((B, Sk, Hkv, D), scale), draw((B, Sk, Hkv, D), scale)
            hdo = draw((B, Sq, Hq, D), 1.0)
            if pinned:
                hq, hk, hv, hdo = (x.pin_memory() for x in (hq, hk, hv, hdo))
            self.host = (hq, hk, hv, hdo)
            self.q, self.k, self.v, self.do = (x.cuda(non_blocking=True) for x in self.host)
        else:
            # drawn on the device: every rank that uses the same seed holds the same tensors
            g = torch.Generator(device="cuda").manual_seed(device_seed)
            draw = lambda shape, s: (torch.randn(shape, generator=g, dtype=torch.float32, device="cuda") * s).to(dtype)
            self.q, self.k, self.v = draw((B, Sq, Hq, D), scale), draw((B, Sk, Hkv, D), scale), draw((B, Sk, Hkv, D), scale)
            self.do = draw((B, Sq, Hq, D), 1.0)
        extras = WORKLOAD_EXTRAS.get(name, {})
        self.extras = extras
        self.bias = self.mask = None
        self.p_drop, self.seed = float(extras.get("dropout", 0.0)), extras.get("seed")
        if extras.get("bias"):
            idx = torch.arange(Sq, device="cuda")
            bias = (1.0 / (1.0 + (idx[:, None] - idx[None, :Sk]).abs().float())).to(dtype)
            self.bias = bias[None, None].expand(B, 1, Sq, Sk).contiguous()
        if extras.get("mask"):
            lengths = torch.randint(Sk // 2, Sk + 1, (B,), generator=torch.Generator().manual_seed(4))
            mask = torch.zeros(B, 1, Sq, Sk, dtype=dtype)
            for bi in range(B):
                mask[bi, :, :, int(lengths[bi]):] = torch.finfo(dtype).min
            self.mask = mask.cuda()
        self.kw = {}
        self.drop_bits = None    # record of the dropout keep bits: written by the forward, read by the backward
        if self.p_drop > 0:
            from jax_flash_attn2 import dropout_bits_buffer
            self.drop_bits = dropout_bits_buffer(self.q, self.k, self.p_drop)
        torch.cuda.synchronize()

    def flops_fwd(self):
        B, Sq, Sk, Hq, _, D = self.shape
        return flops_fwd(B, Sq, Sk, Hq, D, self.causal)

    def shard(self, plan):
        """The slice of this problem a shard plan gives one rank (views, no copies)."""
        from jax_flash_attn2 import sharding
        G = self.shape[3] // self.shape[4]
        out = object.__new__(Inputs)
        out.__dict__.update(self.__dict__)
        out.q, out.k, out.v, out.do, out.kw = sharding.slice_inputs(plan, G, self.q, self.k, self.v, self.do)
        b0, b1 = plan.batch_start, plan.batch_stop
        h0, h1 = plan.kv_head_start * G, plan.kv_head_stop * G
        for name in ("bias", "mask"):
            t = getattr(self, name)
            if t is not None:
                t = t[b0:b1] if t.shape[0] > 1 else t
                setattr(out, name, t[:, h0:h1] if t.shape[1] > 1 else t)
        out.shape = (b1 - b0, self.shape[1], self.shape[2], h1 - h0, plan.kv_head_stop - plan.kv_head_start, self.shape[5])
        return out


def fwd_call(J, x):
    return J.fwd_attention_kernel_call(x.q, x.k, x.v, x.mask, x.bias, None, x.p_drop, x.causal, x.seed,
                                       dropout_bits=x.drop_bits, **x.kw)


def bwd_call(J, x, o, lse):
    return J.bwd_attention_kernel_call(x.do, x.q, x.k, x.v, x.bias, x.mask, o, lse, x.p_drop, x.causal, None, x.seed,
                                       dropout_bits=x.drop_bits, **x.kw)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="fa2_b200", choices=["fa2_b200", "reference"])
    ap.add_argument("--workload", default=HEADLINE, choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0,
                    help="run the workload with this batch size instead of its own (a smaller case of the "
                         "same kernels, e.g. for a profiler capture); the JSON line names it")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline measurement: no sustained / per_config / strong / e2e legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    if args.impl == "reference":
        run_reference(args, args.workload)
        return

    import jax_flash_attn2 as J
    from jax_flash_attn2 import _capi, sharding

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    workload = WORKLOADS[args.workload]
    if args.batch > 0:
        workload = (args.batch,) + workload[1:]
    B, Sq, Sk, Hq, Hkv, D, dtype, causal, scale = workload
    # every rank draws the same per-GPU batch slice shape; seeds differ per rank
    x = Inputs(args.workload, workload, host_seed=1000 + rank, pinned=True)
    hq, hk, hv, hdo = x.host
    extras, bias, mask, p_drop, seed = x.extras, x.bias, x.mask, x.p_drop, x.seed
    fwd = lambda: fwd_call(J, x)
    bwd = lambda o, lse: bwd_call(J, x, o, lse)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        return sharding.max_over_ranks(v, device="cuda")

    ev = lambda: torch.cuda.Event(enable_timing=True)
    f_fwd = x.flops_fwd()
    f_step = 3.5 * f_fwd
    gpu_index = physical_gpu_index(local_rank)

    def time_steps(fn, n):
        """Device time per call of fn over n back-to-back calls (CUDA events on the launching
        stream, barrier + synchronize on both sides), the slowest rank's."""
        barrier()
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / n)

    def step(inp=None):
        inp = x if inp is None else inp
        o_, lse_ = fwd_call(J, inp)
        bwd_call(J, inp, o_, lse_)

    # ---- warm-up -------------------------------------------------------------------------------
    for _ in range(args.warmup):
        step()
    barrier()

    # ---- timed region: K steps of fwd + bwd, device-resident inputs ----------------------------
    # An event between the forward and the backward of every step gives the forward's share inside
    # the step (the forward-only loop further down runs in another power state).
    marks = [(ev(), ev()) for _ in range(args.steps)]
    def marked_steps():
        for m0, m1 in marks:
            m0.record()
            o_, lse_ = fwd_call(J, x)
            m1.record()
            bwd_call(J, x, o_, lse_)
    sampler = ClockSampler(gpu_index)
    sampler.start()
    ms_step = time_steps(marked_steps, 1) / args.steps
    clocks = sampler.stop()
    ms_fwd_in_step = max_over_ranks(statistics.mean(m0.elapsed_time(m1) for m0, m1 in marks))
    status = J.device_status()

    # ---- forward alone, and the kernels of the backward (same K, separate loops) ---------------
    o, lse = fwd()
    ms_fwd = time_steps(fwd, args.steps)

    stage = [ev() for _ in range(4)]
    for e in stage:
        e.record()          # creates the underlying CUDA events
    torch.cuda.synchronize()
    lib = _capi.load()
    pre_ms, main_ms, conv_ms = [], [], []
    for _ in range(args.steps):
        arr = (C.c_void_p * 4)(*[C.c_void_p(e.cuda_event) for e in stage])
        lib.fa2_debug_bwd_stage_events(arr)
        bwd(o, lse)
        torch.cuda.synchronize()
        pre_ms.append(stage[0].elapsed_time(stage[1]))
        main_ms.append(stage[1].elapsed_time(stage[2]))
        conv_ms.append(stage[2].elapsed_time(stage[3]))
    ms_main = max_over_ranks(statistics.mean(main_ms))
    del o, lse

    peaks, peak_kind = load_peaks()
    peak_burst = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    peak_sust = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))

    # ---- sustained: the same step for at least two seconds -------------------------------------
    sustained = None
    if not args.no_extras:
        n_sust = max(args.steps, int(math.ceil(2000.0 / ms_step)) + 1)
        s2 = ClockSampler(gpu_index, period_s=0.02)
        s2.start()
        ms_sust = time_steps(step, n_sust)
        c2 = s2.stop()
        tf = f_step / (ms_sust * 1e-3) / 1e12
        sustained = {
            "steps": n_sust, "seconds": ms_sust * n_sust * 1e-3, "ms_per_step": ms_sust,
            "tflops_per_gpu": tf, "frac_of_sustained_peak": tf / peak_sust, "frac_of_burst_peak": tf / peak_burst,
            "clocks": c2,
            # time x clock: what the step costs in SM cycles, whatever clock the box granted
            "mcycles_per_step": (ms_sust * 1e-3) * (c2["sm_mhz"] or 0),
            "burst_mcycles_per_step": (ms_step * 1e-3) * (clocks["sm_mhz"] or 0),
        }

    ms_e2e = None
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo))
    d2h = h2d   # results o, dq (shaped like q) and dk, dv (like k, v): counted again from the buffers below
    if not args.no_extras:
        # ---- end to end: host buffers in, host buffers out, every step -----------------------------
        # Every step copies its inputs from pinned host memory and its results (o, dq, dk, dv) back to
        # pinned host memory inside the timed region. The three stages run on three streams over two
        # sets of device input buffers, so that step i+1's upload and step i-1's download overlap step
        # i's kernels (PCIe is full duplex); nothing is skipped or cached.
        q, k, v, do = x.q, x.k, x.v, x.do
        ho = torch.empty_like(hq).pin_memory()
        hdq = torch.empty_like(hq).pin_memory()
        hdk = torch.empty_like(hk).pin_memory()
        hdv = torch.empty_like(hv).pin_memory()
        in_sets = [(q, k, v, do), tuple(torch.empty_like(t) for t in (q, k, v, do))]
        s_in, s_comp, s_out = (torch.cuda.Stream() for _ in range(3))
        def e2e_run(n_steps):
            ev_in = [None, None]
            ev_free = [None, None]      # compute of the step that last used input set b has finished
            keep = []
            for i in range(n_steps):
                bset = i & 1
                dq_, dk_, dv_, ddo_ = in_sets[bset]
                with torch.cuda.stream(s_in):
                    if ev_free[bset] is not None:
                        s_in.wait_event(ev_free[bset])
                    dq_.copy_(hq, non_blocking=True); dk_.copy_(hk, non_blocking=True)
                    dv_.copy_(hv, non_blocking=True); ddo_.copy_(hdo, non_blocking=True)
                    ev_in[bset] = torch.cuda.Event(); ev_in[bset].record(s_in)
                with torch.cuda.stream(s_comp):
                    s_comp.wait_event(ev_in[bset])
                    o_, lse_ = J.fwd_attention_kernel_call(dq_, dk_, dv_, mask, bias, None, p_drop, causal, seed)
                    g_ = J.bwd_attention_kernel_call(ddo_, dq_, dk_, dv_, bias, mask, o_, lse_, p_drop, causal, None, seed)
                    ev_free[bset] = torch.cuda.Event(); ev_free[bset].record(s_comp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_free[bset])
                    for t_ in (o_, *g_):
                        t_.record_stream(s_out)
                    ho.copy_(o_, non_blocking=True); hdq.copy_(g_[0], non_blocking=True)
                    hdk.copy_(g_[1], non_blocking=True); hdv.copy_(g_[2], non_blocking=True)
                keep.append((o_, lse_, g_))
                if len(keep) > 2:
                    keep.pop(0)
            for st_ in (s_in, s_comp, s_out):
                torch.cuda.current_stream().wait_stream(st_)
        e2e_steps = max(3, min(args.steps, 10))
        e2e_run(2)
        barrier()
        e0, e1 = ev(), ev()
        e0.record()
        for st_ in (s_in, s_comp, s_out):
            st_.wait_event(e0)
        e2e_run(e2e_steps)
        e1.record()
        barrier()
        ms_e2e = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)
        h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo))
        d2h = sum(t.numel() * t.element_size() for t in (ho, hdq, hdk, hdv))
        del ho, hdq, hdk, hdv, in_sets, q, k, v, do

    # ---- the other configurations, a few steps each --------------------------------------------
    per_config, strong = {}, {}
    if not args.no_extras:
        del x
        torch.cuda.empty_cache()
        few = max(3, min(args.steps, 8))
        for name in sorted(WORKLOADS):
            if name == args.workload:
                continue
            y = Inputs(name, WORKLOADS[name], device_seed=2000 + rank)
            for _ in range(3):
                step(y)
            sm = ClockSampler(gpu_index)
            sm.start()
            ms_s = time_steps(lambda: step(y), few)
            cl = sm.stop()
            ms_f = time_steps(lambda: fwd_call(J, y), few)
            ff = y.flops_fwd()
            per_config[name] = {
                "shape_per_gpu": "B=%d Sq=%d Sk=%d Hq=%d Hkv=%d D=%d" % y.shape + f" causal={y.causal}",
                "dtype": "bf16" if y.dtype == torch.bfloat16 else "fp16", "extras": y.extras, "steps": few,
                "fwd_ms": ms_f, "fwd_bwd_ms": ms_s,
                "fwd_tflops": ff / (ms_f * 1e-3) / 1e12, "fwd_bwd_tflops": 3.5 * ff / (ms_s * 1e-3) / 1e12,
                "fwd_frac_of_peak": ff / (ms_f * 1e-3) / 1e12 / peak_burst,
                "fwd_bwd_frac_of_peak": 3.5 * ff / (ms_s * 1e-3) / 1e12 / peak_burst,
                "sm_mhz": cl["sm_mhz"], "reasons": cl["reasons"],
            }
            del y
            torch.cuda.empty_cache()

        # ---- strong scaling through the shard plan ---------------------------------------------
        for name in STRONG:
            full = Inputs(name, WORKLOADS[name], device_seed=3000)      # the same tensors on every rank
            Bf, _, _, _, Hkv_f, _ = full.shape
            mine = full.shard(sharding.plan(Bf, Hkv_f, world, rank))
            for _ in range(3):
                step(mine)
            ms_s = time_steps(lambda: step(mine), few)
            ms_f = time_steps(lambda: fwd_call(J, mine), few)
            ff = full.flops_fwd()
            rec = {
                "shape": "B=%d Sq=%d Sk=%d Hq=%d Hkv=%d D=%d" % full.shape,
                "shard_per_gpu": "B=%d Hq=%d Hkv=%d" % (mine.shape[0], mine.shape[3], mine.shape[4]),
                "units_per_gpu": mine.shape[0] * mine.shape[4], "steps": few,
                "fwd_ms": ms_f, "fwd_bwd_ms": ms_s,
                "fwd_tflops": ff / (ms_f * 1e-3) / 1e12, "fwd_bwd_tflops": 3.5 * ff / (ms_s * 1e-3) / 1e12,
            }
            if rank == 0:
                # the shard's results against the same slice of the unsharded computation
                o_s, l_s = fwd_call(J, mine)
                g_s = bwd_call(J, mine, o_s, l_s)
                o_f, l_f = fwd_call(J, full)
                g_f = bwd_call(J, full, o_f, l_f)
                G = full.shape[3] // full.shape[4]
                pl = sharding.plan(Bf, Hkv_f, world, 0)
                bs = slice(pl.batch_start, pl.batch_stop)
                hs, hk_ = slice(pl.kv_head_start * G, pl.kv_head_stop * G), slice(pl.kv_head_start, pl.kv_head_stop)
                rel = ((g_s[0].float() - g_f[0][bs, :, hs].float()).norm() / g_f[0][bs, :, hs].float().norm()).item()
                rec["shard_check"] = bool(
                    torch.equal(o_s, o_f[bs, :, hs]) and torch.equal(l_s, l_f[bs, hs]) and
                    torch.equal(g_s[1], g_f[1][bs, :, hk_]) and torch.equal(g_s[2], g_f[2][bs, :, hk_]) and rel < 1e-3)
                rec["shard_check_what"] = ("out, lse, dk, dv of rank 0's shard bitwise equal to the unsharded call; "
                                           f"dq (unordered fp32 reductions) rel-L2 {rel:.2e}")
                del o_s, l_s, g_s, o_f, l_f, g_f
            strong[name] = rec
            del full, mine
            torch.cuda.empty_cache()
        barrier()
        status |= J.device_status()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    value = f_step * world / (ms_step * 1e-3) / 1e12
    fwd_tflops = f_fwd * world / (ms_fwd * 1e-3) / 1e12
    main_tflops = 2.5 * f_fwd / (ms_main * 1e-3) / 1e12      # per GPU: a property of the kernel

    line = {
        "metric": METRIC,
        "value": value,
        "unit": "TFLOP/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16" if dtype == torch.bfloat16 else "fp16",
        "data": "synthetic",
        "config": make_config(args.workload, workload, world, args.batch),
        "per_gpu": {
            "fwd_bwd_tflops": value / world,
            "fwd_tflops": fwd_tflops / world,
            "fwd_ms": ms_fwd,
            "fwd_in_step_ms": ms_fwd_in_step,
            "fwd_in_step_tflops": f_fwd / (ms_fwd_in_step * 1e-3) / 1e12,
            "fwd_in_step_frac_of_peak": f_fwd / (ms_fwd_in_step * 1e-3) / 1e12 / peak_burst,
            "bwd_pre_ms": statistics.mean(pre_ms),
            "bwd_main_ms": ms_main,
            "bwd_dq_convert_ms": statistics.mean(conv_ms),
            "fwd_frac_of_peak": fwd_tflops / world / peak_burst,
            "fwd_bwd_frac_of_peak": value / world / peak_burst,
            "peak": f"{peak_burst} TFLOP/s bf16 burst, {peak_kind}",
        },
        "roofline": {
            "bound": "tensor",
            "kernel": "bwd_main_kernel",
            "achieved": main_tflops,
            "peak": peak_burst,
            "unit": "TFLOP/s",
            "frac": main_tflops / peak_burst,
            "frac_of_sustained_peak": main_tflops / peak_sust,
            "peak_source": f"{peak_kind}: cuBLAS bf16 burst {peak_burst}, sustained {peak_sust}",
            "traffic": BWD_MAIN_DRAM_TRAFFIC_BYTES if (args.workload == HEADLINE and args.batch <= 0) else None,
        },
        "e2e": None if ms_e2e is None else {
            "value": f_step * world / (ms_e2e * 1e-3) / 1e12,
            "unit": "TFLOP/s",
            "ms_per_step": ms_e2e,
            "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h,
            # per GPU and direction, while all N ranks copy at once (uploads, kernels and downloads
            # of consecutive steps overlap): what the host side of the box gives each rank
            "h2d_gbs": h2d / (ms_e2e * 1e-3) / 1e9,
            "d2h_gbs": d2h / (ms_e2e * 1e-3) / 1e9,
            "limit": "host-to-device copies (PCIe and host memory), not the kernels: see ms_per_step above",
        },
        "gpu_launches": 4 * args.steps,
        "device_status": status,
        "clocks": clocks,
    }
    if sustained is not None:
        line["sustained"] = sustained
    if per_config:
        line["per_config"] = per_config
    if strong:
        line["strong"] = {"scaling": "strong", "n_gpus": world, "configs": strong}
    if world == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        tf, units, dt, cores, (sq_s, sk_s, g_) = cpu_sample(workload, 15.0)
        line["cpu_baseline"] = {
            "value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{units} unit(s) of (1 batch element x 1 kv head = {g_} q heads), Sq={sq_s}, Sk={sk_s}, "
                      f"fwd+bwd with the CPU restatement of the reference's blockwise algorithm, {dt:.1f} s",
        }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
