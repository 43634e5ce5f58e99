"""GPU tests of the public class API, autograd, sharding equivalence and full-size properties."""
import math

import pytest
import torch

import workloads as W
from oracle import dense
from oracle.block import BlockAttention

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-30)).item()


def test_flash_attention_class_forward_and_grad():
    import jax_flash_attn2 as J
    fa = J.FlashAttention(J.AttentionConfig(platform=J.Platform.TRITON, backend=J.Backend.GPU))
    c = W.config1(batch=1, seq=256)
    q, k, v = (c[n].cuda().requires_grad_(True) for n in ("q", "k", "v"))
    out = fa(query=q, key=k, value=v, causal=True)
    loss = out.float().mean() * 1000.0
    loss.backward()
    od, _ = dense.attention(c["q"], c["k"], c["v"], causal=True)
    assert (out.detach().cpu().double() - od).abs().max().item() <= 5e-3
    do = torch.full_like(c["q"], 1000.0 / c["q"].numel(), dtype=torch.float32)
    gd = dense.attention_grads(do, c["q"], c["k"], c["v"], causal=True)
    for mine, ref in zip((q.grad, k.grad, v.grad), gd):
        assert rel_l2(mine.cpu(), ref) <= 2e-2


def test_class_rules_sq1_drops_causal_and_sq_ne_sk_drops_mask():
    import jax_flash_attn2 as J
    fa = J.create_flash_attention("gpu", "triton")
    q, k, v, _ = W.make_qkv(2, 1, 256, 4, 2, 64, torch.bfloat16)
    mask = torch.zeros(2, 1, 1, 256, dtype=torch.bfloat16)
    out = fa(q.cuda(), k.cuda(), v.cuda(), attention_mask=mask.cuda(), causal=True)
    od, _ = dense.attention(q, k, v, causal=False)
    assert (out.cpu().double() - od).abs().max().item() <= 2e-2


def test_2d_padding_mask_masks_keys_and_zeroes_padded_rows():
    import jax_flash_attn2 as J
    fa = J.create_flash_attention("gpu", "triton")
    B, S, H, D = 2, 256, 2, 64
    q, k, v, _ = W.make_qkv(B, S, S, H, H, D, torch.float16)
    lengths = [200, 77]
    m2 = torch.zeros(B, S, dtype=torch.int32)
    for b, n in enumerate(lengths):
        m2[b, :n] = 1
    out = fa(q.cuda(), k.cuda(), v.cuda(), attention_mask=m2.cuda(), causal=True).cpu()
    for b, n in enumerate(lengths):
        od, _ = dense.attention(q[b:b + 1, :n], k[b:b + 1, :n], v[b:b + 1, :n], causal=True)
        assert (out[b:b + 1, :n].double() - od).abs().max().item() <= 5e-3
        assert torch.all(out[b, n:] == 0)


def test_bias_with_kv_heads_is_repeated_per_group():
    import jax_flash_attn2 as J
    fa = J.create_flash_attention("gpu", "triton")
    q, k, v, _ = W.make_qkv(1, 128, 128, 4, 2, 64, torch.bfloat16)
    bias = (torch.randn(1, 2, 128, 128) * 0.5).bfloat16()
    out = fa(q.cuda(), k.cuda(), v.cuda(), bias=bias.cuda())
    od, _ = dense.attention(q, k, v, bias=bias.repeat_interleave(2, dim=1))
    assert (out.cpu().double() - od).abs().max().item() <= 2e-2


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_equals_unsharded_bitwise(world):
    """Every (batch, kv head) unit is independent: running the shards one after the other on one
    GPU must reproduce the unsharded result bit for bit, dropout included."""
    import jax_flash_attn2 as J
    from jax_flash_attn2 import sharding
    B, S, Hq, Hkv, D, p, seed = 2, 256, 8, 4, 64, 0.1, 7
    q, k, v, do = (x.cuda() for x in W.make_qkv(B, S, S, Hq, Hkv, D, torch.bfloat16))
    out, lse = J.fwd_attention_kernel_call(q, k, v, None, None, None, p, True, seed)
    dq, dk, dv = J.bwd_attention_kernel_call(do, q, k, v, None, None, out, lse, p, True, None, seed)
    G = Hq // Hkv
    for rank in range(world):
        sh = sharding.plan(B, Hkv, world, rank)
        qs, ks, vs, dos, kw = sharding.slice_inputs(sh, G, q, k, v, do)
        o_s, l_s = J.fwd_attention_kernel_call(qs, ks, vs, None, None, None, p, True, seed, **kw)
        b0, b1, h0, h1 = sh.batch_start, sh.batch_stop, sh.kv_head_start, sh.kv_head_stop
        assert torch.equal(o_s, out[b0:b1, :, h0 * G:h1 * G])
        assert torch.equal(l_s, lse[b0:b1, h0 * G:h1 * G])
        g = J.bwd_attention_kernel_call(dos, qs, ks, vs, None, None, o_s, l_s, p, True, None, seed, **kw)
        assert torch.equal(g[1], dk[b0:b1, :, h0:h1]) and torch.equal(g[2], dv[b0:b1, :, h0:h1])
        assert rel_l2(g[0], dq[b0:b1, :, h0 * G:h1 * G]) < 1e-2


def test_full_size_config2_properties():
    """Llama-3-8B-shaped causal bf16 attention at full size (B=8, S=4096, Hq=32, Hkv=8, D=128),
    checked through properties that need no full-size oracle:
      * causal prefix: the first 512 rows depend on the first 512 keys only;
      * one (batch, head) slice against the dense float64 oracle;
      * linearity of the backward in dO;  * rows of P sum to one => dO = const per row gives dq = 0.
    """
    import jax_flash_attn2 as J
    c = W.config2()
    q, k, v, do = (c[n].cuda() for n in ("q", "k", "v", "do"))
    out, lse = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.0, True, None)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    o_pre, l_pre = J.fwd_attention_kernel_call(q[:, :512], k[:, :512], v[:, :512], None, None, None, 0.0, True, None)
    assert torch.equal(o_pre, out[:, :512]) and torch.equal(l_pre, lse[:, :, :512])
    b, h = 3, 13
    od, ld = dense.attention(c["q"][b:b + 1, :1024, h:h + 1], c["k"][b:b + 1, :1024, h // 4:h // 4 + 1],
                             c["v"][b:b + 1, :1024, h // 4:h // 4 + 1], causal=True)
    assert (out[b:b + 1, :1024, h:h + 1].cpu().double() - od).abs().max().item() <= 2e-2
    assert (lse[b, h, :1024].cpu().double() - ld[0, 0]).abs().max().item() <= 1e-3
    dq, dk, dv = J.bwd_attention_kernel_call(do, q, k, v, None, None, out, lse, 0.0, True, None, None)
    dq2, dk2, dv2 = J.bwd_attention_kernel_call(do * 2, q, k, v, None, None, out, lse, 0.0, True, None, None)
    for a, b2 in ((dq, dq2), (dk, dk2), (dv, dv2)):
        assert torch.isfinite(a.float()).all()
        assert rel_l2(a.float() * 2, b2) <= 1e-2
    # one slice of the gradients against the dense oracle (keys of head group 2, batch 1, truncated problem)
    S = 768
    qs, ks, vs, dos = (x[1:2, :S] for x in (c["q"], c["k"], c["v"], c["do"]))
    o_s, l_s = J.fwd_attention_kernel_call(qs.cuda(), ks.cuda(), vs.cuda(), None, None, None, 0.0, True, None)
    g = J.bwd_attention_kernel_call(dos.cuda(), qs.cuda(), ks.cuda(), vs.cuda(), None, None, o_s, l_s, 0.0, True, None, None)
    gd = dense.attention_grads(dos, qs, ks, vs, causal=True)
    for mine, ref in zip(g, gd):
        assert rel_l2(mine.cpu(), ref) <= 1e-2


def test_config5_slice_properties_head_dim_256():
    """Config 5 shape family (fp16, D=256, causal) at reduced batch/heads but full sequence length
    for one head: causal prefix property and dense-oracle check of a slice."""
    import jax_flash_attn2 as J
    q, k, v, do = W.make_qkv(1, 8192, 8192, 2, 2, 256, torch.float16, 1.0 / 16)
    qc, kc, vc, doc = (x.cuda() for x in (q, k, v, do))
    out, lse = J.fwd_attention_kernel_call(qc, kc, vc, None, None, None, 0.0, True, None)
    o_pre, l_pre = J.fwd_attention_kernel_call(qc[:, :768], kc[:, :768], vc[:, :768], None, None, None, 0.0, True, None)
    assert torch.equal(o_pre, out[:, :768]) and torch.equal(l_pre, lse[:, :, :768])
    od, ld = dense.attention(q[:, :768, :1], k[:, :768, :1], v[:, :768, :1], causal=True)
    assert (out[:, :768, :1].cpu().double() - od).abs().max().item() <= 5e-3
    dq, dk, dv = J.bwd_attention_kernel_call(doc, qc, kc, vc, None, None, out, lse, 0.0, True, None, None)
    for g in (dq, dk, dv):
        assert torch.isfinite(g.float()).all()
    g = J.bwd_attention_kernel_call(doc[:, :768], qc[:, :768], kc[:, :768], vc[:, :768], None, None, o_pre, l_pre,
                                    0.0, True, None, None)
    gd = dense.attention_grads(do[:, :768], q[:, :768], k[:, :768], v[:, :768], causal=True)
    for mine, ref in zip(g, gd):
        assert rel_l2(mine.cpu(), ref) <= 1e-2


def _row_reference(q_row, k, v, do_row, scale, n_keys):
    """float64 attention of one query row over its first n_keys keys: (out, lse, dq)."""
    q_row, do_row = q_row.double(), do_row.double()
    kk, vv = k[:n_keys].double(), v[:n_keys].double()
    s = (kk @ q_row) * scale
    lse = torch.logsumexp(s, 0)
    p = torch.exp(s - lse)
    out = p @ vv
    dp = vv @ do_row
    ds = p * (dp - (p * dp).sum())
    return out, lse, (ds @ kk) * scale


def test_full_size_config4_row_samples_and_checksums():
    """Long-context config at full size (B=1, S=32768, Hq=64, Hkv=8, D=128, causal bf16), where no
    full oracle run is affordable. Checked through properties that do not depend on the size:
      * sampled query rows (first, last, tile edges, random) of out, lse and dq against a float64
        row-by-row computation over all of that row's keys;
      * sum_j dV_j = sum over the group's heads and rows of dO (rows of P sum to one);
      * sum(dK * K) = sum(dQ * Q) per kv head (both are scale * sum(dS * S))."""
    import jax_flash_attn2 as J
    c = W.config4()
    S, Hq, Hkv, D = 32768, 64, 8, 128
    G = Hq // Hkv
    scale = 1.0 / math.sqrt(D)
    q, k, v, do = (c[n].cuda() for n in ("q", "k", "v", "do"))
    out, lse = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.0, True, None)
    dq, dk, dv = J.bwd_attention_kernel_call(do, q, k, v, None, None, out, lse, 0.0, True, None, None)
    assert J.device_status() == 0
    g = torch.Generator().manual_seed(11)
    rows = [0, 1, 127, 128, 255, 256, 4095, 16384, S - 129, S - 1] + torch.randint(0, S, (14,), generator=g).tolist()
    heads = torch.randint(0, Hq, (len(rows),), generator=g).tolist()
    for i, h in zip(rows, heads):
        ro, rl, rdq = _row_reference(q[0, i, h], k[0, :, h // G], v[0, :, h // G], do[0, i, h], scale, i + 1)
        assert (out[0, i, h].double() - ro).abs().max().item() <= 2e-2, (i, h)
        assert abs(lse[0, h, i].item() - rl.item()) <= 1e-3, (i, h)
        assert rel_l2(dq[0, i, h].double(), rdq) <= 1e-2 or (dq[0, i, h].double() - rdq).abs().max().item() <= 1e-4, (i, h)
    # dV column sums per kv head
    sum_dv = dv[0].double().sum(0)                                   # [Hkv, D]
    sum_do = do[0].double().sum(0).view(Hkv, G, D).sum(1)
    assert rel_l2(sum_dv, sum_do) <= 1e-2
    # trace identity per kv head
    t_k = (dk[0].double() * k[0].double()).sum((0, 2))               # [Hkv]
    t_q = (dq[0].double() * q[0].double()).sum((0, 2)).view(Hkv, G).sum(1)
    assert rel_l2(t_k, t_q) <= 1e-2


def test_full_size_config3_one_batch_element_against_the_oracle():
    """Config 3 at full size (B=4, S=2048, H=16, D=64, bf16, bias + padding mask + dropout 0.1):
    the kernels run the whole problem; batch element 2 is compared with the CPU oracle, which
    draws the same dropout bits through the batch offset."""
    import jax_flash_attn2 as J
    c = W.config3()
    dev = {n: c[n].cuda() for n in ("q", "k", "v", "do", "bias", "mask")}
    p, seed = c["dropout_p"], c["dropout_seed"]
    out, lse = J.fwd_attention_kernel_call(dev["q"], dev["k"], dev["v"], dev["mask"], dev["bias"], None, p, False, seed)
    dq, dk, dv = J.bwd_attention_kernel_call(dev["do"], dev["q"], dev["k"], dev["v"], dev["bias"], dev["mask"],
                                             out, lse, p, False, None, seed)
    assert J.device_status() == 0
    b = 2
    sl = lambda x: x[b:b + 1]
    kw = dict(bias=sl(c["bias"]), mask=sl(c["mask"]), causal=False, dropout_p=p, dropout_seed=seed, batch_offset=b)
    blk = BlockAttention()
    ro, rl = blk.forward(sl(c["q"]), sl(c["k"]), sl(c["v"]), **kw)
    o_cpu, l_cpu = out[b:b + 1].cpu(), lse[b:b + 1].cpu()
    assert (o_cpu.float() - ro.float()).abs().max().item() <= 2e-2
    assert (l_cpu - rl).abs().max().item() <= 1e-3
    rq, rk, rv = blk.backward(sl(c["do"]), sl(c["q"]), sl(c["k"]), sl(c["v"]), o_cpu, l_cpu,
                              out_dtype=torch.float32, **kw)
    for mine, ref in ((dq, rq), (dk, rk), (dv, rv)):
        assert rel_l2(mine[b:b + 1].cpu(), ref) <= 1e-2


def test_calls_on_two_streams_and_two_host_threads_do_not_interfere():
    """The library keeps no state between calls (tensor maps live on the caller's stack, work goes
    to the stream handed in), so forward + backward of different problems may be in flight on
    different streams, issued from different host threads, at the same time."""
    import threading
    import jax_flash_attn2 as J
    problems = [W.make_qkv(2, 1024, 1024, 8, 2, 128, torch.bfloat16, 0.2),
                W.make_qkv(1, 777, 1300, 4, 4, 64, torch.float16, 0.3)]
    dev = [tuple(x.cuda() for x in pr) for pr in problems]
    serial = []
    for q, k, v, do in dev:
        o, l = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.0, True, None)
        g = J.bwd_attention_kernel_call(do, q, k, v, None, None, o, l, 0.0, True, None, None)
        serial.append((o, g))
    torch.cuda.synchronize()
    results = [None, None]
    def worker(i):
        q, k, v, do = dev[i]
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            for _ in range(5):
                o, l = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.0, True, None)
                g = J.bwd_attention_kernel_call(do, q, k, v, None, None, o, l, 0.0, True, None, None)
            s.synchronize()
        results[i] = (o, g)
    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for (o, g), (o_ref, g_ref) in zip(results, serial):
        assert torch.equal(o, o_ref) and torch.equal(g[1], g_ref[1]) and torch.equal(g[2], g_ref[2])
        assert rel_l2(g[0], g_ref[0]) < 1e-3
    assert J.device_status() == 0


def test_more_than_65535_batch_times_heads():
    """batch x heads beyond the 65535 limit of a grid's second dimension (every launch uses a
    one-dimensional grid): B=1100, H=64, 16 tokens each; three batch elements against the oracle."""
    import jax_flash_attn2 as J
    B, S, H, D = 1100, 16, 64, 64
    q, k, v, do = W.make_qkv(B, S, S, H, H, D, torch.bfloat16, 0.5)
    qc, kc, vc, doc = (x.cuda() for x in (q, k, v, do))
    out, lse = J.fwd_attention_kernel_call(qc, kc, vc, None, None, None, 0.0, True, None)
    dq, dk, dv = J.bwd_attention_kernel_call(doc, qc, kc, vc, None, None, out, lse, 0.0, True, None, None)
    assert J.device_status() == 0
    blk = BlockAttention()
    for b in (0, 517, B - 1):
        sl = lambda x: x[b:b + 1]
        ro, rl = blk.forward(sl(q), sl(k), sl(v), causal=True)
        assert (sl(out).cpu().float() - ro.float()).abs().max().item() <= 2e-2
        assert (lse[b:b + 1, :, :S].cpu() - rl).abs().max().item() <= 1e-3
        ref = blk.backward(sl(do), sl(q), sl(k), sl(v), sl(out).cpu(), lse[b:b + 1, :, :S].cpu(), causal=True,
                           out_dtype=torch.float32)
        for mine, want in zip((dq, dk, dv), ref):
            assert rel_l2(sl(mine).cpu(), want) <= 1e-2
