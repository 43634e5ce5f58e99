"""CPU tests of the benchmark's bookkeeping: the record both arms print, the FLOP convention and the
shard plan the strong-scaling leg uses (the measurement itself needs a GPU)."""
import importlib.util
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("fa2_bench", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_both_arms_describe_the_workload_with_the_same_record():
    b = _bench()
    wl = b.WORKLOADS[b.HEADLINE]
    cfg = b.make_config(b.HEADLINE, wl, 1)
    assert cfg["workload"] == "llama3_8b_causal_bf16"
    assert cfg["shape_per_gpu"] == "B=8 Sq=4096 Sk=4096 Hq=32 Hkv=8 D=128 causal=True"
    assert cfg["global_batch"] == 8 and b.make_config(b.HEADLINE, wl, 8)["global_batch"] == 64
    assert "640 MiB" in cfg["l2"]                       # q, dO 256 MiB each, k, v 64 MiB each
    small = b.make_config(b.HEADLINE, (2,) + wl[1:], 1, batch_override=2)
    assert small["workload"].endswith("(batch 2)") and "B=2 " in small["shape_per_gpu"]


def test_flop_convention_and_workload_table():
    b = _bench()
    # forward 4*B*Hq*Sq*Sk*D, halved when causal; the benchmark configurations' figures
    assert b.flops_fwd(8, 4096, 4096, 32, 128, True) == 4.0 * 8 * 32 * 4096 * 4096 * 128 / 2
    B, Sq, Sk, Hq, Hkv, D, dtype, causal, _ = b.WORKLOADS["mha_bias_mask_dropout_bf16"]
    assert (B, Sq, Hq, Hkv, D, dtype, causal) == (4, 2048, 16, 16, 64, torch.bfloat16, False)
    assert abs(b.flops_fwd(B, Sq, Sk, Hq, D, causal) - 6.872e10) / 6.872e10 < 1e-3
    assert set(b.STRONG) <= set(b.WORKLOADS) and b.HEADLINE in b.WORKLOADS
    assert b.WORKLOAD_EXTRAS["mha_bias_mask_dropout_bf16"]["dropout"] == 0.1


def test_strong_scaling_shards_cover_the_two_sharded_configurations():
    b = _bench()
    from jax_flash_attn2 import sharding
    for name in b.STRONG:
        B, _, _, Hq, Hkv, *_ = b.WORKLOADS[name]
        for world in (1, 2, 4, 8):
            units = [sharding.plan(B, Hkv, world, r).units for r in range(world)]
            assert sum(units) == B * Hkv and len(set(units)) == 1   # every unit once, equal shares
