"""The N > 1 path on CPU: two gloo ranks split one attention problem by (batch, kv head), each
runs the CPU oracle on its slice with the offsets the shard plan hands out, and the stitched result
must equal the unsharded one bit for bit (dropout included: the offsets keep the Philox counters
global). Also covers the max-over-ranks rule the benchmark uses for its timings."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    import workloads as W
    B, S, Hq, Hkv, D = 2, 128, 4, 2, 32
    q, k, v, do = W.make_qkv(B, S, S, Hq, Hkv, D, torch.bfloat16)
    return (B, S, Hq, Hkv, D), (q, k, v, do)


def _rank_main(rank: int, world: int, port: int, split: str, ok_flags):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "jax-flash-attn2_b200"))
    from jax_flash_attn2 import sharding
    from oracle.block import BlockAttention

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        (B, S, Hq, Hkv, D), (q, k, v, do) = _problem()
        if split == "heads":          # batch 1: the plan has to split the kv heads
            B, q, k, v, do = 1, q[:1], k[:1], v[:1], do[:1]
        G = Hq // Hkv
        kw = dict(causal=True, dropout_p=0.25, dropout_seed=3)
        blk = BlockAttention()
        sh = sharding.plan(B, Hkv, world, rank)
        qs, ks, vs, dos, off = sharding.slice_inputs(sh, G, q, k, v, do)
        o_s, l_s = blk.forward(qs, ks, vs, **kw, **off)
        g_s = blk.backward(dos, qs, ks, vs, o_s, l_s, out_dtype=torch.float32, **kw, **off)
        full = sharding.gather_shards(
            sh, G, [o_s, *g_s], [q.shape, q.shape, k.shape, v.shape], [False, False, True, True])
        o, lse = blk.forward(q, k, v, **kw)
        grads = blk.backward(do, q, k, v, o, lse, out_dtype=torch.float32, **kw)
        same = all(torch.equal(a, b.to(a.dtype)) for a, b in zip(full, [o, *grads]))
        # timing rule: every rank ends up with the slowest rank's figure
        slowest = sharding.max_over_ranks(10.0 + rank)
        ok_flags[rank] = int(same and slowest == 10.0 + world - 1 and sh.units * world == B * Hkv)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("split", ["batch", "heads"])
def test_two_gloo_ranks_reproduce_the_unsharded_result(split):
    world = 2
    ok_flags = mp.get_context("spawn").Array("i", [0] * world)
    mp.spawn(_rank_main, args=(world, _free_port(), split, ok_flags), nprocs=world, join=True)
    assert list(ok_flags) == [1] * world


def test_max_over_ranks_without_a_process_group():
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "jax-flash-attn2_b200"))
    from jax_flash_attn2 import sharding
    assert sharding.max_over_ranks(3.5) == 3.5
