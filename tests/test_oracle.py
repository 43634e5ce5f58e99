"""CPU tests of the oracles: against vectors produced by the reference's own blockwise code
(tests/golden/make_golden.py) and against each other."""
import glob
import math
import os

import numpy as np
import pytest
import torch

from oracle import dense, philox
from oracle.block import BlockAttention

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "ref_jax_*.npz")))


def _arr(x):
    """npz array -> torch tensor; bfloat16 arrays are stored as 2-byte void records."""
    x = np.ascontiguousarray(x)
    if x.dtype.kind == "V" and x.dtype.itemsize == 2:
        return torch.from_numpy(x.view(np.int16)).view(torch.bfloat16)
    return torch.from_numpy(x)


def _t(x):  # golden arrays are [B, H, S, D]; the oracle takes [B, S, H, D]
    return _arr(x).permute(0, 2, 1, 3).contiguous()


def test_golden_files_present():
    assert len(GOLDEN) >= 7


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_block_oracle_matches_reference_vectors(path):
    g = np.load(path)
    q, k, v, do = (_t(g[n]) for n in ("q", "k", "v", "do"))
    f16 = q.dtype != torch.float32
    bias = _arr(g["bias"]) if g["bias"].size else None
    causal = bool(g["causal"])
    scale = float(g["scale"])
    block = int(g["block"])
    blk = BlockAttention(block, block, reference_rounding=f16)
    out, lse = blk.forward(q, k, v, bias=bias, causal=causal, softmax_scale=scale)
    ref_out, ref_lse = _t(g["out"]), torch.from_numpy(g["lse"])
    # fp32 vectors: same algorithm in the same precision -> agreement to rounding noise;
    # fp16 vectors: the reference rounds every block to fp16, the oracle reproduces the casts but
    # not their exact order, so the bound is a few fp16 ulps of O(1) values;
    # bf16 vectors: the same with bf16's 8-bit mantissa (one ulp of an O(1) value is 7.8e-3; the
    # reference keeps its running maximum and row sum in bf16, so its lse carries that error too).
    bf16 = q.dtype == torch.bfloat16
    tol_out, tol_lse = (2e-2, 2e-2) if bf16 else (6e-3, 4e-3) if f16 else (2e-5, 2e-5)
    assert (out.float() - ref_out.float()).abs().max().item() <= tol_out
    assert (lse - ref_lse).abs().max().item() <= tol_lse
    dq, dk, dv = blk.backward(do, q, k, v, ref_out, ref_lse, bias=bias, causal=causal,
                              softmax_scale=scale, out_dtype=torch.float32)
    # the reference differentiates w.r.t. the pre-scaled q: dq = scale * dq_wrt_scaled_q
    ref_dq = _t(g["dq_wrt_scaled_q"]).float() * scale
    ref_dk, ref_dv = _t(g["dk"]).float(), _t(g["dv"]).float()
    tol = 2e-2 if f16 else 2e-5     # measured: 1.4e-2 (bf16), 9e-4 (fp16), 4e-7 (fp32)
    for mine, ref in ((dq, ref_dq), (dk, ref_dk), (dv, ref_dv)):
        rel = ((mine - ref).norm() / ref.norm()).item()
        assert rel <= tol, rel


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("p_drop", [0.0, 0.25])
def test_block_matches_dense(causal, p_drop):
    torch.manual_seed(1)
    B, Sq, Sk, Hq, Hkv, D = 2, 200, 328, 4, 2, 64
    q = torch.randn(B, Sq, Hq, D).bfloat16()
    k = torch.randn(B, Sk, Hkv, D).bfloat16()
    v = torch.randn(B, Sk, Hkv, D).bfloat16()
    bias = torch.randn(B, 1, Sq, Sk).bfloat16()
    mask = torch.zeros(B, 1, 1, Sk).bfloat16()
    mask[..., Sk - 40:] = torch.finfo(torch.bfloat16).min
    do = torch.randn(B, Sq, Hq, D).bfloat16()
    kw = dict(bias=bias, mask=mask, causal=causal, dropout_p=p_drop, dropout_seed=11)
    blk = BlockAttention()
    o, lse = blk.forward(q, k, v, **kw)
    od, lsed = dense.attention(q, k, v, **kw)
    assert (o.double() - od).abs().max().item() < 1e-2       # o is rounded to bf16
    assert (lse.double() - lsed).abs().max().item() < 1e-5
    g = blk.backward(do, q, k, v, od.float(), lse, out_dtype=torch.float32, **kw)
    gd = dense.attention_grads(do, q, k, v, **kw)
    for a, b in zip(g, gd):
        assert ((a.double() - b).norm() / b.norm()).item() < 1e-5


def test_causal_is_bottom_right_aligned_and_dead_rows_are_zero():
    torch.manual_seed(2)
    q = torch.randn(1, 6, 1, 16)
    k = torch.randn(1, 4, 1, 16)
    v = torch.randn(1, 4, 1, 16)
    o, lse = BlockAttention(4, 4).forward(q, k, v, causal=True)
    # Sq=6 > Sk=4: query i sees key j iff j <= i - 2, so rows 0 and 1 see nothing
    assert torch.all(o[0, :2] == 0) and torch.all(torch.isinf(lse[0, 0, :2]))
    od, _ = dense.attention(q, k, v, causal=True)
    assert (o.double() - od).abs().max().item() < 1e-5


def test_philox_known_answers():
    # Random123 known-answer vectors for philox4x32-10
    out = philox.philox4x32_10(np.uint32(0), np.uint32(0), np.uint32(0), np.uint32(0), 0, 0)
    assert [int(x) for x in out] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    f = 0xFFFFFFFF
    out = philox.philox4x32_10(np.uint32(f), np.uint32(f), np.uint32(f), np.uint32(f), f, f)
    assert [int(x) for x in out] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    out = philox.philox4x32_10(np.uint32(0x243F6A88), np.uint32(0x85A308D3), np.uint32(0x13198A2E),
                               np.uint32(0x03707344), 0xA4093822, 0x299F31D0)
    assert [int(x) for x in out] == [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]


def test_dropout_keep_rate_and_determinism():
    p = 0.1
    m1 = philox.keep_mask(42, p, 2, 3, 64, 200)
    m2 = philox.keep_mask(42, p, 2, 3, 64, 200)
    m3 = philox.keep_mask(43, p, 2, 3, 64, 200)
    assert np.array_equal(m1, m2) and not np.array_equal(m1, m3)
    n = m1.size
    sigma = math.sqrt(p * (1 - p) / n)
    assert abs(m1.mean() - (1 - p)) < 4 * sigma
    # a shard (batch 1, heads 1..2) reproduces the bits of the full problem
    shard = philox.keep_mask(42, p, 1, 2, 64, 200, batch_offset=1, head_offset=1, heads_q_global=3)
    assert np.array_equal(shard, m1[1:, 1:3])
