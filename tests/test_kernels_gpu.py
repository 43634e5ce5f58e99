"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracle.

Tolerances (from the build's target): output max-abs <= 2e-2 (bf16) / 5e-3 (fp16), lse within
1e-3, dq / dk / dv relative L2 <= 1e-2.
"""
import math

import numpy as np
import pytest
import torch

import workloads as W
from oracle import philox
from oracle.block import BlockAttention

pytestmark = pytest.mark.gpu

OUT_TOL = {torch.bfloat16: 2e-2, torch.float16: 5e-3}
LSE_TOL = 1e-3
GRAD_TOL = 1e-2


def _J():
    import jax_flash_attn2 as J
    return J


def rel_l2(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-30)).item()


def run_case(B, Sq, Sk, Hq, Hkv, D, dtype, causal, scale=1.0, bias_heads=0, mask_kind=None, p=0.0,
             softmax_scale=None, seed=42, backward=True):
    J = _J()
    q, k, v, do = W.make_qkv(B, Sq, Sk, Hq, Hkv, D, dtype, scale)
    g = torch.Generator().manual_seed(5)
    bias = None
    if bias_heads:
        bias = (0.5 * torch.randn(B, bias_heads, Sq, Sk, generator=g)).to(dtype)
    mask = None
    if mask_kind == "pad":       # key padding, finfo.min, broadcast over heads and rows
        mask = torch.zeros(B, 1, 1, Sk, dtype=dtype)
        for b in range(B):
            mask[b, ..., Sk - 17 * (b + 1):] = torch.finfo(dtype).min
    elif mask_kind == "full_f32":  # per-element fp32 mask with -inf entries
        mask = torch.zeros(B, 1, Sq, Sk, dtype=torch.float32)
        mask.masked_fill_(torch.rand(B, 1, Sq, Sk, generator=g) < 0.2, float("-inf"))
        mask[..., 0] = 0   # keep every row alive
    dev = lambda x: None if x is None else x.cuda()
    out, lse = J.fwd_attention_kernel_call(dev(q), dev(k), dev(v), dev(mask), dev(bias), softmax_scale, p, causal, seed)
    kw = dict(bias=bias, mask=mask, causal=causal, dropout_p=p, dropout_seed=seed, softmax_scale=softmax_scale)
    blk = BlockAttention()
    ro, rl = blk.forward(q, k, v, **kw)
    assert J.device_status() == 0
    o_cpu, l_cpu = out.cpu(), lse.cpu()[:, :, :Sq]
    assert not torch.isnan(o_cpu.float()).any()
    assert (o_cpu.float() - ro.float()).abs().max().item() <= OUT_TOL[dtype]
    fin = torch.isfinite(rl)
    assert torch.equal(torch.isfinite(l_cpu), fin)
    if fin.any():
        assert (l_cpu[fin] - rl[fin]).abs().max().item() <= LSE_TOL
    if not backward:
        return
    dq, dk, dv = J.bwd_attention_kernel_call(dev(do), dev(q), dev(k), dev(v), dev(bias), dev(mask), out, lse,
                                             p, causal, softmax_scale, seed)
    assert J.device_status() == 0
    rq, rk, rv = blk.backward(do, q, k, v, o_cpu, l_cpu, out_dtype=torch.float32, **kw)
    for name, mine, ref in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        m = mine.cpu()
        assert not torch.isnan(m.float()).any(), name
        assert rel_l2(m, ref) <= GRAD_TOL, (name, rel_l2(m, ref))


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
def test_basic_shapes(D, dtype, causal):
    run_case(2, 384, 384, 4, 2, D, dtype, causal)


@pytest.mark.parametrize("shape", [
    (1, 128, 128, 1, 1), (1, 1, 128, 2, 1), (1, 300, 300, 2, 2), (2, 200, 456, 2, 1),
    (1, 128, 384, 2, 1), (1, 384, 128, 2, 1), (1, 77, 513, 3, 3), (1, 640, 64, 2, 2),
])
@pytest.mark.parametrize("causal", [False, True])
def test_ragged_and_unequal_lengths(shape, causal):
    B, Sq, Sk, Hq, Hkv = shape
    run_case(B, Sq, Sk, Hq, Hkv, 128, torch.bfloat16, causal)


@pytest.mark.parametrize("shape,causal,dtype", [
    ((1, 128, 128, 1, 1), False, torch.float16), ((2, 512, 512, 2, 2), True, torch.bfloat16),
    ((1, 300, 457, 2, 1), True, torch.float16), ((1, 384, 128, 2, 2), True, torch.float16),
    ((1, 1, 200, 4, 2), False, torch.bfloat16), ((1, 64, 128, 1, 1), False, torch.float16),
    ((1, 640, 64, 2, 2), True, torch.bfloat16),
])
def test_head_dim_256(shape, causal, dtype):
    B, Sq, Sk, Hq, Hkv = shape
    run_case(B, Sq, Sk, Hq, Hkv, 256, dtype, causal, scale=1.0 / 16)


def test_head_dim_256_with_bias_mask_dropout():
    run_case(1, 256, 320, 2, 2, 256, torch.bfloat16, False, scale=1.0 / 16, bias_heads=1, mask_kind="pad", p=0.2)
    run_case(1, 200, 200, 4, 2, 256, torch.float16, True, scale=1.0 / 16, bias_heads=4, p=0.1)


@pytest.mark.parametrize("D,dtype,causal", [
    (8, torch.float16, False), (32, torch.bfloat16, True), (40, torch.float16, True),
    (56, torch.bfloat16, False), (80, torch.bfloat16, True), (96, torch.float16, False),
    (112, torch.bfloat16, True), (160, torch.float16, True), (192, torch.bfloat16, False),
    (224, torch.bfloat16, True),
])
def test_head_dims_between_the_kernel_sizes(D, dtype, causal):
    """Head dims other than 64 / 128 / 256 (the reference pads them: PADDED_HEADS,
    _forward_triton.py:337-346): the tensor maps cut the head dim into equal zero-padded blocks."""
    run_case(2, 200, 328, 4, 2, D, dtype, causal, scale=D ** -0.25)


def test_padded_head_dim_with_bias_mask_dropout():
    run_case(1, 256, 320, 2, 2, 96, torch.bfloat16, False, scale=0.3, bias_heads=1, mask_kind="pad", p=0.2)
    run_case(1, 200, 200, 4, 2, 192, torch.float16, True, scale=0.25, bias_heads=4, p=0.1)


@pytest.mark.parametrize("D,dtype,causal,S,lengths,extras", [
    (128, torch.bfloat16, True, 512, [512, 300, 128, 1], {}),
    (128, torch.bfloat16, False, 384, [200, 384, 0], {}),
    (64, torch.float16, True, 300, [77, 300], {}),
    (64, torch.bfloat16, False, 320, [129, 255], dict(bias_heads=4, p=0.2)),
    (256, torch.float16, True, 320, [200, 65, 320], {}),
    (256, torch.bfloat16, False, 256, [100, 256], dict(bias_heads=1, p=0.1)),
    (96, torch.bfloat16, True, 256, [256, 130], {}),
])
def test_per_batch_lengths(D, dtype, causal, S, lengths, extras):
    """Per-batch sequence lengths (the reference's varlen mode, _forward_triton.py:267-279): batch
    element b must come out as the attention over its first lengths[b] rows alone, with zeros
    behind them in the output and in all three gradients; what sits in the padding (large finite
    values here) must not matter."""
    J = _J()
    B, Hq, Hkv = len(lengths), 4, 2
    scale = D ** -0.25
    q, k, v, do = W.make_qkv(B, S, S, Hq, Hkv, D, dtype, scale)
    for b, n in enumerate(lengths):
        for x in (q, k, v, do):
            x[b, n:] = 50.0
    g = torch.Generator().manual_seed(9)
    bias_heads, p = extras.get("bias_heads", 0), extras.get("p", 0.0)
    bias = (0.5 * torch.randn(B, bias_heads, S, S, generator=g)).to(dtype) if bias_heads else None
    seqlens = torch.tensor(lengths, dtype=torch.int32)
    dev = lambda x: None if x is None else x.cuda()
    out, lse = J.fwd_attention_kernel_call(dev(q), dev(k), dev(v), None, dev(bias), None, p, causal, 11,
                                           seqlens=seqlens.cuda())
    dq, dk, dv = J.bwd_attention_kernel_call(dev(do), dev(q), dev(k), dev(v), dev(bias), None, out, lse, p,
                                             causal, None, 11, seqlens=seqlens.cuda())
    assert J.device_status() == 0
    out, lse, dq, dk, dv = (x.cpu() for x in (out, lse, dq, dk, dv))
    blk = BlockAttention()
    for b, n in enumerate(lengths):
        assert torch.all(out[b, n:] == 0) and torch.all(dq[b, n:] == 0)
        assert torch.all(dk[b, n:] == 0) and torch.all(dv[b, n:] == 0)
        assert torch.all(lse[b, :, n:S] == float("-inf"))
        if n == 0:
            continue
        sl = lambda x: x[b:b + 1, :n]
        kw = dict(bias=None if bias is None else bias[b:b + 1, :, :n, :n], causal=causal, dropout_p=p,
                  dropout_seed=11, batch_offset=b)
        ro, rl = blk.forward(sl(q), sl(k), sl(v), **kw)
        assert (sl(out).float() - ro.float()).abs().max().item() <= OUT_TOL[dtype]
        assert (lse[b:b + 1, :, :n] - rl).abs().max().item() <= LSE_TOL
        rq, rk, rv = blk.backward(sl(do), sl(q), sl(k), sl(v), sl(out), lse[b:b + 1, :, :n],
                                  out_dtype=torch.float32, **kw)
        for name, mine, ref in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
            if n == 1 and name != "dv":     # one key: the weight is 1 whatever q and k are
                assert sl(mine).float().abs().max().item() <= 1e-5 and ref.abs().max().item() <= 1e-5
                continue
            assert rel_l2(sl(mine), ref) <= GRAD_TOL, (name, b, rel_l2(sl(mine), ref))


def test_per_batch_lengths_on_a_split_problem():
    """Lengths and split-KV together: a low-occupancy problem (split along the keys) whose batch
    elements are shorter than the buffers."""
    J = _J()
    B, S, Hq, Hkv, D, dtype = 2, 2048, 2, 1, 128, torch.bfloat16
    lengths = [1500, 129]
    q, k, v, do = W.make_qkv(B, S, S, Hq, Hkv, D, dtype, D ** -0.25)
    seqlens = torch.tensor(lengths, dtype=torch.int32).cuda()
    args = (q.cuda(), k.cuda(), v.cuda(), None, None, None, 0.0, True, None)
    o_s, l_s = J.fwd_attention_kernel_call(*args, seqlens=seqlens)
    o_u, l_u = J.fwd_attention_kernel_call(*args, seqlens=seqlens, split_kv=False)
    assert J.device_status() == 0
    blk = BlockAttention()
    for b, n in enumerate(lengths):
        ro, rl = blk.forward(q[b:b + 1, :n], k[b:b + 1, :n], v[b:b + 1, :n], causal=True)
        for o, l in ((o_s, l_s), (o_u, l_u)):
            assert (o[b:b + 1, :n].cpu().float() - ro.float()).abs().max().item() <= OUT_TOL[dtype]
            assert (l[b:b + 1, :, :n].cpu() - rl).abs().max().item() <= LSE_TOL
            assert torch.all(o[b, n:] == 0) and torch.all(l[b, :, n:S] == float("-inf"))


def test_seqlens_needs_equal_sequence_lengths():
    J = _J()
    q, k, v, _ = W.make_qkv(1, 128, 256, 2, 2, 64, torch.bfloat16)
    with pytest.raises(AssertionError, match="QSeq != KSeq"):
        J.fwd_attention_kernel_call(q.cuda(), k.cuda(), v.cuda(), seqlens=torch.tensor([5], dtype=torch.int32).cuda())


@pytest.mark.parametrize("D,dtype,B,Sk,Hq,Hkv,causal", [
    (128, torch.bfloat16, 3, 1000, 32, 8, False), (128, torch.float16, 1, 129, 8, 1, True),
    (64, torch.bfloat16, 2, 4096, 16, 2, False), (256, torch.float16, 2, 300, 8, 4, True),
    (96, torch.bfloat16, 1, 77, 6, 3, False),
])
def test_decode_rows_with_grouped_heads(D, dtype, B, Sk, Hq, Hkv, causal):
    """One query row per head (decode). The library runs the query heads of a key/value head as
    rows of one tile (K and V are read once per group); the result, lse included, must be the one
    of the plain head-by-head computation, causal or not (a single row sees every key)."""
    J = _J()
    q, k, v, _ = W.make_qkv(B, 1, Sk, Hq, Hkv, D, dtype, D ** -0.25)
    out, lse = J.fwd_attention_kernel_call(q.cuda(), k.cuda(), v.cuda(), None, None, None, 0.0, causal, None)
    ro, rl = BlockAttention().forward(q, k, v, causal=False)
    assert J.device_status() == 0
    assert (out.cpu().float() - ro.float()).abs().max().item() <= OUT_TOL[dtype]
    assert (lse.cpu()[:, :, :1] - rl).abs().max().item() <= LSE_TOL
    # the same through [B, H, S, D] storage (head stride 1 row, sequence stride irrelevant)
    qt = q.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3).cuda()
    out2, lse2 = J.fwd_attention_kernel_call(qt, k.cuda(), v.cuda(), None, None, None, 0.0, causal, None)
    assert torch.equal(out2, out) and torch.equal(lse2[:, :, :1], lse[:, :, :1])


@pytest.mark.parametrize("case", [
    dict(B=1, Sq=1, Sk=32768, Hq=32, Hkv=8, D=128, dtype=torch.bfloat16, causal=False),   # decode, packed heads
    dict(B=2, Sq=1, Sk=5000, Hq=8, Hkv=8, D=64, dtype=torch.float16, causal=False),       # decode, MHA, ragged
    dict(B=1, Sq=256, Sk=4096, Hq=2, Hkv=1, D=128, dtype=torch.bfloat16, causal=True),    # short prefill chunk
    dict(B=1, Sq=300, Sk=3000, Hq=4, Hkv=2, D=96, dtype=torch.float16, causal=True, p=0.1, bias_heads=4),
    dict(B=1, Sq=2048, Sk=2048, Hq=4, Hkv=4, D=128, dtype=torch.bfloat16, causal=True),   # some splits see no key
    dict(B=1, Sq=1, Sk=9000, Hq=16, Hkv=4, D=256, dtype=torch.bfloat16, causal=False),    # decode, head dim 256
    dict(B=1, Sq=384, Sk=2500, Hq=2, Hkv=2, D=192, dtype=torch.float16, causal=True, p=0.1),
    # head dim 64: the bias tiles are staged through shared memory, also by the split items
    dict(B=1, Sq=256, Sk=4096, Hq=2, Hkv=1, D=64, dtype=torch.bfloat16, causal=True, p=0.1, bias_heads=2),
    dict(B=1, Sq=300, Sk=2048, Hq=2, Hkv=2, D=48, dtype=torch.float16, causal=False, bias_heads=1),
])
def test_split_kv_low_occupancy_problems(case):
    """Problems with few (batch, head, query tile) items are cut along the key sequence and merged
    by a second kernel. The library must report scratch for them, and the split result must agree
    with the unsplit one and with the oracle (dropout bits and bias included: both are indexed by
    absolute positions)."""
    J = _J()
    from jax_flash_attn2 import _capi
    import ctypes
    B, Sq, Sk, Hq, Hkv, D = (case[k] for k in ("B", "Sq", "Sk", "Hq", "Hkv", "D"))
    dtype, causal, p, bias_heads = case["dtype"], case["causal"], case.get("p", 0.0), case.get("bias_heads", 0)
    q, k, v, _ = W.make_qkv(B, Sq, Sk, Hq, Hkv, D, dtype, D ** -0.25)
    g = torch.Generator().manual_seed(3)
    bias = (0.5 * torch.randn(B, bias_heads, Sq, Sk, generator=g)).to(dtype) if bias_heads else None
    prob = _capi.Problem()
    prob.batch, prob.seqlen_q, prob.seqlen_k, prob.heads_q, prob.heads_kv, prob.head_dim = B, Sq, Sk, Hq, Hkv, D
    prob.dtype = _capi.FA2_BF16 if dtype == torch.bfloat16 else _capi.FA2_FP16
    prob.softmax_scale, prob.dropout_p, prob.causal = 1.0, p, int(causal)
    prob.heads_q_global = Hq
    assert _capi.load().fa2_fwd_workspace_bytes(ctypes.byref(prob)) > 0
    dev = lambda x: None if x is None else x.cuda()
    o_s, l_s = J.fwd_attention_kernel_call(dev(q), dev(k), dev(v), None, dev(bias), None, p, causal, 5)
    o_u, l_u = J.fwd_attention_kernel_call(dev(q), dev(k), dev(v), None, dev(bias), None, p, causal, 5, split_kv=False)
    assert J.device_status() == 0
    ro, rl = BlockAttention().forward(q, k, v, bias=bias, causal=causal and Sq > 1, dropout_p=p, dropout_seed=5)
    for o, l in ((o_s, l_s), (o_u, l_u)):
        assert (o.cpu().float() - ro.float()).abs().max().item() <= OUT_TOL[dtype]
        assert (l.cpu()[:, :, :Sq] - rl).abs().max().item() <= LSE_TOL
    assert (o_s.float() - o_u.float()).abs().max().item() <= OUT_TOL[dtype] / 2
    # The parts are kept and merged in fp32 and rounded to 16 bit once. What separates split from
    # unsplit is then the rounding of P against different running maxima: about one last place
    # of the 16-bit type (measured 2.8e-3 bf16, 3.7e-4 fp16 on these cases).
    assert rel_l2(o_s.cpu(), o_u.cpu().float()) <= {torch.bfloat16: 5e-3, torch.float16: 7e-4}[dtype]
    if Sq > 1:
        # the merged output and lse feed the backward like those of an unsplit forward
        do = torch.randn(B, Sq, Hq, D, generator=g).to(dtype)
        grads = J.bwd_attention_kernel_call(dev(do), dev(q), dev(k), dev(v), dev(bias), None, o_s, l_s, p,
                                            causal, None, 5)
        ref = BlockAttention().backward(do, q, k, v, o_s.cpu(), l_s.cpu()[:, :, :Sq], bias=bias, causal=causal,
                                        dropout_p=p, dropout_seed=5, out_dtype=torch.float32)
        for mine, want in zip(grads, ref):
            assert rel_l2(mine.cpu(), want) <= GRAD_TOL
        if p > 0:
            # the record of the keep bits written by split items serves the backward like any other
            bits = J.dropout_bits_buffer(dev(q), dev(k), p)
            o_r, l_r = J.fwd_attention_kernel_call(dev(q), dev(k), dev(v), None, dev(bias), None, p, causal, 5,
                                                   dropout_bits=bits)
            assert torch.equal(o_r, o_s)
            g_r = J.bwd_attention_kernel_call(dev(do), dev(q), dev(k), dev(v), dev(bias), None, o_s, l_s, p, causal,
                                              None, 5, dropout_bits=bits)
            assert torch.equal(g_r[1], grads[1]) and torch.equal(g_r[2], grads[2])


def _fuzz_cases(n, seed):
    g = torch.Generator().manual_seed(seed)
    pick = lambda xs: xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    cases = []
    for _ in range(n):
        D = pick([32, 64, 64, 96, 128, 128, 192, 256])
        hkv, grp = pick([1, 2, 3]), pick([1, 2, 4])
        sq = pick([1, 17, 128, 130, 257, 400, 513])
        sk = pick([sq, sq, 64, 200, 385, 640])
        feat = pick(["plain", "plain", "bias1", "biasH", "pad", "full_f32", "drop", "all"])
        if sk < 64 and feat in ("pad", "all"):
            feat = "full_f32"    # the key-padding mask of run_case would leave no key at all
        cases.append(dict(B=pick([1, 2, 3]), Sq=sq, Sk=sk, Hq=hkv * grp, Hkv=hkv, D=D,
                          dtype=pick([torch.bfloat16, torch.float16]), causal=pick([False, True]), feat=feat))
    return cases


@pytest.mark.parametrize("case", _fuzz_cases(28, 20240611), ids=lambda c: "-".join(str(v).replace("torch.", "") for v in c.values()))
def test_seeded_random_shapes(case):
    """A fixed, seeded sample of the argument space (shapes on and off the tile grid, grouped
    heads, every head-dim kernel, both dtypes, all score features) against the oracle."""
    feat = case["feat"]
    Hq = case["Hq"]
    run_case(case["B"], case["Sq"], case["Sk"], Hq, case["Hkv"], case["D"], case["dtype"], case["causal"],
             scale=case["D"] ** -0.25,
             bias_heads={"bias1": 1, "biasH": Hq, "all": 1}.get(feat, 0),
             mask_kind={"pad": "pad", "full_f32": "full_f32", "all": "pad"}.get(feat),
             p={"drop": 0.15, "all": 0.1}.get(feat, 0.0))


@pytest.mark.parametrize("shape,dtype,causal", [
    ((1, 256, 256, 2, 1), torch.bfloat16, True),       # one work item
    ((3, 700, 700, 8, 2), torch.float16, True),        # ragged rows, several groups
    ((2, 300, 513, 4, 2), torch.bfloat16, False),      # Sq != Sk, ragged keys
    ((1, 640, 64, 6, 1), torch.bfloat16, True),        # more query rows than keys: tiles without work
    ((2, 2048, 2048, 16, 4), torch.bfloat16, True),    # 256 work items: more than one per SM
    ((1, 1024, 1024, 2, 2), torch.float16, True),      # one head per group
])
def test_head_dim_128_grouped_heads_and_persistent_items(shape, dtype, causal):
    """Head dim 128 with grouped query heads: few and many work items per persistent CTA, items
    whose second query tile has no work, ragged rows and keys. Every row, and the backward fed
    with the forward's output, must match the oracle."""
    B, Sq, Sk, Hq, Hkv = shape
    run_case(B, Sq, Sk, Hq, Hkv, 128, dtype, causal, scale=128 ** -0.25)


def test_grouped_heads_forward_with_per_batch_lengths():
    J = _J()
    B, S, Hq, Hkv, D, dtype = 3, 512, 4, 2, 128, torch.bfloat16
    lengths = [512, 130, 0]
    q, k, v, _ = W.make_qkv(B, S, S, Hq, Hkv, D, dtype, D ** -0.25)
    seqlens = torch.tensor(lengths, dtype=torch.int32).cuda()
    out, lse = J.fwd_attention_kernel_call(q.cuda(), k.cuda(), v.cuda(), None, None, None, 0.0, True, None,
                                           seqlens=seqlens)
    assert J.device_status() == 0
    out, lse = out.cpu(), lse.cpu()
    blk = BlockAttention()
    for b, n in enumerate(lengths):
        assert torch.all(out[b, n:] == 0) and torch.all(lse[b, :, n:S] == float("-inf"))
        if n:
            ro, rl = blk.forward(q[b:b + 1, :n], k[b:b + 1, :n], v[b:b + 1, :n], causal=True)
            assert (out[b:b + 1, :n].float() - ro.float()).abs().max().item() <= OUT_TOL[dtype]
            assert (lse[b:b + 1, :, :n] - rl).abs().max().item() <= LSE_TOL


@pytest.mark.parametrize("G", [1, 2, 4, 8])
def test_gqa_groups(G):
    run_case(1, 256, 256, 8, 8 // G, 64, torch.float16, True)


@pytest.mark.parametrize("bias_heads,mask_kind,p", [
    (1, None, 0.0), (4, None, 0.0), (0, "pad", 0.0), (0, "full_f32", 0.0), (1, "pad", 0.1),
    (0, None, 0.3), (4, "full_f32", 0.2),
])
@pytest.mark.parametrize("causal", [False, True])
def test_bias_mask_dropout(bias_heads, mask_kind, p, causal):
    run_case(2, 256, 320, 4, 2, 64, torch.bfloat16, causal, bias_heads=bias_heads, mask_kind=mask_kind, p=p)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bias_shape,mask_shape", [
    ((2, 4, 256, 320), None), ((1, 1, 256, 320), (2, 1, 256, 320)), ((2, 2, 256, 320), (1, 4, 256, 320)),
])
def test_staged_score_terms_every_broadcast_pattern(dtype, bias_shape, mask_shape):
    """Head dim 64 streams 16-bit bias / mask tiles through shared memory (forward: per-warp TMA
    rings, backward: one tile per step). Every broadcast pattern of the two terms (batch 1 or B;
    heads 1, Hkv or Hq), both dtypes, with dropout on top, against the oracle."""
    J = _J()
    B, Sq, Sk, Hq, Hkv, D, p, seed = 2, 256, 320, 4, 2, 64, 0.1, 8
    q, k, v, do = W.make_qkv(B, Sq, Sk, Hq, Hkv, D, dtype, D ** -0.25)
    g = torch.Generator().manual_seed(6)
    bias = (0.5 * torch.randn(*bias_shape, generator=g)).to(dtype)
    mask = None
    if mask_shape is not None:
        mask = torch.zeros(*mask_shape, dtype=dtype)
        mask.masked_fill_(torch.rand(*mask_shape, generator=g) < 0.2, float("-inf"))
        mask[..., 0] = 0
    dev = lambda x: None if x is None else x.cuda()
    out, lse = J.fwd_attention_kernel_call(dev(q), dev(k), dev(v), dev(mask), dev(bias), None, p, True, seed)
    dq, dk, dv = J.bwd_attention_kernel_call(dev(do), dev(q), dev(k), dev(v), dev(bias), dev(mask), out, lse, p, True,
                                             None, seed)
    assert J.device_status() == 0
    kw = dict(bias=bias, mask=mask, causal=True, dropout_p=p, dropout_seed=seed)
    blk = BlockAttention()
    ro, rl = blk.forward(q, k, v, **kw)
    assert (out.cpu().float() - ro.float()).abs().max().item() <= OUT_TOL[dtype]
    fin = torch.isfinite(rl)
    assert (lse.cpu()[:, :, :Sq][fin] - rl[fin]).abs().max().item() <= LSE_TOL
    ref = blk.backward(do, q, k, v, out.cpu(), lse.cpu()[:, :, :Sq], out_dtype=torch.float32, **kw)
    for name, mine, want in zip(("dq", "dk", "dv"), (dq, dk, dv), ref):
        assert rel_l2(mine.cpu(), want) <= GRAD_TOL, (name, rel_l2(mine.cpu(), want))


def test_bias_misaligned_rows_take_the_scalar_path():
    run_case(1, 130, 203, 2, 2, 128, torch.float16, False, bias_heads=2, p=0.1)


def test_explicit_and_negative_softmax_scale():
    run_case(1, 256, 256, 2, 2, 64, torch.bfloat16, True, softmax_scale=0.05)
    run_case(1, 256, 256, 2, 2, 64, torch.bfloat16, False, softmax_scale=-0.05, backward=False)


def test_config1_shape_fp16_mean_loss():
    """Config 1: causal GQA fp16, q [2,512,16,64], loss = mean(out). The cotangent 2^-20 puts the
    gradients in fp16's subnormal range, so they are compared after scaling the cotangent to 1
    (the backward is linear in it) and, as stored, against the oracle rounded to fp16."""
    J = _J()
    c = W.config1()
    q, k, v = c["q"], c["k"], c["v"]
    out, lse = J.fwd_attention_kernel_call(q.cuda(), k.cuda(), v.cuda(), None, None, None, 0.0, True, None)
    blk = BlockAttention()
    ro, rl = blk.forward(q, k, v, causal=True)
    assert (out.cpu().float() - ro.float()).abs().max().item() <= OUT_TOL[torch.float16]
    assert (lse.cpu()[:, :, :512] - rl).abs().max().item() <= LSE_TOL
    ones = torch.ones_like(q)
    dq, dk, dv = J.bwd_attention_kernel_call(ones.cuda(), q.cuda(), k.cuda(), v.cuda(), None, None, out, lse,
                                             0.0, True, None, None)
    rq, rk, rv = blk.backward(ones, q, k, v, out.cpu(), lse.cpu()[:, :, :512], causal=True, out_dtype=torch.float32)
    for mine, ref in ((dq, rq), (dk, rk), (dv, rv)):
        assert rel_l2(mine.cpu(), ref) <= GRAD_TOL
    do = c["do"]
    dq, dk, dv = J.bwd_attention_kernel_call(do.cuda(), q.cuda(), k.cuda(), v.cuda(), None, None, out, lse,
                                             0.0, True, None, None)
    # As stored, the gradients are fp16 values of 1e-7..1e-5 on a 6e-8 grid: against the float32
    # oracle the storage format alone costs up to 13 %. Against the oracle rounded to fp16 the
    # kernel still has to meet 1e-2 (the backward rescales dS by a power of two taken from
    # max|dO|, so nothing underflows before that final rounding).
    s = float(do.flatten()[0])
    for mine, ref in ((dq, rq), (dk, rk), (dv, rv)):
        ref16 = (ref * s).to(torch.float16)
        assert rel_l2(mine.cpu(), ref16) <= GRAD_TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_cotangent_magnitude_does_not_matter(dtype):
    """dO scaled by 2^-10 or 2^10 must give gradients scaled by the same factor (to rounding):
    inputs and outputs stay in fp16's normal range, but without the internal power-of-two
    scaling dS = P (dP - delta) would underflow for the small cotangent."""
    J = _J()
    q, k, v, do = (x.cuda() for x in W.make_qkv(1, 256, 256, 4, 2, 64, dtype))
    out, lse = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.0, True, None)
    base = J.bwd_attention_kernel_call(do, q, k, v, None, None, out, lse, 0.0, True, None, None)
    for f in (2.0 ** -10, 2.0 ** 10):
        g = J.bwd_attention_kernel_call((do.float() * f).to(dtype), q, k, v, None, None, out, lse, 0.0, True, None, None)
        for a, b in zip(g, base):
            assert rel_l2(a.float() / f, b) <= GRAD_TOL


def test_dropout_mask_is_reproducible_and_keep_rate_matches():
    """With v = identity columns the output row is the dropped-out attention row itself, so the
    kernel's keep mask can be read back and compared bit for bit with the oracle's Philox bits."""
    J = _J()
    B, S, H, D, p, seed = 1, 128, 2, 128, 0.25, 1234
    q = torch.zeros(B, S, H, D, dtype=torch.float16)          # uniform attention: P = 1/S
    k = torch.zeros(B, S, H, D, dtype=torch.float16)
    v = torch.eye(S, D, dtype=torch.float16)[None, :, None, :].expand(B, S, H, D).contiguous()
    o1, _ = J.fwd_attention_kernel_call(q.cuda(), k.cuda(), v.cuda(), None, None, None, p, False, seed)
    o2, _ = J.fwd_attention_kernel_call(q.cuda(), k.cuda(), v.cuda(), None, None, None, p, False, seed)
    o3, _ = J.fwd_attention_kernel_call(q.cuda(), k.cuda(), v.cuda(), None, None, None, p, False, seed + 1)
    assert torch.equal(o1, o2) and not torch.equal(o1, o3)
    kept = (o1.cpu().float() > 0).permute(0, 2, 1, 3).numpy()          # [B, H, Sq, Sk]
    want = philox.keep_mask(seed, p, B, H, S, S)
    assert np.array_equal(kept, want)
    n = kept.size
    assert abs(kept.mean() - (1 - p)) < 4 * math.sqrt(p * (1 - p) / n)
    vals = o1.cpu().float()[o1.cpu().float() > 0]
    assert torch.allclose(vals, torch.full_like(vals, 1.0 / (S * (1 - p))), rtol=2e-3)


def test_seed_read_from_device_memory_gives_the_same_bits():
    """A seed handed over as a one-element int64 CUDA tensor is read by the kernels on the device;
    forward and backward must reproduce the results of the same seed given by value (seed above
    2^32 so that both key words matter), for every kernel family."""
    J = _J()
    seed = (7 << 32) + 12345
    for D, dtype in ((64, torch.bfloat16), (128, torch.float16), (256, torch.bfloat16)):
        q, k, v, do = (x.cuda() for x in W.make_qkv(2, 200, 200, 4, 2, D, dtype, D ** -0.25))
        seed_dev = torch.tensor([seed], dtype=torch.int64, device="cuda")
        o1, l1 = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.2, True, seed)
        o2, l2 = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.2, True, seed_dev)
        assert torch.equal(o1, o2) and torch.equal(l1[:, :, :200], l2[:, :, :200])   # lse is padded to 256
        g1 = J.bwd_attention_kernel_call(do, q, k, v, None, None, o1, l1, 0.2, True, None, seed)
        g2 = J.bwd_attention_kernel_call(do, q, k, v, None, None, o1, l1, 0.2, True, None, seed_dev)
        assert torch.equal(g1[1], g2[1]) and torch.equal(g1[2], g2[2]) and rel_l2(g1[0], g2[0]) < 1e-3
        seed_dev += 1    # a new seed in the same buffer: different bits, no host round trip
        o3, _ = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.2, True, seed_dev)
        assert not torch.equal(o1, o3)
    assert J.device_status() == 0


def test_calls_can_be_captured_in_a_cuda_graph():
    """The library launches on the given stream only and never synchronises, so forward and
    backward can be recorded into a CUDA graph (the way XLA command buffers replay custom calls)
    and replayed on new input values in the same buffers."""
    J = _J()
    q, k, v, do = (x.cuda() for x in W.make_qkv(2, 384, 384, 4, 2, 128, torch.bfloat16, 0.3))
    o_ref, l_ref = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.0, True, None)   # also warms up
    g_ref = J.bwd_attention_kernel_call(do, q, k, v, None, None, o_ref, l_ref, 0.0, True, None, None)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        o, l = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.0, True, None)
        g = J.bwd_attention_kernel_call(do, q, k, v, None, None, o, l, 0.0, True, None, None)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(o, o_ref) and torch.equal(g[1], g_ref[1]) and torch.equal(g[2], g_ref[2])
    q2, k2, v2, do2 = (x.cuda() for x in W.make_qkv(2, 384, 384, 4, 2, 128, torch.bfloat16, 0.2))
    o_ref2, l_ref2 = J.fwd_attention_kernel_call(q2, k2, v2, None, None, None, 0.0, True, None)
    g_ref2 = J.bwd_attention_kernel_call(do2, q2, k2, v2, None, None, o_ref2, l_ref2, 0.0, True, None, None)
    for dst, src in ((q, q2), (k, k2), (v, v2), (do, do2)):
        dst.copy_(src)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(o, o_ref2) and torch.equal(g[1], g_ref2[1]) and torch.equal(g[2], g_ref2[2])
    assert rel_l2(g[0], g_ref2[0]) < 1e-3
    assert J.device_status() == 0


def test_reruns_are_bitwise_identical_forward_and_dkdv():
    J = _J()
    q, k, v, do = (x.cuda() for x in W.make_qkv(2, 512, 512, 4, 2, 128, torch.bfloat16, 0.3))
    o1, l1 = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.0, True, None)
    o2, l2 = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.0, True, None)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    g1 = J.bwd_attention_kernel_call(do, q, k, v, None, None, o1, l1, 0.0, True, None, None)
    g2 = J.bwd_attention_kernel_call(do, q, k, v, None, None, o1, l1, 0.0, True, None, None)
    assert torch.equal(g1[1], g2[1]) and torch.equal(g1[2], g2[2])
    # dq is accumulated with floating-point reductions in arbitrary order: equal up to rounding
    assert rel_l2(g1[0], g2[0]) < 1e-2


def test_strided_inputs_bhsd_storage():
    """[B,H,S,D] storage viewed as [B,S,H,D] is taken through strides, without a copy."""
    J = _J()
    q, k, v, do = W.make_qkv(2, 256, 256, 4, 2, 64, torch.bfloat16)
    qs = q.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3).cuda()
    ks = k.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3).cuda()
    vs = v.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3).cuda()
    assert not qs.is_contiguous()
    o1, l1 = J.fwd_attention_kernel_call(qs, ks, vs, None, None, None, 0.0, True, None)
    o2, l2 = J.fwd_attention_kernel_call(q.cuda(), k.cuda(), v.cuda(), None, None, None, 0.0, True, None)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    g1 = J.bwd_attention_kernel_call(do.cuda(), qs, ks, vs, None, None, o1, l1, 0.0, True, None, None)
    g2 = J.bwd_attention_kernel_call(do.cuda(), q.cuda(), k.cuda(), v.cuda(), None, None, o2, l2, 0.0, True, None, None)
    assert torch.equal(g1[1], g2[1]) and torch.equal(g1[2], g2[2])


def test_unsupported_arguments_raise_before_launch():
    J = _J()
    from jax_flash_attn2._capi import Fa2Error
    for d in (72, 144, 320):     # not a multiple of 16 / of 32 / above 256
        q = torch.zeros(1, 128, 2, d, dtype=torch.bfloat16, device="cuda")
        with pytest.raises(Fa2Error, match="head_dim"):
            J.fwd_attention_kernel_call(q, q, q)
    q = torch.zeros(1, 128, 2, 64, dtype=torch.float32, device="cuda")
    with pytest.raises(AssertionError, match="fp16 and bf16"):
        J.fwd_attention_kernel_call(q, q, q)
    q = torch.zeros(1, 128, 2, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(Fa2Error, match="dropout_p"):
        J.fwd_attention_kernel_call(q, q, q, dropout_prob=1.5)
    assert J.device_status() == 0


def test_entry_points_work_on_a_host_thread_that_never_called_cuda():
    """A framework may call the library from a worker thread that has made no CUDA runtime call yet
    (torch's autograd thread when every allocation is served from the cache). The entry points must
    make the device context current themselves before they build their tensor maps."""
    import ctypes as C
    import threading
    J = _J()
    from jax_flash_attn2 import _capi
    from jax_flash_attn2._kernel_calls import _strides
    lib = _capi.load()
    q, k, v, _ = (x.cuda() for x in W.make_qkv(1, 256, 256, 2, 1, 64, torch.bfloat16, 0.35))
    ref, ref_lse = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.0, True, None)
    out, lse = torch.empty_like(ref), torch.empty_like(ref_lse)
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    a = _capi.FwdParams()
    a.p.batch, a.p.seqlen_q, a.p.seqlen_k, a.p.heads_q, a.p.heads_kv, a.p.head_dim = 1, 256, 256, 2, 1, 64
    a.p.dtype, a.p.causal, a.p.softmax_scale, a.p.heads_q_global = _capi.FA2_BF16, 1, 64 ** -0.5, 2
    for name, t in (("q", q), ("k", k), ("v", v), ("o", out)):
        setattr(a, name, t.data_ptr())
        setattr(a, name + "_strides", _strides(t))
    a.lse, a.lse_stride_b, a.lse_stride_h = lse.data_ptr(), lse.stride(0), lse.stride(1)
    result = {}

    def worker():       # no torch call in here: only the C ABI
        result["rc"] = lib.fa2_fwd(C.byref(a), C.c_void_p(stream))
        result["msg"] = lib.fa2_last_error()

    t = threading.Thread(target=worker)
    t.start()
    t.join()
    torch.cuda.synchronize()
    assert result["rc"] == 0, result["msg"]
    assert torch.equal(out, ref) and torch.equal(lse[:, :, :256], ref_lse[:, :, :256])
