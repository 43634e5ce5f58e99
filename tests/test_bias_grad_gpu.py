"""GPU tests of what the library adds around the bias: its gradient (the reference returns none,
flash_attention_triton/_flash_attention.py:88), a bias with one head per key/value head read by
index instead of being repeated (the reference repeats it, flash_attention.py:161-164), the
shard offsets of the dropout stream given as a device operand, and the record of the dropout keep
bits that the forward can write for the backward."""
import pytest
import torch

import workloads as W
from oracle import dense
from oracle.block import BlockAttention

pytestmark = pytest.mark.gpu

OUT_TOL = {torch.bfloat16: 2e-2, torch.float16: 5e-3}
GRAD_TOL = 1e-2


def rel_l2(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-30)).item()


def _bias(shape, dtype, seed=5):
    g = torch.Generator().manual_seed(seed)
    return (0.5 * torch.randn(*shape, generator=g)).to(dtype)


@pytest.mark.parametrize("D,dtype,causal,Sq,Sk,bias_batch,bias_heads,p", [
    (128, torch.bfloat16, True, 256, 256, 2, 4, 0.0),      # one entry per (batch, query head): nothing shared
    (128, torch.bfloat16, False, 200, 328, 1, 1, 0.0),     # summed over batch and all heads
    (64, torch.float16, True, 300, 300, 2, 2, 0.1),        # one head per key/value head, with dropout
    (64, torch.bfloat16, False, 256, 320, 1, 4, 0.2),      # summed over the batch
    (256, torch.bfloat16, True, 200, 200, 2, 1, 0.0),      # head dim 256 kernel, summed over heads
    (256, torch.float16, False, 130, 257, 1, 2, 0.1),
    (96, torch.bfloat16, True, 256, 256, 2, 4, 0.0),       # padded head dim
])
def test_bias_gradient_against_both_oracles(D, dtype, causal, Sq, Sk, bias_batch, bias_heads, p):
    import jax_flash_attn2 as J
    B, Hq, Hkv, seed = 2, 4, 2, 77
    q, k, v, do = W.make_qkv(B, Sq, Sk, Hq, Hkv, D, dtype, D ** -0.25)
    bias = _bias((bias_batch, bias_heads, Sq, Sk), dtype)
    dev = lambda x: x.cuda()
    out, lse = J.fwd_attention_kernel_call(dev(q), dev(k), dev(v), None, dev(bias), None, p, causal, seed)
    dq, dk, dv, dbias = J.bwd_attention_kernel_call(dev(do), dev(q), dev(k), dev(v), dev(bias), None, out, lse,
                                                    p, causal, None, seed, bias_grad=True)
    assert J.device_status() == 0
    assert dbias.shape == bias.shape and dbias.dtype == torch.float32
    kw = dict(bias=bias, causal=causal, dropout_p=p, dropout_seed=seed)
    blk = BlockAttention()
    ro, _ = blk.forward(q, k, v, **kw)
    assert (out.cpu().float() - ro.float()).abs().max().item() <= OUT_TOL[dtype]
    ref = blk.backward(do, q, k, v, out.cpu(), lse.cpu()[:, :, :Sq], out_dtype=torch.float32, bias_grad=True, **kw)
    for name, mine, want in zip(("dq", "dk", "dv", "dbias"), (dq, dk, dv, dbias), ref):
        assert rel_l2(mine.cpu(), want) <= GRAD_TOL, (name, rel_l2(mine.cpu(), want))
    # the independent float64 dense oracle (its own forward, so a looser bound on 16-bit inputs)
    want64 = dense.attention_grads(do, q, k, v, bias_grad=True, **kw)[3]
    assert rel_l2(dbias.cpu().double(), want64) <= 2 * GRAD_TOL
    if causal and Sq == Sk:
        # entries above the diagonal take no gradient: they must have been cleared, not left over
        upper = torch.triu(torch.ones(Sq, Sk, dtype=torch.bool), diagonal=1)
        assert torch.all(dbias.cpu()[..., upper] == 0)


def test_bias_gradient_with_per_batch_lengths_is_zero_behind_the_length():
    import jax_flash_attn2 as J
    B, S, Hq, Hkv, D, dtype = 2, 256, 4, 2, 64, torch.bfloat16
    lengths = [256, 100]
    q, k, v, do = W.make_qkv(B, S, S, Hq, Hkv, D, dtype, D ** -0.25)
    bias = _bias((B, Hq, S, S), dtype)
    seqlens = torch.tensor(lengths, dtype=torch.int32).cuda()
    dev = lambda x: x.cuda()
    out, lse = J.fwd_attention_kernel_call(dev(q), dev(k), dev(v), None, dev(bias), None, 0.0, True, None, seqlens=seqlens)
    dbias = J.bwd_attention_kernel_call(dev(do), dev(q), dev(k), dev(v), dev(bias), None, out, lse, 0.0, True, None,
                                        None, seqlens=seqlens, bias_grad=True)[3].cpu()
    blk = BlockAttention()
    for b, n in enumerate(lengths):
        assert torch.all(dbias[b, :, n:, :] == 0) and torch.all(dbias[b, :, :, n:] == 0)
        sl = lambda x: x[b:b + 1, :n]
        bb = bias[b:b + 1, :, :n, :n]
        ro, rl = blk.forward(sl(q), sl(k), sl(v), bias=bb, causal=True)
        want = blk.backward(sl(do), sl(q), sl(k), sl(v), sl(out.cpu()), lse.cpu()[b:b + 1, :, :n], bias=bb, causal=True,
                            out_dtype=torch.float32, bias_grad=True)[3]
        assert rel_l2(dbias[b:b + 1, :, :n, :n], want) <= GRAD_TOL


def test_autograd_returns_the_bias_gradient_in_the_bias_dtype():
    import jax_flash_attn2 as J
    fa = J.create_flash_attention("gpu", "triton")
    q, k, v, do = W.make_qkv(1, 256, 256, 4, 2, 64, torch.bfloat16, 0.35)
    bias = _bias((1, 2, 256, 256), torch.bfloat16)        # one head per key/value head
    qd, kd, vd = (x.cuda().requires_grad_(True) for x in (q, k, v))
    bd = bias.cuda().requires_grad_(True)
    out = fa(qd, kd, vd, bias=bd, causal=True)
    out.backward(do.cuda())
    assert bd.grad is not None and bd.grad.dtype == torch.bfloat16 and bd.grad.shape == bias.shape
    want = dense.attention_grads(do, q, k, v, bias=bias, causal=True, bias_grad=True)
    for mine, ref in zip((qd.grad, kd.grad, vd.grad, bd.grad), want):
        assert rel_l2(mine.cpu().double(), ref) <= 2 * GRAD_TOL


@pytest.mark.parametrize("D", [64, 128, 256])
def test_bias_with_one_head_per_kv_head_is_read_by_index(D):
    """The kernels read bias head h // group for query head h; the result must be the one of the
    same bias repeated per group in memory (what the reference's `_handle_bias` builds), bit for
    bit in the forward and in dk / dv."""
    import jax_flash_attn2 as J
    B, S, Hq, Hkv, dtype = 2, 200, 8, 2, torch.bfloat16
    q, k, v, do = (x.cuda() for x in W.make_qkv(B, S, S, Hq, Hkv, D, dtype, D ** -0.25))
    bias = _bias((B, Hkv, S, S), dtype).cuda()
    rep = bias.repeat_interleave(Hq // Hkv, dim=1)
    o1, l1 = J.fwd_attention_kernel_call(q, k, v, None, bias, None, 0.1, True, 3)
    o2, l2 = J.fwd_attention_kernel_call(q, k, v, None, rep, None, 0.1, True, 3)
    assert torch.equal(o1, o2) and torch.equal(l1[:, :, :S], l2[:, :, :S])
    g1 = J.bwd_attention_kernel_call(do, q, k, v, bias, None, o1, l1, 0.1, True, None, 3)
    g2 = J.bwd_attention_kernel_call(do, q, k, v, rep, None, o1, l1, 0.1, True, None, 3)
    assert torch.equal(g1[1], g2[1]) and torch.equal(g1[2], g2[2]) and rel_l2(g1[0], g2[0]) < 1e-3
    assert J.device_status() == 0


def test_shard_offsets_read_from_device_memory_give_the_same_bits():
    """(batch_offset, head_offset) as an int32 [2] device operand must reproduce the results of the
    same offsets given by value: forward and backward, every kernel family."""
    import jax_flash_attn2 as J
    for D, dtype in ((64, torch.bfloat16), (128, torch.float16), (256, torch.bfloat16)):
        q, k, v, do = (x.cuda() for x in W.make_qkv(2, 200, 200, 4, 2, D, dtype, D ** -0.25))
        off = torch.tensor([3, 8], dtype=torch.int32, device="cuda")
        kw = dict(batch_offset=3, head_offset=8, heads_q_global=16)
        o1, l1 = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.2, True, 9, **kw)
        o2, l2 = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.2, True, 9, heads_q_global=16, offsets_dev=off)
        o3, _ = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.2, True, 9, heads_q_global=16)
        assert torch.equal(o1, o2) and torch.equal(l1[:, :, :200], l2[:, :, :200]) and not torch.equal(o1, o3)
        g1 = J.bwd_attention_kernel_call(do, q, k, v, None, None, o1, l1, 0.2, True, None, 9, **kw)
        g2 = J.bwd_attention_kernel_call(do, q, k, v, None, None, o1, l1, 0.2, True, None, 9, heads_q_global=16,
                                         offsets_dev=off)
        assert torch.equal(g1[1], g2[1]) and torch.equal(g1[2], g2[2]) and rel_l2(g1[0], g2[0]) < 1e-3
    assert J.device_status() == 0


def _decode_bit_record(bits, B, H, Sq, Sk):
    """uint32 record [B, H, ceil(Sq/128), ceil(Sk/128), 4, 128] -> bool [B, H, Sq, Sk]: word w of row
    r holds the flag of key 32 w + 2 p in bit p and that of key 32 w + 2 p + 1 in bit 16 + p."""
    nqt, nkt = (Sq + 127) // 128, (Sk + 127) // 128
    rec = bits.cpu().view(B, H, nqt, nkt, 4, 128).to(torch.int64) & 0xFFFFFFFF
    keep = torch.zeros(B, H, nqt * 128, nkt * 128, dtype=torch.bool)
    for w in range(4):
        words = rec[:, :, :, :, w, :]                      # [B, H, nqt, nkt, 128 rows]
        for p in range(16):
            for e in range(2):
                flag = ((words >> (p + 16 * e)) & 1).bool()   # key 32 w + 2 p + e of every tile
                col = 32 * w + 2 * p + e
                keep.view(B, H, nqt, 128, nkt, 128)[:, :, :, :, :, col] = flag.permute(0, 1, 2, 4, 3)
    return keep[:, :, :Sq, :Sk]


@pytest.mark.parametrize("D", [64, 128, 256])
def test_dropout_bit_record_holds_the_oracle_mask(D):
    """The forward's optional record of the keep bits must be the Philox mask of the oracle, bit for
    bit, for every head-dim kernel (non-causal: every tile is written)."""
    import jax_flash_attn2 as J
    from oracle import philox
    B, Sq, Sk, Hq, Hkv, p, seed = 2, 200, 328, 4, 2, 0.3, 99
    q, k, v, _ = (x.cuda() for x in W.make_qkv(B, Sq, Sk, Hq, Hkv, D, torch.bfloat16, D ** -0.25))
    bits = J.dropout_bits_buffer(q, k, p)
    bits.fill_(-1)
    o1, _ = J.fwd_attention_kernel_call(q, k, v, None, None, None, p, False, seed, dropout_bits=bits,
                                        batch_offset=1, head_offset=4, heads_q_global=12)
    o2, _ = J.fwd_attention_kernel_call(q, k, v, None, None, None, p, False, seed,
                                        batch_offset=1, head_offset=4, heads_q_global=12)
    assert torch.equal(o1, o2) and J.device_status() == 0
    want = torch.from_numpy(philox.keep_mask(seed, p, B, Hq, Sq, Sk, 1, 4, 12))
    assert torch.equal(_decode_bit_record(bits, B, Hq, Sq, Sk), want)
    assert J.dropout_bits_buffer(q, k, 0.0) is None


@pytest.mark.parametrize("D,causal,extras", [(64, True, False), (64, False, True), (32, True, False), (128, True, False)])
def test_backward_with_the_bit_record_equals_backward_that_redraws(D, causal, extras):
    """Given the forward's record, the head-dim-64 backward reads the keep bits from it instead of
    running Philox; the gradients must be those of the backward that draws the bits again (dk / dv
    bit for bit). Kernels that cannot stage the record (head dim 128) ignore it."""
    import jax_flash_attn2 as J
    B, S, Hq, Hkv, p, seed, dtype = 2, 300, 4, 2, 0.2, 5, torch.bfloat16
    q, k, v, do = (x.cuda() for x in W.make_qkv(B, S, S, Hq, Hkv, D, dtype, D ** -0.25))
    bias = _bias((B, 1, S, S), dtype).cuda() if extras else None
    seqlens = torch.tensor([300, 131], dtype=torch.int32).cuda() if extras else None
    bits = J.dropout_bits_buffer(q, k, p)
    out, lse = J.fwd_attention_kernel_call(q, k, v, None, bias, None, p, causal, seed, dropout_bits=bits, seqlens=seqlens)
    g1 = J.bwd_attention_kernel_call(do, q, k, v, bias, None, out, lse, p, causal, None, seed, dropout_bits=bits,
                                     seqlens=seqlens)
    g2 = J.bwd_attention_kernel_call(do, q, k, v, bias, None, out, lse, p, causal, None, seed, seqlens=seqlens)
    assert J.device_status() == 0
    assert torch.equal(g1[1], g2[1]) and torch.equal(g1[2], g2[2]) and rel_l2(g1[0], g2[0]) < 1e-3


def test_class_api_with_dropout_matches_the_dense_oracle_gradients():
    import jax_flash_attn2 as J
    fa = J.create_flash_attention("gpu", "triton")
    q, k, v, do = W.make_qkv(2, 256, 256, 4, 2, 64, torch.bfloat16, 0.35)
    qd, kd, vd = (x.cuda().requires_grad_(True) for x in (q, k, v))
    out = fa(qd, kd, vd, causal=True, dropout_prob=0.15, dropout_seed=21)
    out.backward(do.cuda())
    want = dense.attention_grads(do, q, k, v, causal=True, dropout_p=0.15, dropout_seed=21)
    for mine, ref in zip((qd.grad, kd.grad, vd.grad), want):
        assert rel_l2(mine.cpu().double(), ref) <= 2 * GRAD_TOL
