"""GPU tests of the bit-reproducible backward (`deterministic`): the reference's dq is reproducible
from run to run because its dq program owns a query tile and adds the key tiles in a loop
(flash_attention_triton/_backward_triton.py:438-516); here the key tiles add their parts to a
float32 accumulator, by default in arrival order, with `deterministic` in descending order of
their index."""
import pytest
import torch

import workloads as W
from oracle.block import BlockAttention

pytestmark = pytest.mark.gpu

GRAD_TOL = 1e-2


def rel_l2(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-30)).item()


@pytest.mark.parametrize("case", [
    # more key-tile blocks (32 x 8 = 256) than SMs: blocks wait for blocks of earlier waves
    dict(B=1, Sq=4096, Sk=4096, Hq=32, Hkv=8, D=128, dtype=torch.bfloat16, causal=True, oracle=False),
    dict(B=2, Sq=1024, Sk=1024, Hq=8, Hkv=2, D=128, dtype=torch.float16, causal=True),
    dict(B=2, Sq=700, Sk=1000, Hq=4, Hkv=4, D=128, dtype=torch.bfloat16, causal=True),      # ragged, Sq != Sk
    dict(B=2, Sq=640, Sk=900, Hq=4, Hkv=2, D=64, dtype=torch.bfloat16, causal=False),
    dict(B=2, Sq=512, Sk=512, Hq=4, Hkv=2, D=64, dtype=torch.float16, causal=True, p=0.1, bias_heads=4),
    dict(B=2, Sq=520, Sk=520, Hq=4, Hkv=2, D=256, dtype=torch.bfloat16, causal=True),       # head dim 256 kernel
    dict(B=1, Sq=300, Sk=450, Hq=2, Hkv=2, D=192, dtype=torch.float16, causal=False, p=0.1),
    # per-batch lengths (one element empty): checked against the default path only
    dict(B=3, Sq=600, Sk=600, Hq=4, Hkv=2, D=96, dtype=torch.bfloat16, causal=True, lengths=(600, 130, 0),
         oracle=False),
])
def test_deterministic_backward_is_bit_reproducible(case):
    import jax_flash_attn2 as J
    B, Sq, Sk, Hq, Hkv, D = (case[k] for k in ("B", "Sq", "Sk", "Hq", "Hkv", "D"))
    dtype, causal, p, bias_heads = case["dtype"], case["causal"], case.get("p", 0.0), case.get("bias_heads", 0)
    q, k, v, do = W.make_qkv(B, Sq, Sk, Hq, Hkv, D, dtype, D ** -0.25)
    g = torch.Generator().manual_seed(11)
    bias = (0.5 * torch.randn(B, bias_heads, Sq, Sk, generator=g)).to(dtype) if bias_heads else None
    seqlens = torch.tensor(case["lengths"], dtype=torch.int32).cuda() if "lengths" in case else None
    dev = lambda x: None if x is None else x.cuda()
    qd, kd, vd, dod, bd = dev(q), dev(k), dev(v), dev(do), dev(bias)
    out, lse = J.fwd_attention_kernel_call(qd, kd, vd, None, bd, None, p, causal, 9, seqlens=seqlens)
    call = lambda det: J.bwd_attention_kernel_call(dod, qd, kd, vd, bd, None, out, lse, p, causal, None, 9,
                                                   seqlens=seqlens, deterministic=det)
    first = call(True)
    assert J.device_status() == 0
    for _ in range(3):
        again = call(True)
        for a, b in zip(first, again):
            assert torch.equal(a, b)
    assert J.device_status() == 0
    # the same gradients as the default path (dk, dv bitwise: only the order of the dq adds differs)
    plain = call(False)
    assert torch.equal(first[1], plain[1]) and torch.equal(first[2], plain[2])
    assert rel_l2(first[0], plain[0]) <= 1e-3
    if case.get("oracle", True):
        kw = dict(bias=bias, causal=causal, dropout_p=p, dropout_seed=9)
        ref = BlockAttention().backward(do, q, k, v, out.cpu(), lse.cpu()[:, :, :Sq], out_dtype=torch.float32, **kw)
        for mine, want in zip(first, ref):
            assert rel_l2(mine.cpu(), want) <= GRAD_TOL
