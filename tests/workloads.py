"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

The reference draws its inputs from jax PRNG keys 0/1/2; without jax those streams cannot be
reproduced, and parity only needs both sides to see the same arrays, so the tensors are drawn on
the CPU with torch generators seeded q=0, k=1, v=2, dO=3, lengths=4 and then cast to 16 bit.
"""
from __future__ import annotations

import math

import torch


def _normal(shape, seed, scale, dtype):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * scale).to(dtype)


def make_qkv(B, Sq, Sk, Hq, Hkv, D, dtype, scale=1.0, with_do=True):
    q = _normal((B, Sq, Hq, D), 0, scale, dtype)
    k = _normal((B, Sk, Hkv, D), 1, scale, dtype)
    v = _normal((B, Sk, Hkv, D), 2, scale, dtype)
    do = _normal((B, Sq, Hq, D), 3, 1.0, dtype) if with_do else None
    return q, k, v, do


def config1(batch=2, seq=512):
    """Causal GQA, fp16: q [B,16,S,64] generated in [B,H,S,D] then viewed as [B,S,H,D]."""
    dt = torch.float16
    q = _normal((batch, 16, seq, 64), 0, 1.0, dt).permute(0, 2, 1, 3).contiguous()
    k = _normal((batch, 4, seq, 64), 1, 1.0, dt).permute(0, 2, 1, 3).contiguous()
    v = _normal((batch, 4, seq, 64), 2, 1.0, dt).permute(0, 2, 1, 3).contiguous()
    do = torch.full_like(q, 1.0 / q.numel())   # gradient of mean(out)
    return dict(q=q, k=k, v=v, do=do, causal=True)


def config2(batch=8, seq=4096, hq=32, hkv=8):
    """Llama-3-8B-shaped causal bf16 attention."""
    q, k, v, do = make_qkv(batch, seq, seq, hq, hkv, 128, torch.bfloat16, 1.0 / math.sqrt(128))
    return dict(q=q, k=k, v=v, do=do, causal=True)


def config3(batch=4, seq=2048, heads=16):
    """MHA with bias, padding mask and dropout, bf16, non-causal."""
    dt = torch.bfloat16
    q, k, v, do = make_qkv(batch, seq, seq, heads, heads, 64, dt)
    idx = torch.arange(seq)
    bias = (1.0 / (1.0 + (idx[:, None] - idx[None, :]).abs().float())).to(dt)[None, None].expand(batch, 1, seq, seq).contiguous()
    g = torch.Generator().manual_seed(4)
    lengths = torch.randint(seq // 2, seq + 1, (batch,), generator=g)
    mask = torch.zeros(batch, 1, seq, seq, dtype=dt)
    for b in range(batch):
        mask[b, :, :, int(lengths[b]):] = torch.finfo(dt).min
    return dict(q=q, k=k, v=v, do=do, causal=False, bias=bias, mask=mask, dropout_p=0.1, dropout_seed=42)


def config4(seq=32768, hq=64, hkv=8):
    """Long-context causal GQA, bf16."""
    q, k, v, do = make_qkv(1, seq, seq, hq, hkv, 128, torch.bfloat16, 1.0 / math.sqrt(128))
    return dict(q=q, k=k, v=v, do=do, causal=True)


def config5(batch=4, seq=8192, heads=8):
    """Large head dim MHA, fp16, causal."""
    q, k, v, do = make_qkv(batch, seq, seq, heads, heads, 256, torch.float16, 1.0 / 16)
    return dict(q=q, k=k, v=v, do=do, causal=True)


def attention_flops(B, Sq, Sk, Hq, D, causal):
    """Forward FLOPs: 4*B*Hq*Sq*Sk*D, halved when causal; backward = 2.5x, fwd+bwd = 3.5x."""
    f = 4.0 * B * Hq * Sq * Sk * D
    return f * 0.5 if causal else f
