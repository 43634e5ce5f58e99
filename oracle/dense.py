"""TEST INFRASTRUCTURE ONLY — dense float64 attention with autograd gradients.

An independent second oracle: softmax(scale q k^T + bias + mask [+ causal]) v computed densely
in float64, gradients by torch autograd. Semantics follow the reference's dense helper
jax_flash_attn2/refrence_call.py:23-104 (GQA repeat, bottom-right aligned causal mask
`col > row + sk - sq` masked, rows without a visible key give 0) restricted to the arguments the
public class can reach (no window, no softcap). Used to check oracle/block.py.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this module.
"""
from __future__ import annotations

import math

import torch

from . import philox


def attention(q, k, v, bias=None, mask=None, softmax_scale=None, causal=False, dropout_p=0.0,
              dropout_seed=0, batch_offset=0, head_offset=0, heads_q_global=None):
    """q [B,Sq,Hq,D], k/v [B,Sk,Hkv,D] (any float dtype). Returns (out float64 [B,Sq,Hq,D],
    lse float64 [B,Hq,Sq]); differentiable w.r.t. q, k, v."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    G = Hq // Hkv
    scale = 1.0 / math.sqrt(D) if softmax_scale is None else softmax_scale
    qd = q.to(torch.float64).permute(0, 2, 1, 3)
    kd = k.to(torch.float64).permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    vd = v.to(torch.float64).permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    s = (qd @ kd.transpose(-1, -2)) * scale
    if bias is not None:
        bias = bias.to(torch.float64)
        if bias.shape[1] not in (1, Hq):     # one bias head per key/value head (flash_attention.py:161-164)
            bias = bias.repeat_interleave(Hq // bias.shape[1], dim=1)
        s = s + bias
    if mask is not None:
        s = s + mask.to(torch.float64)
    if causal:
        qi = torch.arange(Sq)[:, None]
        kj = torch.arange(Sk)[None, :]
        s = s.masked_fill(kj > qi + (Sk - Sq), -math.inf)
    lse = torch.logsumexp(s, dim=-1)
    dead = torch.isinf(lse) & (lse < 0)
    p = torch.exp(s - torch.where(dead, torch.zeros_like(lse), lse)[..., None])
    p = torch.where(dead[..., None], torch.zeros_like(p), p)
    if dropout_p > 0:
        keep = torch.from_numpy(
            philox.keep_mask(dropout_seed, dropout_p, B, Hq, Sq, Sk, batch_offset, head_offset, heads_q_global)
        )
        p = p * keep / (1.0 - dropout_p)
    out = p @ vd
    return out.permute(0, 2, 1, 3), lse


def attention_grads(dO, q, k, v, bias_grad=False, **kw):
    """(dq, dk, dv) in float64 for the cotangent dO; with `bias_grad` also the gradient of
    kw["bias"], in the bias's own shape."""
    q_, k_, v_ = (x.detach().to(torch.float64).requires_grad_(True) for x in (q, k, v))
    wrt = (q_, k_, v_)
    if bias_grad:
        kw = dict(kw, bias=kw["bias"].detach().to(torch.float64).requires_grad_(True))
        wrt = wrt + (kw["bias"],)
    out, _ = attention(q_, k_, v_, **kw)
    return torch.autograd.grad(out, wrt, dO.to(torch.float64))
