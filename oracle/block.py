"""TEST INFRASTRUCTURE ONLY — CPU restatement of the reference's blockwise attention.

Follows the reference's pure-JAX FlashAttention-2 ("Platform.JAX"):
  * wrapper   jax_flash_attn2/flash_attention_jax/_flash_attention.py:98-133
              (BSHD -> BHSD, block sizes clamped to the sequence, q pre-scaled, transpose back)
  * forward   jax_flash_attn2/flash_attention_jax/_forward_jax.py:41-55, 84-158
              (block loops, bias add, masking, online softmax, lse = log(exp(lse-m)+l)+m,
               final o * exp(m - lse))
  * backward  jax_flash_attn2/flash_attention_jax/_backward_jax.py:62-66, 80-156
              (D = rowsum(dO*O), p = exp(s - L), dV += p^T dO, dP = dO v^T, dS = p*(dP - D),
               dQ += dS k, dK += dS^T q)
  * GQA head repeat and bias head rules  jax_flash_attn2/flash_attention.py:141-169, 337
  * bottom-right aligned causal mask and all-masked rows -> 0
              jax_flash_attn2/refrence_call.py:55-83,
              jax_flash_attn2/flash_attention_triton/_forward_triton.py:127-132, 440-441

Differences from the reference, on purpose:
  * arithmetic is float32 throughout (inputs are the 16-bit arrays up-cast), so this is the
    exact-arithmetic target both the reference and the CUDA kernels approximate;
    `reference_rounding=True` reproduces the reference's casts to the input dtype after every
    block (_forward_jax.py:132-139, _backward_jax.py:134-140) to show its own error envelope;
  * masks are additive (0 / -inf / finfo.min), the form the CUDA path takes; causal is a flag;
  * dropout is FlashAttention-2 dropout (weights dropped after the softmax statistics, scaled by
    1/(1-p)) with the Philox bits of oracle/philox.py, which is what the Triton path of the
    reference does (_forward_triton.py:140-143, 435-436); the JAX path's score dropout
    (_forward_jax.py:109-115) is unreachable from the public class and is not restated;
  * gradients are returned for the un-scaled q (the Triton path's convention).

PARITY PIN: the reference ships no tests or golden vectors for this path and cannot be imported
where this build runs (no jax). tests/golden/make_golden.py executes the reference's own
_fwd_flash_attn / _bwd_flash_attn source on a small numpy stand-in for the jax calls they use and
stores the results; tests/test_oracle.py checks this restatement against those vectors.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this module.
"""
from __future__ import annotations

import math
import typing as tp

import torch

from . import philox


def _expand_term(x: tp.Optional[torch.Tensor], b: int, h: int, sq: int, sk: int) -> tp.Optional[torch.Tensor]:
    if x is None:
        return None
    return x.to(torch.float32).expand(b, h, sq, sk)


def _expand_bias(x: tp.Optional[torch.Tensor], b: int, h: int, sq: int, sk: int) -> tp.Optional[torch.Tensor]:
    """Bias head rules of jax_flash_attn2/flash_attention.py:151-169: 1 or Hq heads broadcast,
    Hkv heads are repeated per group ("b h q k -> b (h r) q k")."""
    if x is not None and x.shape[1] not in (1, h):
        x = x.repeat_interleave(h // x.shape[1], dim=1)
    return _expand_term(x, b, h, sq, sk)


def _visible(i0: int, bq: int, j0: int, bk: int, off: int) -> torch.Tensor:
    """Causal visibility of a (bq x bk) block: key j visible from query i iff j <= i + off."""
    qi = torch.arange(i0, i0 + bq)[:, None]
    kj = torch.arange(j0, j0 + bk)[None, :]
    return kj <= qi + off


class BlockAttention:
    """Blockwise attention forward / backward on CPU tensors in [B, S, H, D] layout."""

    def __init__(self, blocksize_q: int = 128, blocksize_k: int = 128, reference_rounding: bool = False):
        self.bq = blocksize_q
        self.bk = blocksize_k
        self.ref_round = reference_rounding

    # -------------------------------------------------------------------------------------
    def forward(self, q, k, v, bias=None, mask=None, softmax_scale=None, causal=False,
                dropout_p=0.0, dropout_seed=0, batch_offset=0, head_offset=0, heads_q_global=None):
        """Returns (out [B,Sq,Hq,D] in q.dtype, lse [B,Hq,Sq] float32 natural log)."""
        dt = q.dtype
        B, Sq, Hq, D = q.shape
        Sk, Hkv = k.shape[1], k.shape[2]
        G = Hq // Hkv
        scale = 1.0 / math.sqrt(D) if softmax_scale is None else softmax_scale
        rd = (lambda x: x.to(dt).to(torch.float32)) if self.ref_round else (lambda x: x)
        qf = rd(q.to(torch.float32).permute(0, 2, 1, 3) * scale)
        kf = k.to(torch.float32).permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
        vf = v.to(torch.float32).permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
        bias_f = _expand_bias(bias, B, Hq, Sq, Sk)
        mask_f = _expand_term(mask, B, Hq, Sq, Sk)
        keep = None
        if dropout_p > 0:
            keep = torch.from_numpy(
                philox.keep_mask(dropout_seed, dropout_p, B, Hq, Sq, Sk, batch_offset, head_offset, heads_q_global)
            )
        inv_keep = 1.0 / (1.0 - dropout_p) if dropout_p > 0 else 1.0
        off = Sk - Sq
        bq, bk = min(self.bq, Sq), min(self.bk, Sk)
        o = torch.zeros(B, Hq, Sq, D, dtype=torch.float32)
        lse = torch.full((B, Hq, Sq), -math.inf, dtype=torch.float32)
        for i0 in range(0, Sq, bq):
            i1 = min(i0 + bq, Sq)
            q_i = qf[:, :, i0:i1]
            o_i = torch.zeros(B, Hq, i1 - i0, D)
            m_i = torch.full((B, Hq, i1 - i0), -math.inf)
            l_i = torch.zeros(B, Hq, i1 - i0)
            for j0 in range(0, Sk, bk):
                j1 = min(j0 + bk, Sk)
                if causal and j0 > (i1 - 1) + off:
                    break  # block entirely above the diagonal (_forward_jax.py:141)
                s = rd(q_i @ kf[:, :, j0:j1].transpose(-1, -2))
                if bias_f is not None:
                    s = s + bias_f[:, :, i0:i1, j0:j1]
                if mask_f is not None:
                    s = s + mask_f[:, :, i0:i1, j0:j1]
                if causal:
                    s = s.masked_fill(~_visible(i0, i1 - i0, j0, j1 - j0, off), -math.inf)
                m_new = torch.maximum(m_i, s.max(dim=-1).values)
                m_safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
                p = rd(torch.exp(s - m_safe[..., None]))
                alpha = torch.exp(torch.where(torch.isinf(m_i), torch.full_like(m_i, -math.inf), m_i - m_safe))
                l_i = l_i * alpha + p.sum(-1)
                if keep is not None:
                    p = p * keep[:, :, i0:i1, j0:j1]
                o_i = rd(o_i * alpha[..., None] + p @ vf[:, :, j0:j1])
                m_i = m_new
            has = l_i > 0
            l_safe = torch.where(has, l_i, torch.ones_like(l_i))
            o[:, :, i0:i1] = torch.where(has[..., None], o_i * (inv_keep / l_safe)[..., None], torch.zeros_like(o_i))
            lse[:, :, i0:i1] = torch.where(has, m_i + torch.log(l_safe), torch.full_like(l_i, -math.inf))
        return o.permute(0, 2, 1, 3).to(dt), lse

    # -------------------------------------------------------------------------------------
    def backward(self, dO, q, k, v, o, lse, bias=None, mask=None, softmax_scale=None, causal=False,
                 dropout_p=0.0, dropout_seed=0, batch_offset=0, head_offset=0, heads_q_global=None,
                 out_dtype=None, bias_grad=False):
        """Returns (dq, dk, dv) in `out_dtype` (default: the input dtype); dk / dv are summed over
        the query heads of each key/value head. With `bias_grad` a fourth result is the gradient of
        the bias (float32, the bias's shape): dS summed over the batch elements and heads that share
        a bias entry. The reference computes no such gradient; dS is the quantity of
        _backward_jax.py:121 (`dS = p * (dP - D)`), which is d loss / d (scores + bias)."""
        dt = q.dtype if out_dtype is None else out_dtype
        B, Sq, Hq, D = q.shape
        Sk, Hkv = k.shape[1], k.shape[2]
        G = Hq // Hkv
        scale = 1.0 / math.sqrt(D) if softmax_scale is None else softmax_scale
        rd = (lambda x: x.to(q.dtype).to(torch.float32)) if self.ref_round else (lambda x: x)
        qf = q.to(torch.float32).permute(0, 2, 1, 3)
        kf = k.to(torch.float32).permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
        vf = v.to(torch.float32).permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
        of = o.to(torch.float32).permute(0, 2, 1, 3)
        dof = dO.to(torch.float32).permute(0, 2, 1, 3)
        bias_f = _expand_bias(bias, B, Hq, Sq, Sk)
        mask_f = _expand_term(mask, B, Hq, Sq, Sk)
        dbias = torch.zeros(B, Hq, Sq, Sk) if bias_grad else None
        keep = None
        if dropout_p > 0:
            keep = torch.from_numpy(
                philox.keep_mask(dropout_seed, dropout_p, B, Hq, Sq, Sk, batch_offset, head_offset, heads_q_global)
            )
        inv_keep = 1.0 / (1.0 - dropout_p) if dropout_p > 0 else 1.0
        off = Sk - Sq
        bq, bk = min(self.bq, Sq), min(self.bk, Sk)
        delta = (dof * of).sum(-1)                       # _backward_jax.py:62
        dq = torch.zeros_like(qf)
        dk = torch.zeros_like(kf)
        dv = torch.zeros_like(vf)
        lse_safe = torch.where(torch.isinf(lse), torch.full_like(lse, math.inf), lse)
        for j0 in range(0, Sk, bk):
            j1 = min(j0 + bk, Sk)
            k_j, v_j = kf[:, :, j0:j1], vf[:, :, j0:j1]
            for i0 in range(0, Sq, bq):
                i1 = min(i0 + bq, Sq)
                if causal and j0 > (i1 - 1) + off:
                    continue
                s = (qf[:, :, i0:i1] * scale) @ k_j.transpose(-1, -2)
                if bias_f is not None:
                    s = s + bias_f[:, :, i0:i1, j0:j1]
                if mask_f is not None:
                    s = s + mask_f[:, :, i0:i1, j0:j1]
                if causal:
                    s = s.masked_fill(~_visible(i0, i1 - i0, j0, j1 - j0, off), -math.inf)
                p = torch.exp(s - lse_safe[:, :, i0:i1, None])
                dp = dof[:, :, i0:i1] @ v_j.transpose(-1, -2)
                if keep is not None:
                    kp = keep[:, :, i0:i1, j0:j1] * inv_keep
                    p_drop, dp = p * kp, dp * kp
                else:
                    p_drop = p
                dv[:, :, j0:j1] = rd(dv[:, :, j0:j1] + p_drop.transpose(-1, -2) @ dof[:, :, i0:i1])
                ds = p * (dp - delta[:, :, i0:i1, None])
                if dbias is not None:
                    dbias[:, :, i0:i1, j0:j1] = ds
                dq[:, :, i0:i1] = rd(dq[:, :, i0:i1] + (ds @ k_j) * scale)
                dk[:, :, j0:j1] = rd(dk[:, :, j0:j1] + (ds.transpose(-1, -2) @ qf[:, :, i0:i1]) * scale)
        dk = dk.reshape(B, Hkv, G, Sk, D).sum(2)
        dv = dv.reshape(B, Hkv, G, Sk, D).sum(2)
        grads = (dq.permute(0, 2, 1, 3).to(dt), dk.permute(0, 2, 1, 3).to(dt), dv.permute(0, 2, 1, 3).to(dt))
        if dbias is None:
            return grads
        bb, bh = bias.shape[0], bias.shape[1]
        if bh not in (1, Hq):                            # one bias head per key/value head
            dbias = dbias.reshape(B, bh, Hq // bh, Sq, Sk).sum(2)
        elif bh == 1:
            dbias = dbias.sum(1, keepdim=True)
        if bb == 1:
            dbias = dbias.sum(0, keepdim=True)
        return grads + (dbias,)
