"""Differentiable attention op over the CUDA kernels.

Mirrors the structure of the reference's `flash_attention_call` custom_vjp
(jax_flash_attn2/flash_attention_triton/_flash_attention.py:27-157): the forward saves
(q, k, v, bias, attention_mask, out, lse, dropout_seed); the backward returns gradients for
q, k and v (mask and seed get none). One addition: a bias that requires a gradient gets one, where
the reference returns None (:88). torch.autograd.Function plays the part of
jax.custom_vjp because JAX is not available where this library is built and tested.
"""
from __future__ import annotations

import typing as tp

import torch

from ._kernel_calls import (
    bwd_attention_kernel_call,
    dropout_bits_buffer,
    fwd_attention_kernel_call,
    normalise_attention_mask,
    seqlens_from_padding_mask,
)


class _FlashAttentionCall(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, attention_mask, bias, softmax_scale, dropout_prob, causal, dropout_seed, shard):
        # one more residual than the reference keeps: the record of the dropout keep bits, so that
        # the backward reads them instead of running Philox again (None without dropout)
        bits = dropout_bits_buffer(q, k, dropout_prob)
        out, lse = fwd_attention_kernel_call(
            q, k, v, attention_mask, bias, softmax_scale, dropout_prob, causal, dropout_seed,
            dropout_bits=bits, **shard
        )   # `shard` also carries the per-batch lengths, when there are any
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.dropout_bits = bits
        ctx.extras = (attention_mask, bias, softmax_scale, dropout_prob, causal, dropout_seed, shard)
        ctx.bias_grad = bias is not None and bias.requires_grad
        return out

    @staticmethod
    def backward(ctx, dO):
        q, k, v, out, lse = ctx.saved_tensors
        attention_mask, bias, softmax_scale, dropout_prob, causal, dropout_seed, shard = ctx.extras
        grads = bwd_attention_kernel_call(
            dO, q, k, v, bias, attention_mask, out, lse, dropout_prob, causal, softmax_scale, dropout_seed,
            bias_grad=ctx.bias_grad, dropout_bits=ctx.dropout_bits, **shard
        )
        dbias = grads[3].to(bias.dtype) if ctx.bias_grad else None
        return grads[0], grads[1], grads[2], None, dbias, None, None, None, None, None


def flash_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    attention_mask: tp.Optional[torch.Tensor] = None,
    bias: tp.Optional[torch.Tensor] = None,
    softmax_scale: tp.Optional[float] = None,
    dropout_prob: float = 0.0,
    causal: bool = False,
    dropout_seed: tp.Optional[int] = None,
    varlen_mode: bool = True,
    *,
    batch_offset: int = 0,
    head_offset: int = 0,
    heads_q_global: tp.Optional[int] = None,
) -> torch.Tensor:
    """Same signature as the reference's `triton_flash_attention`
    (flash_attention_triton/_flash_attention.py:125-157).

    A 2-D [B, S] `attention_mask` is a padding mask. With `varlen_mode=True` (the default, as in
    the reference) it is read the way the reference's varlen mode reads it: row b has
    `sum(mask[b])` real tokens and they come first; the kernels then work on per-batch lengths and
    skip the padding (no packing, no mask tensor). Unlike the reference this also holds for
    batch 1 (where the reference ignores the mask, _forward_triton.py:475) and a bias may be given
    as well. With `varlen_mode=False` the mask may have its real tokens anywhere: keys are masked
    through an additive term and padded rows are zeroed afterwards.
    The three keyword-only arguments place a shard inside the unsharded problem so that dropout
    draws the same bits on every partitioning."""
    sq, sk = q.shape[1], k.shape[1]
    shard = dict(batch_offset=batch_offset, head_offset=head_offset, heads_q_global=heads_q_global)
    if attention_mask is not None and attention_mask.dim() == 2 and varlen_mode:
        shard["seqlens"] = seqlens_from_padding_mask(attention_mask, sq, sk)
        attention_mask = None
    add_mask, row_keep = normalise_attention_mask(attention_mask, q.dtype, sq, sk)
    out = _FlashAttentionCall.apply(
        q, k, v, add_mask, bias, softmax_scale, float(dropout_prob), bool(causal), dropout_seed, shard
    )
    if row_keep is not None:
        out = out * row_keep[:, :, None, None].to(out.dtype)
    return out
