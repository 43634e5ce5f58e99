"""Host launchers of the CUDA kernels, on torch CUDA tensors.

These two functions stand where the reference has `_fwd_attention_kernel_call`
(jax_flash_attn2/flash_attention_triton/_forward_triton.py:462-592) and
`_bwd_attention_kernel_call` (jax_flash_attn2/flash_attention_triton/_backward_triton.py:948-1173):
same argument meaning, same checks, same error behaviour (assertion / ValueError before any
launch). torch is used for device memory and streams only; all arithmetic happens in
libfa2_b200.so. There is no fallback: without the library or without a GPU these raise.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import typing as tp

import torch

from . import _capi

_DTYPE_CODE = {torch.float16: _capi.FA2_FP16, torch.bfloat16: _capi.FA2_BF16, torch.float32: _capi.FA2_FP32}


_raw_stream_fn = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _launch(fn, params, device: torch.device) -> None:
    """Calls one C-ABI entry point on torch's current stream of `device`. The device is only
    switched when it is not the current one, and the stream handle is taken through the raw
    accessor when torch has it: for small problems the host side of a call is what one waits for."""
    index = device.index
    current = torch.cuda.current_device()
    if index is None:
        index = current
    if index != current:
        with torch.cuda.device(index):
            _launch(fn, params, device)
        return
    if _raw_stream_fn is not None:
        stream = _raw_stream_fn(index)
    else:
        stream = torch.cuda.current_stream(index).cuda_stream
    _capi.check(fn(C.byref(params), C.c_void_p(stream)))


def _strides(x: torch.Tensor) -> _capi.Strides:
    """(batch, sequence, head) element strides of a [B, S, H, D] tensor."""
    return _capi.Strides(x.stride(0), x.stride(1), x.stride(2))


def _unit_last(x: torch.Tensor) -> torch.Tensor:
    return x if x.stride(-1) == 1 else x.contiguous()


def _score_term(x: tp.Optional[torch.Tensor], batch: int, heads: int, sq: int, sk: int, name: str,
                heads_kv: tp.Optional[int] = None):
    """Broadcast rules of calc_bias_strides (flash_attention_triton/_utils.py:151-193): batch in
    {1, B}, heads in {1, Hq}, the two sequence dims equal to (Sq, Sk); additionally the query dim
    may be 1 (a key-padding term), and a term with one head per key/value head (`heads_kv`) is
    indexed by query head // group size inside the kernels, without the repeat of the reference
    (flash_attention.py:161-164). Returns (ScoreTerm, tensor kept alive)."""
    term = _capi.ScoreTerm()
    if x is None:
        return term, None
    if x.dim() != 4:
        raise ValueError(f"{name} must have four dimensions, got shape {tuple(x.shape)}")
    if x.dtype not in _DTYPE_CODE:
        raise ValueError(f"{name} has unsupported dtype {x.dtype}")
    bb, bh, bq, bk = x.shape
    if bb not in (1, batch):
        raise ValueError(f"{name} batch size must be {batch} or 1, got {bb}")
    per_kv_head = heads_kv is not None and bh == heads_kv and bh not in (1, heads)
    if bh not in (1, heads) and not per_kv_head:
        raise ValueError(f"{name} heads must be {heads} or 1, got {bh}")
    if bq not in (1, sq) or bk != sk:
        raise ValueError(f"{name} sequence dims must be ({sq}, {sk}), got ({bq}, {bk})")
    x = _unit_last(x)
    term.ptr = x.data_ptr()
    term.dtype = _DTYPE_CODE[x.dtype]
    term.head_div = heads // heads_kv if per_kv_head else 1
    term.stride_b = 0 if bb == 1 else x.stride(0)
    term.stride_h = 0 if bh == 1 else x.stride(1)
    term.stride_q = 0 if bq == 1 else x.stride(2)
    return term, x


def normalise_attention_mask(
    attention_mask: tp.Optional[torch.Tensor], dtype: torch.dtype, sq: int, sk: int
) -> tp.Tuple[tp.Optional[torch.Tensor], tp.Optional[torch.Tensor]]:
    """Turns the accepted mask forms into an additive term.

    * 4-D floating mask [B, 1|Hq, Sq, Sk] (0 keeps, finfo.min / -inf drops): used as is.
    * 4-D bool / integer mask (non-zero keeps): converted to 0 / -inf.
    * 2-D [B, S] padding mask (non-zero = real token) with tokens anywhere in the row: becomes a
      key-padding term [B,1,1,Sk]; the second return value is the [B, Sq] row mask with which the
      caller zeroes the padded query rows. (The reference's own reading of a 2-D mask, real tokens
      first, is served by `seqlens_from_padding_mask` and the kernels' per-batch lengths.)
    """
    if attention_mask is None:
        return None, None
    m = attention_mask
    if m.dim() == 2:
        if sq != sk:
            raise AssertionError("Attention mask is not supported with QSeq != KSeq")
        keep = m != 0
        add = torch.zeros(m.shape, dtype=torch.float32, device=m.device)
        add.masked_fill_(~keep, float("-inf"))
        return add[:, None, None, :].contiguous(), keep
    if m.dim() != 4:
        raise ValueError(f"attention_mask must be 2-D or 4-D, got shape {tuple(m.shape)}")
    if m.is_floating_point():
        return m, None
    add = torch.zeros(m.shape, dtype=dtype, device=m.device)
    add.masked_fill_(m == 0, float("-inf"))
    return add, None


def seqlens_from_padding_mask(attention_mask: torch.Tensor, sq: int, sk: int) -> torch.Tensor:
    """Per-batch lengths of a 2-D [B, S] padding mask, the way the reference's varlen mode reads
    it (_forward_triton.py:500-510; _utils.py:211-221): the number of non-zero entries of a row
    is the length of that sequence and its real tokens come first. Computed on the device, no
    host synchronisation."""
    if attention_mask.dim() != 2:
        raise ValueError(f"a padding mask must be 2-D, got shape {tuple(attention_mask.shape)}")
    if sq != sk:
        raise AssertionError("Attention mask is not supported with QSeq != KSeq")
    if attention_mask.shape[1] != sq:
        raise ValueError(f"padding mask must be [batch, {sq}], got {tuple(attention_mask.shape)}")
    return (attention_mask != 0).sum(dim=1, dtype=torch.int32).contiguous()


def _seqlens_ptr(seqlens: tp.Optional[torch.Tensor], q: torch.Tensor, sk: int):
    if seqlens is None:
        return None, None
    batch, sq = q.shape[0], q.shape[1]
    if sq != sk:
        raise AssertionError("Attention mask is not supported with QSeq != KSeq")
    if seqlens.dtype != torch.int32 or seqlens.dim() != 1 or seqlens.shape[0] != batch:
        raise ValueError(f"seqlens must be int32 of shape [{batch}], got {seqlens.dtype} {tuple(seqlens.shape)}")
    if seqlens.device != q.device:
        raise ValueError("seqlens must live on the device of q")
    seqlens = seqlens.contiguous()
    return seqlens.data_ptr(), seqlens


def _seed_ptr(dropout_seed, q: torch.Tensor):
    """A seed given as a one-element int64 / uint64 CUDA tensor stays on the device: the kernels
    read it there (no host synchronisation). Returns (device pointer or None, tensor kept alive)."""
    if not isinstance(dropout_seed, torch.Tensor):
        return None, None
    if dropout_seed.numel() != 1 or dropout_seed.dtype not in (torch.int64, torch.uint64):
        raise ValueError("a tensor dropout_seed must hold one int64 / uint64 value")
    if dropout_seed.device != q.device:
        raise ValueError("a tensor dropout_seed must live on the device of q")
    dropout_seed = dropout_seed.contiguous()
    return dropout_seed.data_ptr(), dropout_seed


def _offsets_ptr(offsets_dev, q: torch.Tensor):
    """(batch_offset, head_offset) as an int32 [2] CUDA tensor: read by the kernels on the device
    in place of the two integer arguments. Returns (device pointer or None, tensor kept alive)."""
    if offsets_dev is None:
        return None, None
    if offsets_dev.dtype != torch.int32 or offsets_dev.numel() != 2:
        raise ValueError("offsets_dev must hold two int32 values (batch offset, head offset)")
    if offsets_dev.device != q.device:
        raise ValueError("offsets_dev must live on the device of q")
    offsets_dev = offsets_dev.contiguous()
    return offsets_dev.data_ptr(), offsets_dev


def dropout_bits_buffer(q: torch.Tensor, k: torch.Tensor, dropout_prob: float,
                        max_bytes: int = 1 << 30) -> tp.Optional[torch.Tensor]:
    """An uninitialised buffer for the record of dropout keep bits of a (q, k) problem: pass it as
    `dropout_bits` to the forward call, which fills it, and to the backward call of the same
    problem, which then reads the bits instead of drawing them again. None without dropout, or
    when the record (Sq * Sk / 8 bytes per batch element and head, rounded up to whole tiles)
    would exceed `max_bytes`."""
    if not dropout_prob > 0.0:
        return None
    batch, sq, hq, _ = q.shape
    nbytes = batch * hq * ((sq + 127) // 128) * ((k.shape[1] + 127) // 128) * 2048
    if nbytes > max_bytes:
        return None
    return torch.empty((nbytes // 4,), dtype=torch.int32, device=q.device)


def _dropout_bits_ptr(dropout_bits, q: torch.Tensor):
    if dropout_bits is None:
        return None, 0
    if dropout_bits.dtype != torch.int32 or dropout_bits.device != q.device or not dropout_bits.is_contiguous():
        raise ValueError("dropout_bits must be a contiguous int32 tensor on the device of q (see dropout_bits_buffer)")
    return dropout_bits.data_ptr(), dropout_bits.numel() * 4


def _problem(q, k, softmax_scale, dropout_prob, causal, dropout_seed, batch_offset, head_offset, heads_q_global):
    batch, sq, hq, d = q.shape
    _, sk, hkv, _ = k.shape
    p = _capi.Problem()
    p.batch, p.seqlen_q, p.seqlen_k = batch, sq, sk
    p.heads_q, p.heads_kv, p.head_dim = hq, hkv, d
    p.dtype = _DTYPE_CODE[q.dtype]
    p.causal = int(bool(causal))
    p.softmax_scale = float(1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale)
    p.dropout_p = float(dropout_prob)
    if isinstance(dropout_seed, torch.Tensor):
        p.dropout_seed = 0           # read on the device, see _seed_ptr
    else:
        p.dropout_seed = int(0 if dropout_seed is None else dropout_seed) & 0xFFFFFFFFFFFFFFFF
    p.batch_offset = int(batch_offset)
    p.head_offset = int(head_offset)
    p.heads_q_global = int(hq if heads_q_global is None else heads_q_global)
    return p


def _check_qkv(q, k, v):
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("fa2_b200 runs on CUDA tensors only; there is no CPU path")
    batch, sq, hq, d = q.shape
    _, sk, hkv, _ = k.shape
    expected = (batch, sk, hkv, d)
    assert tuple(k.shape) == expected, f"key shape is {tuple(k.shape)} and we excepted it to be like {expected}"
    assert tuple(v.shape) == expected, f"value shape is {tuple(v.shape)} and we excepted it to be like {expected}"
    assert hq % hkv == 0, f"nheads_q = {hq} is not divisible by nheads_kv = {hkv}"
    assert q.dtype == k.dtype == v.dtype, "All tensors must have the same type"
    assert q.dtype in (torch.float16, torch.bfloat16), "Only support fp16 and bf16"


def fwd_attention_kernel_call(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    attention_mask: tp.Optional[torch.Tensor] = None,
    bias: tp.Optional[torch.Tensor] = None,
    softmax_scale: tp.Optional[float] = None,
    dropout_prob: float = 0.0,
    causal: bool = False,
    dropout_seed: tp.Optional[int] = None,
    *,
    batch_offset: int = 0,
    head_offset: int = 0,
    heads_q_global: tp.Optional[int] = None,
    seqlens: tp.Optional[torch.Tensor] = None,
    split_kv: bool = True,
    offsets_dev: tp.Optional[torch.Tensor] = None,
    dropout_bits: tp.Optional[torch.Tensor] = None,
) -> tp.Tuple[torch.Tensor, torch.Tensor]:
    """Forward launch. q [B,Sq,Hq,D]; k, v [B,Sk,Hkv,D]; `attention_mask` here is already an
    additive 4-D term (see normalise_attention_mask); `seqlens` (int32 [B], device) gives every
    batch element its own length, the reference's varlen mode without packing; `split_kv=False`
    withholds the scratch with which the library splits low-occupancy problems along the key
    sequence (same result, computed by fewer SMs); `offsets_dev` (int32 [2], device) carries
    (batch_offset, head_offset) as a device operand; `dropout_bits` (from `dropout_bits_buffer`)
    receives the record of the keep bits for the backward call. Returns
    (out [B,Sq,Hq,D] in q.dtype, lse [B,Hq,ceil(Sq/128)*128] float32, natural log; columns >= Sq
    are not written)."""
    _check_qkv(q, k, v)
    lib = _capi.load()
    q, k, v = _unit_last(q), _unit_last(k), _unit_last(v)
    batch, sq, hq, d = q.shape
    sk = k.shape[1]
    out = torch.empty((batch, sq, hq, d), dtype=q.dtype, device=q.device)
    sq_rounded = (sq + 127) // 128 * 128
    lse = torch.empty((batch, hq, sq_rounded), dtype=torch.float32, device=q.device)

    a = _capi.FwdParams()
    a.p = _problem(q, k, softmax_scale, dropout_prob, causal, dropout_seed, batch_offset, head_offset, heads_q_global)
    a.q, a.q_strides = q.data_ptr(), _strides(q)
    a.k, a.k_strides = k.data_ptr(), _strides(k)
    a.v, a.v_strides = v.data_ptr(), _strides(v)
    a.o, a.o_strides = out.data_ptr(), _strides(out)
    a.lse, a.lse_stride_b, a.lse_stride_h = lse.data_ptr(), lse.stride(0), lse.stride(1)
    a.bias, _keep_b = _score_term(bias, batch, hq, sq, sk, "bias", k.shape[2])
    a.mask, _keep_m = _score_term(attention_mask, batch, hq, sq, sk, "attention_mask")
    a.seqlens, _keep_s = _seqlens_ptr(seqlens, q, sk)
    a.dropout_seed_dev, _keep_d = _seed_ptr(dropout_seed, q)
    a.offsets_dev, _keep_f = _offsets_ptr(offsets_dev, q)
    a.dropout_bits, a.dropout_bits_bytes = _dropout_bits_ptr(dropout_bits, q)
    # low-occupancy problems (decode steps) are split along the key sequence if scratch is offered
    nbytes = lib.fa2_fwd_workspace_bytes(C.byref(a.p)) if split_kv else 0
    if nbytes:
        _keep_w = torch.empty((nbytes,), dtype=torch.uint8, device=q.device)
        a.workspace, a.workspace_bytes = _keep_w.data_ptr(), nbytes
    _launch(lib.fa2_fwd, a, q.device)
    return out, lse


def bwd_attention_kernel_call(
    dO: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    bias: tp.Optional[torch.Tensor],
    attention_mask: tp.Optional[torch.Tensor],
    o: torch.Tensor,
    M: torch.Tensor,
    dropout_prob: float,
    causal: bool,
    softmax_scale: tp.Optional[float],
    dropout_seed: tp.Optional[int],
    *,
    batch_offset: int = 0,
    head_offset: int = 0,
    heads_q_global: tp.Optional[int] = None,
    seqlens: tp.Optional[torch.Tensor] = None,
    offsets_dev: tp.Optional[torch.Tensor] = None,
    bias_grad: bool = False,
    dropout_bits: tp.Optional[torch.Tensor] = None,
    deterministic: tp.Optional[bool] = None,
):
    """Backward launch; `M` is the lse returned by the forward. Returns (dq, dk, dv) in the input
    dtype; dk and dv are already reduced over the query heads of each key/value head. With
    `bias_grad=True` a fourth result is the gradient of `bias` in float32 and in the bias's own
    shape (summed over the batch elements / query heads that share an entry); the reference has no
    bias cotangent (flash_attention_triton/_flash_attention.py:88). `deterministic=True` makes dq
    bit-reproducible from call to call like the reference's (its dq program adds the key tiles in a
    loop, _backward_triton.py:438-516) at the price of a slower backward; the default (None) reads
    the environment variable FA2_B200_DETERMINISTIC (unset or "0": off)."""
    _check_qkv(q, k, v)
    lib = _capi.load()
    if deterministic is None:
        deterministic = os.environ.get("FA2_B200_DETERMINISTIC", "0") not in ("", "0")
    q, k, v, o, dO = map(_unit_last, (q, k, v, o, dO))
    batch, sq, hq, d = q.shape
    sk = k.shape[1]
    assert tuple(dO.shape) == tuple(q.shape) and tuple(o.shape) == tuple(q.shape)
    assert dO.dtype == q.dtype and o.dtype == q.dtype
    dq = torch.empty_like(q, memory_format=torch.contiguous_format)
    dk = torch.empty_like(k, memory_format=torch.contiguous_format)
    dv = torch.empty_like(v, memory_format=torch.contiguous_format)

    a = _capi.BwdParams()
    a.p = _problem(q, k, softmax_scale, dropout_prob, causal, dropout_seed, batch_offset, head_offset, heads_q_global)
    nbytes = lib.fa2_bwd_workspace_bytes(C.byref(a.p))
    if nbytes == 0:
        _capi.check(_capi.FA2_ERR_INVALID_ARG)
    workspace = torch.empty((nbytes,), dtype=torch.uint8, device=q.device)
    a.q, a.q_strides = q.data_ptr(), _strides(q)
    a.k, a.k_strides = k.data_ptr(), _strides(k)
    a.v, a.v_strides = v.data_ptr(), _strides(v)
    a.o, a.o_strides = o.data_ptr(), _strides(o)
    a.d_o, a.do_strides = dO.data_ptr(), _strides(dO)
    a.lse, a.lse_stride_b, a.lse_stride_h = M.data_ptr(), M.stride(0), M.stride(1)
    a.bias, _keep_b = _score_term(bias, batch, hq, sq, sk, "bias", k.shape[2])
    a.mask, _keep_m = _score_term(attention_mask, batch, hq, sq, sk, "attention_mask")
    dbias = None
    if bias_grad:
        if bias is None or bias.shape[2] != sq:
            raise ValueError("bias_grad needs a bias with a full query dimension")
        dbias = torch.empty(tuple(bias.shape), dtype=torch.float32, device=q.device)
        a.dbias.ptr, a.dbias.batch, a.dbias.heads = dbias.data_ptr(), bias.shape[0], bias.shape[1]
    a.dq, a.dq_strides = dq.data_ptr(), _strides(dq)
    a.dk, a.dk_strides = dk.data_ptr(), _strides(dk)
    a.dv, a.dv_strides = dv.data_ptr(), _strides(dv)
    a.workspace, a.workspace_bytes = workspace.data_ptr(), nbytes
    a.seqlens, _keep_s = _seqlens_ptr(seqlens, q, sk)
    a.dropout_seed_dev, _keep_d = _seed_ptr(dropout_seed, q)
    a.offsets_dev, _keep_f = _offsets_ptr(offsets_dev, q)
    a.dropout_bits, a.dropout_bits_bytes = _dropout_bits_ptr(dropout_bits, q)
    a.deterministic = int(bool(deterministic))
    _launch(lib.fa2_bwd, a, q.device)
    if bias_grad:
        return dq, dk, dv, dbias
    return dq, dk, dv


def device_status() -> int:
    """Reads (and clears) the status word a kernel sets when one of its bounded waits ran out."""
    lib = _capi.load()
    return int(lib.fa2_debug_device_status(C.c_void_p(torch.cuda.current_stream().cuda_stream)))
