"""JAX side of the XLA FFI binding: drop-in bodies for the reference's two launch functions.

`_fwd_attention_kernel_call` / `_bwd_attention_kernel_call` below take the place of the functions
of the same name in jax_flash_attn2/flash_attention_triton/_forward_triton.py:462-592 and
_backward_triton.py:948-1173; `flash_attention_call` repeats the reference's custom_vjp
(flash_attention_triton/_flash_attention.py:27-122) over them, and `sharded_flash_attention`
spreads a call over a (batch, kv head) mesh with shard_map.

NOT RUN WHERE THIS LIBRARY IS BUILT AND TESTED: JAX is not installed there. Importing this module
without JAX raises ImportError at once; nothing else in the package imports it. The call sequence
it issues is the one the tested torch / ctypes layer issues (jax_flash_attn2/_kernel_calls.py).
"""
from __future__ import annotations

import ctypes
import functools
import math
import os
import typing as tp

import jax  # noqa: E402  (ImportError here means: this optional module cannot be used)
import jax.numpy as jnp
import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
FA2_ABI_VERSION = 3000      # of the include/fa2_b200.h this module was written against
_SCRATCH_SLACK = 128        # kScratchSlack of fa2_xla_ffi.cc: room to align a scratch result
_core = ctypes.CDLL(os.path.join(_HERE, "..", "libfa2_b200.so"), mode=ctypes.RTLD_GLOBAL)
_core.fa2_version.restype = ctypes.c_int
if _core.fa2_version() // 1000 != FA2_ABI_VERSION // 1000 or _core.fa2_version() < FA2_ABI_VERSION:
    raise ImportError(f"libfa2_b200.so has ABI version {_core.fa2_version()}, this binding needs {FA2_ABI_VERSION}")
_shim = ctypes.CDLL(os.path.join(_HERE, "libfa2_b200_xla.so"))
for _name in ("fa2_b200_fwd", "fa2_b200_bwd"):
    jax.ffi.register_ffi_target(_name, jax.ffi.pycapsule(getattr(_shim, _name)), platform="CUDA")


class _Problem(ctypes.Structure):   # fa2_problem of include/fa2_b200.h
    _fields_ = [
        ("batch", ctypes.c_int32), ("seqlen_q", ctypes.c_int32), ("seqlen_k", ctypes.c_int32),
        ("heads_q", ctypes.c_int32), ("heads_kv", ctypes.c_int32), ("head_dim", ctypes.c_int32),
        ("dtype", ctypes.c_int32), ("causal", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float), ("dropout_p", ctypes.c_float),
        ("dropout_seed", ctypes.c_uint64),
        ("batch_offset", ctypes.c_int32), ("head_offset", ctypes.c_int32),
        ("heads_q_global", ctypes.c_int32),
    ]


for _fn in (_core.fa2_bwd_workspace_bytes, _core.fa2_fwd_workspace_bytes, _core.fa2_dropout_bits_bytes):
    _fn.restype = ctypes.c_size_t
    _fn.argtypes = [ctypes.POINTER(_Problem)]


def _problem(q_shape, k_shape, dtype, dropout_prob=0.0) -> _Problem:
    p = _Problem()
    p.batch, p.seqlen_q, p.heads_q, p.head_dim = (int(x) for x in q_shape)
    p.seqlen_k, p.heads_kv = int(k_shape[1]), int(k_shape[2])
    p.dtype = 1 if dtype == jnp.bfloat16 else 0
    p.softmax_scale = 1.0
    p.dropout_p = float(dropout_prob)
    p.heads_q_global = p.heads_q
    return p


def _workspace_bytes(q_shape, k_shape, dtype) -> int:
    n = int(_core.fa2_bwd_workspace_bytes(ctypes.byref(_problem(q_shape, k_shape, dtype))))
    if n == 0:
        raise ValueError("fa2_b200: unsupported problem (head_dim, dtype or shape)")
    return n + _SCRATCH_SLACK


def _fwd_workspace_bytes(q_shape, k_shape, dtype, dropout_prob) -> int:
    """Scratch with which the forward splits a low-occupancy problem along the key sequence
    (nothing for most problems: only the alignment slack is declared then)."""
    n = int(_core.fa2_fwd_workspace_bytes(ctypes.byref(_problem(q_shape, k_shape, dtype, dropout_prob))))
    return n + _SCRATCH_SLACK


def _dropout_bits_words(q_shape, k_shape, dtype, dropout_prob, max_bytes=1 << 30) -> int:
    """Elements of the uint32 record of dropout keep bits the forward writes for the backward (1: no
    record, the backward draws the bits again: no dropout, or a record above max_bytes)."""
    n = int(_core.fa2_dropout_bits_bytes(ctypes.byref(_problem(q_shape, k_shape, dtype, dropout_prob))))
    return n // 4 if 0 < n <= max_bytes else 1


def _operands(q, bias, attention_mask):
    """(bias, additive mask, seqlens) with one-element dummies for what is absent. A 2-D
    [B, S] attention_mask is a padding mask: it becomes per-batch lengths (real tokens first),
    the reference's varlen mode without packing (_forward_triton.py:500-510)."""
    dummy = jnp.zeros((1,), q.dtype)
    seqlens = dummy
    mask = dummy
    if attention_mask is not None:
        if attention_mask.ndim == 2:
            seqlens = jnp.sum(attention_mask != 0, axis=1, dtype=jnp.int32)
        elif jnp.issubdtype(attention_mask.dtype, jnp.floating):
            mask = attention_mask
        else:
            mask = jnp.where(attention_mask != 0, 0.0, -jnp.inf).astype(q.dtype)
    return (dummy if bias is None else bias), mask, seqlens


def _seed_operand(q, dropout_seed):
    """The seed as a device operand (two uint32 words: low, high), so that a traced seed does not
    re-specialise the call; a python int or None goes through the attribute instead."""
    if dropout_seed is None or isinstance(dropout_seed, int):
        return jnp.zeros((1,), q.dtype), (0 if dropout_seed is None else dropout_seed)
    s = jnp.asarray(dropout_seed).reshape(()).astype(jnp.uint32)   # jax without x64: 32-bit seeds
    return jnp.stack([s, jnp.zeros((), jnp.uint32)]), 0


def _offsets_operand(q, offsets):
    """(batch offset, head offset) of this shard inside the unsharded problem as an int32 [2]
    operand (a traced value under shard_map); None means (0, 0)."""
    if offsets is None:
        return jnp.zeros((1,), q.dtype)
    return jnp.asarray(offsets, dtype=jnp.int32).reshape((2,))


def _attrs(q, softmax_scale, dropout_prob, causal, dropout_seed, heads_q_global):
    return dict(
        softmax_scale=np.float32(1.0 / math.sqrt(q.shape[-1]) if softmax_scale is None else softmax_scale),
        dropout_p=np.float32(dropout_prob),
        causal=bool(causal),
        dropout_seed=np.int64(0 if dropout_seed is None else dropout_seed),
        batch_offset=np.int32(0),          # shards pass their position as the `offsets` operand
        head_offset=np.int32(0),
        heads_q_global=np.int32(heads_q_global or q.shape[2]),
    )


def _fwd_attention_kernel_call(q, k, v, attention_mask=None, bias=None, softmax_scale=None,
                               dropout_prob=0.0, causal=False, dropout_seed=None, varlen_mode=True,
                               *, offsets=None, heads_q_global=None, return_dropout_bits=False):
    del varlen_mode
    assert q.shape[2] % k.shape[2] == 0, f"nheads_q = {q.shape[2]} is not divisible by nheads_kv = {k.shape[2]}"
    assert q.dtype == k.dtype == v.dtype, "All tensors must have the same type"
    assert q.dtype in (jnp.float16, jnp.bfloat16), "Only support fp16 and bf16"
    batch, sq, hq, _ = q.shape
    bias_, mask_, seqlens = _operands(q, bias, attention_mask)
    seed_op, seed_attr = _seed_operand(q, dropout_seed)
    out_types = (
        jax.ShapeDtypeStruct(q.shape, q.dtype),
        jax.ShapeDtypeStruct((batch, hq, -(-sq // 128) * 128), jnp.float32),
        jax.ShapeDtypeStruct((_dropout_bits_words(q.shape, k.shape, q.dtype, dropout_prob),), jnp.uint32),
        jax.ShapeDtypeStruct((_fwd_workspace_bytes(q.shape, k.shape, q.dtype, dropout_prob),), jnp.uint8),
    )
    out, lse, bits, _ = jax.ffi.ffi_call("fa2_b200_fwd", out_types)(
        q, k, v, bias_, mask_, seqlens, seed_op, _offsets_operand(q, offsets),
        **_attrs(q, softmax_scale, dropout_prob, causal, seed_attr, heads_q_global))
    if return_dropout_bits:
        return out, lse, bits
    return out, lse


def _bwd_attention_kernel_call(dO, q, k, v, bias, attention_mask, o, M, dropout_prob, causal,
                               softmax_scale, dropout_seed, varlen_mode=True, *, offsets=None,
                               heads_q_global=None, bias_grad=False, dropout_bits=None, deterministic=None):
    del varlen_mode
    if deterministic is None:   # bit-reproducible dq at the price of a slower backward
        deterministic = os.environ.get("FA2_B200_DETERMINISTIC", "0") not in ("", "0")
    bias_, mask_, seqlens = _operands(q, bias, attention_mask)
    seed_op, seed_attr = _seed_operand(q, dropout_seed)
    want_dbias = bias_grad and bias is not None
    out_types = (
        jax.ShapeDtypeStruct(q.shape, q.dtype),
        jax.ShapeDtypeStruct(k.shape, k.dtype),
        jax.ShapeDtypeStruct(v.shape, v.dtype),
        jax.ShapeDtypeStruct(bias.shape if want_dbias else (1,), jnp.float32),
        jax.ShapeDtypeStruct((_workspace_bytes(q.shape, k.shape, q.dtype),), jnp.uint8),
    )
    dq, dk, dv, dbias, _ = jax.ffi.ffi_call("fa2_b200_bwd", out_types)(
        dO, q, k, v, bias_, mask_, o, M, seqlens, seed_op, _offsets_operand(q, offsets),
        jnp.zeros((1,), jnp.uint32) if dropout_bits is None else dropout_bits,
        deterministic=bool(deterministic),
        **_attrs(q, softmax_scale, dropout_prob, causal, seed_attr, heads_q_global))
    return dq, dk, dv, (dbias.astype(bias.dtype) if want_dbias else None)


# Static (re-trace on change): softmax_scale, dropout_prob, causal, varlen_mode, as in the reference
# (flash_attention_triton/_flash_attention.py:91-92, nondiff_argnums=(5, 6, 7, 9)), plus the two
# static additions at the end. dropout_seed (8) and offsets (10) are traced operands: they take the
# place of differentiable arguments and get a None cotangent, like the seed in the reference (:88).
@functools.partial(jax.custom_vjp, nondiff_argnums=(5, 6, 7, 9, 11, 12))
def flash_attention_call(q, k, v, attention_mask=None, bias=None, softmax_scale=None, dropout_prob=0.0,
                         causal=False, dropout_seed=None, varlen_mode=True, offsets=None,
                         heads_q_global=None, bias_grad=False):
    return _fwd_attention_kernel_call(q, k, v, attention_mask, bias, softmax_scale, dropout_prob, causal,
                                      dropout_seed, varlen_mode, offsets=offsets,
                                      heads_q_global=heads_q_global)[0]


def _vjp_fwd(q, k, v, attention_mask, bias, softmax_scale, dropout_prob, causal, dropout_seed, varlen_mode,
             offsets, heads_q_global, bias_grad):
    out, lse, bits = _fwd_attention_kernel_call(q, k, v, attention_mask, bias, softmax_scale, dropout_prob,
                                                causal, dropout_seed, varlen_mode, offsets=offsets,
                                                heads_q_global=heads_q_global, return_dropout_bits=True)
    # one residual more than the reference keeps: the record of the dropout keep bits
    return out, (q, k, v, bias, attention_mask, out, lse, dropout_seed, offsets, bits)


def _vjp_bwd(softmax_scale, dropout_prob, causal, varlen_mode, heads_q_global, bias_grad, residual, dO):
    q, k, v, bias, attention_mask, out, lse, dropout_seed, offsets, bits = residual
    dq, dk, dv, dbias = _bwd_attention_kernel_call(
        dO, q, k, v, bias, attention_mask, out, lse, dropout_prob, causal, softmax_scale, dropout_seed,
        varlen_mode, offsets=offsets, heads_q_global=heads_q_global, bias_grad=bias_grad, dropout_bits=bits)
    # cotangents of (q, k, v, attention_mask, bias, dropout_seed, offsets)
    return dq, dk, dv, None, dbias, None, None


flash_attention_call.defvjp(_vjp_fwd, _vjp_bwd)


def sharded_flash_attention(q, k, v, *, causal=False, softmax_scale=None, dropout_prob=0.0,
                            dropout_seed=None, mesh_shape: tp.Optional[tp.Tuple[int, int]] = None):
    """One call spread over the local GPUs by (batch, kv head): every device runs the single-GPU
    kernels on its slice, no collective is issued (the query heads of a kv head are contiguous, so
    q's head axis shards consistently with k / v). Each shard hands its position in the mesh to the
    kernels as a traced int32 [2] operand, which keeps the dropout bits those of the unsharded call
    and needs one trace for all mesh positions; the body is the custom_vjp above, so jax.grad works
    through the sharded call and the backward sees the same offsets."""
    from jax.experimental.shard_map import shard_map
    from jax.sharding import Mesh, PartitionSpec as P

    devices = jax.devices()
    nb, nh = mesh_shape or (math.gcd(q.shape[0], len(devices)), len(devices) // math.gcd(q.shape[0], len(devices)))
    mesh = Mesh(np.array(devices[: nb * nh]).reshape(nb, nh), ("b", "h"))
    spec = P("b", None, "h", None)
    hq_global = q.shape[2]
    pb, ph = q.shape[0] // nb, q.shape[2] // nh

    def local(q_, k_, v_):
        offsets = jnp.stack([jax.lax.axis_index("b") * pb, jax.lax.axis_index("h") * ph]).astype(jnp.int32)
        return flash_attention_call(q_, k_, v_, None, None, softmax_scale, dropout_prob, causal, dropout_seed,
                                    True, offsets, hq_global, False)

    return shard_map(local, mesh, in_specs=(spec, spec, spec), out_specs=spec, check_rep=False)(q, k, v)
