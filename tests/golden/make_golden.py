"""Generates tests/golden/ref_jax_*.npz by executing the reference's own blockwise code.

The reference (erfanzar/jax-flash-attn2) cannot be imported where this library is built: jax is
not installed. Its pure-JAX forward and backward (`_fwd_flash_attn`, `_bwd_flash_attn`) only use
a handful of jax calls (einsum, exp, where, while_loop, dynamic_slice ...). This script installs
a small numpy stand-in for exactly those calls under the module names `jax`, `jax.numpy`,
`jax.lax`, `jax.sharding` and `eformer.escale`, loads the reference's source files unmodified
from REFERENCE_ROOT, runs them on seeded inputs and stores inputs and outputs. The vectors pin
oracle/block.py (see tests/test_oracle.py). Nothing is copied from the reference: it is executed
where it lies. Run:  python tests/golden/make_golden.py /path/to/reference
(or set REFERENCE_ROOT in the environment).
"""
from __future__ import annotations

import importlib
import os
import sys
import types

import ml_dtypes
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE_ROOT = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT", "")
if not os.path.isdir(REFERENCE_ROOT):
    raise SystemExit("usage: python tests/golden/make_golden.py /path/to/jax-flash-attn2 (the reference checkout)")


def _install_numpy_jax():
    jax = types.ModuleType("jax")
    jnp = types.ModuleType("jax.numpy")
    lax = types.ModuleType("jax.lax")
    sharding = types.ModuleType("jax.sharding")
    rnd = types.ModuleType("jax.random")
    eformer = types.ModuleType("eformer")
    escale = types.ModuleType("eformer.escale")

    def _drop_precision(fn):
        def wrapped(*a, precision=None, **kw):
            # numpy has no bfloat16 contraction kernel: bfloat16 operands are contracted in float32
            # and the result rounded to bfloat16 once, which is also what XLA's CPU dot does for
            # 16-bit operands. (float16 stays on numpy's own float16 path, as in the first vectors.)
            arrays = [x for x in a if isinstance(x, np.ndarray)]
            if arrays and all(x.dtype == ml_dtypes.bfloat16 for x in arrays):
                a = tuple(x.astype(np.float32) if isinstance(x, np.ndarray) else x for x in a)
                return fn(*a, **kw).astype(ml_dtypes.bfloat16)
            return fn(*a, **kw)
        return wrapped

    for name in ("zeros", "full", "where", "maximum", "minimum", "max", "exp", "log", "sum",
                 "expand_dims", "float32", "float16", "inf", "broadcast_to", "zeros_like"):
        setattr(jnp, name, getattr(np, name))
    jnp.einsum = _drop_precision(np.einsum)
    jnp.matmul = _drop_precision(np.matmul)
    jnp.dtype = np.dtype
    jnp.bfloat16 = ml_dtypes.bfloat16

    def dynamic_slice_in_dim(x, start, size, axis=0):
        idx = [slice(None)] * x.ndim
        idx[axis] = slice(int(start), int(start) + int(size))
        return x[tuple(idx)]

    def dynamic_update_slice_in_dim(x, update, start, axis=0):
        out = np.array(x, copy=True)
        idx = [slice(None)] * x.ndim
        idx[axis] = slice(int(start), int(start) + update.shape[axis])
        out[tuple(idx)] = update
        return out

    def while_loop(cond, body, state):
        while cond(state):
            state = body(state)
        return state

    lax.dynamic_slice_in_dim = dynamic_slice_in_dim
    lax.dynamic_update_slice_in_dim = dynamic_update_slice_in_dim
    lax.while_loop = while_loop
    lax.PrecisionLike = object
    lax.select = lambda c, a, b: np.where(c, a, b)

    class _EvalShape:
        def __init__(self, shape):
            self.shape = shape

    def eval_shape(fn):
        return _EvalShape(fn().shape)

    class custom_vjp:  # only the call-through is needed: fwd/bwd are invoked directly below
        def __init__(self, fn, nondiff_argnums=()):
            self.fn = fn

        def defvjp(self, fwd, bwd):
            self.fwd, self.bwd = fwd, bwd

        def __call__(self, *a, **kw):
            return self.fn(*a, **kw)

    jax.jit = lambda fn=None, **kw: fn if fn is not None else (lambda f: f)
    jax.named_call = lambda fn, name=None: fn
    jax.eval_shape = eval_shape
    jax.custom_vjp = custom_vjp
    jax.Array = np.ndarray
    jax.device_put = lambda x, d=None: x
    jax.numpy, jax.lax, jax.sharding, jax.random = jnp, lax, sharding, rnd
    rnd.PRNGKey = object
    sharding.NamedSharding = type("NamedSharding", (), {})
    sharding.SingleDeviceSharding = type("SingleDeviceSharding", (), {})
    sharding.PartitionSpec = tuple
    escale.with_sharding_constraint = lambda arr, sharding: arr
    eformer.escale = escale
    sys.modules.update({
        "jax": jax, "jax.numpy": jnp, "jax.lax": lax, "jax.sharding": sharding, "jax.random": rnd,
        "eformer": eformer, "eformer.escale": escale,
    })


def _load_reference():
    _install_numpy_jax()
    pkg = types.ModuleType("ref_flash_attention_jax")
    pkg.__path__ = [os.path.join(REFERENCE_ROOT, "jax_flash_attn2", "flash_attention_jax")]
    sys.modules["ref_flash_attention_jax"] = pkg
    fwd = importlib.import_module("ref_flash_attention_jax._forward_jax")
    bwd = importlib.import_module("ref_flash_attention_jax._backward_jax")
    return fwd._fwd_flash_attn, bwd._bwd_flash_attn


def _case(name, B, H, S, D, dtype, causal, with_bias, block, seed):
    fwd, bwd = _load_reference()
    rng = np.random.default_rng(seed)
    scale = 1.0 / np.sqrt(D)
    q = rng.standard_normal((B, H, S, D), dtype=np.float32).astype(dtype)
    k = rng.standard_normal((B, H, S, D), dtype=np.float32).astype(dtype)
    v = rng.standard_normal((B, H, S, D), dtype=np.float32).astype(dtype)
    do = rng.standard_normal((B, H, S, D), dtype=np.float32).astype(dtype)
    bias = (0.5 * rng.standard_normal((B, H, S, S), dtype=np.float32)).astype(dtype) if with_bias else None
    mask = np.tril(np.ones((S, S), dtype=bool))[None, None] if causal else None
    mask_b = np.broadcast_to(mask, (B, H, S, S)) if causal else None
    # The wrapper (flash_attention_jax/_flash_attention.py:112-119) pre-scales q in the input dtype.
    q_scaled = (q * np.asarray(scale, dtype=dtype)).astype(dtype) if dtype != np.float32 else q * np.float32(scale)
    out, res = fwd(q_scaled, k, v, mask_b, bias, 0.0, True, None, block, block, dtype, None)
    lse = res[1]
    dq_s, dk, dv, _, _ = bwd(0.0, True, None, block, block, dtype, None, res, do)
    np.savez_compressed(
        os.path.join(HERE, f"ref_jax_{name}.npz"),
        q=q, k=k, v=v, do=do, bias=bias if with_bias else np.zeros((0,), dtype), causal=np.array(causal),
        scale=np.float32(scale), block=np.array(block),
        out=np.asarray(out), lse=np.asarray(lse, dtype=np.float32),
        dq_wrt_scaled_q=np.asarray(dq_s), dk=np.asarray(dk), dv=np.asarray(dv),
    )
    print(name, "out", out.dtype, out.shape, "lse", lse.shape)


if __name__ == "__main__":
    _case("f32_causal", 1, 2, 128, 32, np.float32, True, False, 64, 0)
    _case("f32_bias", 1, 2, 128, 32, np.float32, False, True, 64, 1)
    _case("f32_causal_bias_b128", 1, 1, 256, 32, np.float32, True, True, 128, 2)
    _case("f16_causal", 1, 2, 256, 32, np.float16, True, False, 128, 3)
    # 16-bit inputs at the head dims and block size of the CUDA kernels, causal mask and bias together
    _case("bf16_causal_bias_d64_b128", 1, 1, 512, 64, ml_dtypes.bfloat16, True, True, 128, 4)
    _case("bf16_causal_bias_d128_b128", 1, 1, 384, 128, ml_dtypes.bfloat16, True, True, 128, 5)
    _case("f16_causal_bias_d128_b128", 1, 1, 256, 128, np.float16, True, True, 128, 6)
