"""ctypes binding of libfa2_b200.so (declared in include/fa2_b200.h).

The structures mirror the C header field by field. Nothing here computes anything: if the
library is missing the import of the kernels fails loudly, there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# FA2_B200_LIB points at another build of the same library (e.g. one compiled with other tuning
# macros); by default the in-tree build is used.
LIB_PATH = os.environ.get("FA2_B200_LIB") or os.path.join(_PKG_ROOT, "libfa2_b200.so")

FA2_FP16, FA2_BF16, FA2_FP32 = 0, 1, 2
FA2_OK = 0
FA2_ERR_INVALID_ARG, FA2_ERR_UNSUPPORTED, FA2_ERR_CUDA, FA2_ERR_WORKSPACE = -1, -2, -3, -4

EXPORTED_SYMBOLS = (
    "fa2_fwd",
    "fa2_bwd",
    "fa2_fwd_workspace_bytes",
    "fa2_bwd_workspace_bytes",
    "fa2_last_error",
    "fa2_version",
    "fa2_debug_device_status",
    "fa2_debug_bwd_stage_events",
    "fa2_bwd_static_scratch",
    "fa2_dropout_bits_bytes",
)
FA2_BWD_STATIC_SCRATCH_BYTES = 32 * 1024 * 1024
# FA2_ABI_VERSION of the header these structures were written against (major * 1000 + minor)
FA2_ABI_VERSION = 3000


class Strides(C.Structure):
    _fields_ = [("b", C.c_int64), ("s", C.c_int64), ("h", C.c_int64)]


class ScoreTerm(C.Structure):
    _fields_ = [
        ("ptr", C.c_void_p),
        ("dtype", C.c_int32),
        ("head_div", C.c_int32),
        ("stride_b", C.c_int64),
        ("stride_h", C.c_int64),
        ("stride_q", C.c_int64),
    ]


class ScoreGrad(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("batch", C.c_int32), ("heads", C.c_int32)]


class Problem(C.Structure):
    _fields_ = [
        ("batch", C.c_int32),
        ("seqlen_q", C.c_int32),
        ("seqlen_k", C.c_int32),
        ("heads_q", C.c_int32),
        ("heads_kv", C.c_int32),
        ("head_dim", C.c_int32),
        ("dtype", C.c_int32),
        ("causal", C.c_int32),
        ("softmax_scale", C.c_float),
        ("dropout_p", C.c_float),
        ("dropout_seed", C.c_uint64),
        ("batch_offset", C.c_int32),
        ("head_offset", C.c_int32),
        ("heads_q_global", C.c_int32),
    ]


class FwdParams(C.Structure):
    _fields_ = [
        ("p", Problem),
        ("q", C.c_void_p), ("q_strides", Strides),
        ("k", C.c_void_p), ("k_strides", Strides),
        ("v", C.c_void_p), ("v_strides", Strides),
        ("o", C.c_void_p), ("o_strides", Strides),
        ("lse", C.c_void_p),
        ("lse_stride_b", C.c_int64), ("lse_stride_h", C.c_int64),
        ("bias", ScoreTerm),
        ("mask", ScoreTerm),
        ("seqlens", C.c_void_p),
        ("dropout_seed_dev", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("offsets_dev", C.c_void_p),
        ("dropout_bits", C.c_void_p),
        ("dropout_bits_bytes", C.c_size_t),
    ]


class BwdParams(C.Structure):
    _fields_ = [
        ("p", Problem),
        ("q", C.c_void_p), ("q_strides", Strides),
        ("k", C.c_void_p), ("k_strides", Strides),
        ("v", C.c_void_p), ("v_strides", Strides),
        ("o", C.c_void_p), ("o_strides", Strides),
        ("d_o", C.c_void_p), ("do_strides", Strides),
        ("lse", C.c_void_p),
        ("lse_stride_b", C.c_int64), ("lse_stride_h", C.c_int64),
        ("bias", ScoreTerm),
        ("mask", ScoreTerm),
        ("dq", C.c_void_p), ("dq_strides", Strides),
        ("dk", C.c_void_p), ("dk_strides", Strides),
        ("dv", C.c_void_p), ("dv_strides", Strides),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("seqlens", C.c_void_p),
        ("dropout_seed_dev", C.c_void_p),
        ("offsets_dev", C.c_void_p),
        ("dbias", ScoreGrad),
        ("dropout_bits", C.c_void_p),
        ("dropout_bits_bytes", C.c_size_t),
        ("deterministic", C.c_int32),
    ]


class Fa2Error(RuntimeError):
    """A call into libfa2_b200.so returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"fa2_b200 error {code}: {message}")
        self.code = code


_lib = None


def load() -> C.CDLL:
    """Loads the shared library once and declares the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python {os.path.join(_PKG_ROOT, 'build.py')}`. "
            "There is no fallback implementation."
        )
    lib = C.CDLL(LIB_PATH)
    lib.fa2_version.argtypes = []
    lib.fa2_version.restype = C.c_int
    found = lib.fa2_version()
    if found // 1000 != FA2_ABI_VERSION // 1000 or found < FA2_ABI_VERSION:
        # a stale build would read the parameter blocks with another layout
        raise ImportError(
            f"{LIB_PATH} reports ABI version {found}, this binding needs {FA2_ABI_VERSION}: rebuild it with "
            f"`python {os.path.join(_PKG_ROOT, 'build.py')} --force`."
        )
    lib.fa2_fwd.argtypes = [C.POINTER(FwdParams), C.c_void_p]
    lib.fa2_fwd.restype = C.c_int
    lib.fa2_bwd.argtypes = [C.POINTER(BwdParams), C.c_void_p]
    lib.fa2_bwd.restype = C.c_int
    lib.fa2_fwd_workspace_bytes.argtypes = [C.POINTER(Problem)]
    lib.fa2_fwd_workspace_bytes.restype = C.c_size_t
    lib.fa2_bwd_workspace_bytes.argtypes = [C.POINTER(Problem)]
    lib.fa2_bwd_workspace_bytes.restype = C.c_size_t
    lib.fa2_dropout_bits_bytes.argtypes = [C.POINTER(Problem)]
    lib.fa2_dropout_bits_bytes.restype = C.c_size_t
    lib.fa2_last_error.argtypes = []
    lib.fa2_last_error.restype = C.c_char_p
    lib.fa2_debug_device_status.argtypes = [C.c_void_p]
    lib.fa2_debug_device_status.restype = C.c_int
    lib.fa2_bwd_static_scratch.argtypes = [C.POINTER(BwdParams), C.c_void_p]
    lib.fa2_bwd_static_scratch.restype = C.c_int
    lib.fa2_debug_bwd_stage_events.argtypes = [C.POINTER(C.c_void_p)]
    lib.fa2_debug_bwd_stage_events.restype = C.c_int
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != FA2_OK:
        raise Fa2Error(code, load().fa2_last_error().decode("utf-8", "replace"))
