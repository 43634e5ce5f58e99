"""GPU test of fa2_bwd_static_scratch, the backward entry point for callers that cannot hand the
library a workspace (no allocator reachable, or allocation forbidden where they run). It must give
the gradients fa2_bwd gives with a caller-owned workspace, on consecutive calls that share the
built-in scratch array. Collected last on purpose (the file name sorts after the others)."""
import ctypes as C
import math

import pytest
import torch

import workloads as W

pytestmark = pytest.mark.gpu


def _params(_capi, q, k, v, o, do, lse, dq, dk, dv, causal):
    from jax_flash_attn2._kernel_calls import _strides
    B, Sq, Hq, D = q.shape
    a = _capi.BwdParams()
    a.p.batch, a.p.seqlen_q, a.p.seqlen_k = B, Sq, k.shape[1]
    a.p.heads_q, a.p.heads_kv, a.p.head_dim = Hq, k.shape[2], D
    a.p.dtype = _capi.FA2_BF16 if q.dtype == torch.bfloat16 else _capi.FA2_FP16
    a.p.causal = int(causal)
    a.p.softmax_scale = 1.0 / math.sqrt(D)
    a.p.heads_q_global = Hq
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
        setattr(a, name, t.data_ptr())
        setattr(a, name + "_strides", _strides(t))
    a.d_o, a.do_strides = do.data_ptr(), _strides(do)
    a.lse, a.lse_stride_b, a.lse_stride_h = lse.data_ptr(), lse.stride(0), lse.stride(1)
    return a


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-30)).item()


def test_static_scratch_backward_matches_workspace_backward_twice_in_a_row():
    import jax_flash_attn2 as J
    from jax_flash_attn2 import _capi
    lib = _capi.load()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two different problems back to back: the second call finds the first call's leftovers
    for (B, S, Hq, Hkv, D, dtype, causal) in ((2, 384, 4, 2, 128, torch.bfloat16, True),
                                               (1, 300, 8, 8, 64, torch.float16, False)):
        q, k, v, do = (x.cuda() for x in W.make_qkv(B, S, S, Hq, Hkv, D, dtype, 0.5))
        out, lse = J.fwd_attention_kernel_call(q, k, v, None, None, None, 0.0, causal, None)
        ref_dq, ref_dk, ref_dv = J.bwd_attention_kernel_call(do, q, k, v, None, None, out, lse, 0.0, causal, None, None)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        a = _params(_capi, q, k, v, out, do, lse, dq, dk, dv, causal)       # workspace left null
        _capi.check(lib.fa2_bwd_static_scratch(C.byref(a), stream))
        torch.cuda.synchronize()
        assert J.device_status() == 0
        # dk / dv are bit-reproducible; dq is accumulated by unordered fp32 reductions
        assert torch.equal(dk, ref_dk) and torch.equal(dv, ref_dv)
        assert _rel(dq, ref_dq) <= 1e-2
        # and once more on the same inputs, this time watching the device's memory: with the
        # outputs allocated beforehand the call itself must not take or return a single byte,
        # neither from the driver (free memory of the device) nor from torch's caching allocator
        dq2, dk2, dv2 = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        a2 = _params(_capi, q, k, v, out, do, lse, dq2, dk2, dv2, causal)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        stats_before = torch.cuda.memory_stats()
        _capi.check(lib.fa2_bwd_static_scratch(C.byref(a2), stream))
        torch.cuda.synchronize()
        stats_after = torch.cuda.memory_stats()
        assert torch.cuda.mem_get_info()[0] == free_before
        for key in ("allocation.all.allocated", "allocation.all.freed", "segment.all.allocated"):
            assert stats_after[key] == stats_before[key], key
        assert torch.equal(dk2, ref_dk) and torch.equal(dv2, ref_dv)
        assert _rel(dq2, ref_dq) <= 1e-2


def test_static_scratch_backward_refuses_problems_beyond_its_limit():
    from jax_flash_attn2 import _capi
    lib = _capi.load()
    a = _capi.BwdParams()
    a.p.batch, a.p.seqlen_q, a.p.seqlen_k = 8, 4096, 4096
    a.p.heads_q, a.p.heads_kv, a.p.head_dim = 32, 8, 128
    a.p.dtype, a.p.softmax_scale, a.p.heads_q_global = _capi.FA2_BF16, 0.1, 32
    assert lib.fa2_bwd_workspace_bytes(C.byref(a.p)) > _capi.FA2_BWD_STATIC_SCRATCH_BYTES
    rc = lib.fa2_bwd_static_scratch(C.byref(a), None)
    assert rc == _capi.FA2_ERR_WORKSPACE
    assert b"built-in scratch" in lib.fa2_last_error()
