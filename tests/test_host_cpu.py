"""CPU tests: public API surface, argument validation, C-ABI exports, shard planning."""
import ctypes as C
import os
import re

import pytest
import torch

import jax_flash_attn2 as J
from jax_flash_attn2 import _capi, sharding
from jax_flash_attn2._kernel_calls import _score_term, normalise_attention_mask

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "fa2_b200.h")).read()
    debug_header = open(os.path.join(ROOT, "include", "fa2_b200_debug.h")).read()
    assert "fa2_debug" not in header      # test / measurement hooks stay out of the attention ABI
    declared = set(re.findall(r"\b(fa2_[a-z_0-9]+)\s*\(", header + debug_header))
    assert declared, "no declarations found"
    lib = _capi.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(_capi.EXPORTED_SYMBOLS) <= declared
    assert lib.fa2_version() == _capi.FA2_ABI_VERSION == 3000
    assert f"#define FA2_ABI_VERSION {_capi.FA2_ABI_VERSION}" in header


def test_validation_errors_come_before_any_launch():
    lib = _capi.load()
    a = _capi.FwdParams()
    assert lib.fa2_fwd(None, None) == _capi.FA2_ERR_INVALID_ARG
    a.p.batch, a.p.seqlen_q, a.p.seqlen_k = 1, 128, 128
    a.p.heads_q, a.p.heads_kv, a.p.head_dim = 3, 2, 128
    a.p.dtype = _capi.FA2_BF16
    a.p.softmax_scale = 1.0
    assert lib.fa2_fwd(C.byref(a), None) == _capi.FA2_ERR_INVALID_ARG
    assert b"divisible" in lib.fa2_last_error()
    a.p.heads_q = 4
    for d in (72, 136, 288):       # not a multiple of 16 / of 32 / above 256
        a.p.head_dim = d
        assert lib.fa2_fwd(C.byref(a), None) == _capi.FA2_ERR_UNSUPPORTED
        assert b"head_dim" in lib.fa2_last_error()
    a.p.head_dim = 96              # padded to 128 inside: the workspace is sized for 128 columns
    rows = 1 * 4 * 128
    # statistics, fp32 dq accumulator, one word, (head dim 128) 4 KiB of statistics in MMA operand
    # form per 128 rows, and a counter per 128-row tile (256-byte granules) for the ordered mode
    assert lib.fa2_bwd_workspace_bytes(C.byref(a.p)) == 2 * rows * 4 + rows * 128 * 4 + 256 + rows // 128 * 4096 + 256
    a.p.head_dim = 64
    assert lib.fa2_bwd_workspace_bytes(C.byref(a.p)) == 2 * rows * 4 + rows * 64 * 4 + 256 + 256
    a.p.head_dim = 96
    a.p.head_dim = 128
    a.p.dropout_p = 1.0
    assert lib.fa2_fwd(C.byref(a), None) == _capi.FA2_ERR_INVALID_ARG
    a.p.dropout_p = 0.0
    a.p.dtype = _capi.FA2_FP32
    assert lib.fa2_fwd(C.byref(a), None) == _capi.FA2_ERR_UNSUPPORTED
    a.p.dtype = _capi.FA2_BF16
    assert lib.fa2_fwd(C.byref(a), None) == _capi.FA2_ERR_INVALID_ARG   # null pointers
    assert b"non-null" in lib.fa2_last_error()
    # workspace size is pure arithmetic
    n = lib.fa2_bwd_workspace_bytes(C.byref(a.p))
    rows = 1 * 4 * 128
    assert n == 2 * rows * 4 + rows * 128 * 4 + 256 + rows // 128 * 4096 + 256
    b = _capi.BwdParams()
    b.p = a.p
    assert lib.fa2_bwd(C.byref(b), None) == _capi.FA2_ERR_INVALID_ARG


def _bwd_params_with_fake_pointers(workspace_address):
    """A backward parameter block whose pointers are never dereferenced: validation stops first."""
    lib = _capi.load()
    b = _capi.BwdParams()
    b.p.batch, b.p.seqlen_q, b.p.seqlen_k = 1, 128, 128
    b.p.heads_q, b.p.heads_kv, b.p.head_dim = 4, 2, 128
    b.p.dtype, b.p.softmax_scale, b.p.heads_q_global = _capi.FA2_BF16, 1.0, 4
    for name in ("q", "k", "v", "o", "d_o", "lse", "dq", "dk", "dv"):
        setattr(b, name, 0x10000)
    b.lse_stride_h, b.lse_stride_b = 128, 4 * 128
    b.workspace = workspace_address
    b.workspace_bytes = lib.fa2_bwd_workspace_bytes(C.byref(b.p))
    return lib, b


def test_workspace_alignment_contract_is_128_bytes():
    """A caller whose allocator hands out 128-byte-aligned temporaries (XLA's buffer assignment
    does) must get past the workspace check; 64-byte alignment is refused with a clear message.
    No kernel is launched: with fake pointers the call stops at the next validation step."""
    lib, b = _bwd_params_with_fake_pointers(0x20000 + 64)
    assert lib.fa2_bwd(C.byref(b), None) == _capi.FA2_ERR_WORKSPACE
    assert b"128-byte aligned" in lib.fa2_last_error()
    lib, b = _bwd_params_with_fake_pointers(0x20000 + 128)
    b.q_strides = _capi.Strides(0, 0, 0)          # the next check after the workspace: operand strides
    rc = lib.fa2_bwd(C.byref(b), None)
    assert rc != _capi.FA2_OK and rc != _capi.FA2_ERR_WORKSPACE
    b.workspace_bytes -= 1
    assert lib.fa2_bwd(C.byref(b), None) == _capi.FA2_ERR_WORKSPACE


def test_bias_gradient_arguments_are_validated():
    lib, b = _bwd_params_with_fake_pointers(0x20000)
    b.dbias.ptr, b.dbias.batch, b.dbias.heads = 0x30000, 1, 4
    assert lib.fa2_bwd(C.byref(b), None) == _capi.FA2_ERR_INVALID_ARG
    assert b"bias is not" in lib.fa2_last_error()
    b.bias.ptr, b.bias.dtype = 0x40000, _capi.FA2_BF16
    b.dbias.heads = 3
    assert lib.fa2_bwd(C.byref(b), None) == _capi.FA2_ERR_INVALID_ARG
    assert b"heads 1, 2 or 4" in lib.fa2_last_error()


def test_problems_whose_item_counts_overflow_are_refused():
    lib = _capi.load()
    p = _capi.Problem()
    p.dtype, p.softmax_scale = _capi.FA2_BF16, 1.0
    p.batch, p.seqlen_q, p.seqlen_k, p.heads_q, p.heads_kv, p.head_dim = 65536, 16384, 16384, 64, 8, 128
    p.heads_q_global = 64
    assert lib.fa2_bwd_workspace_bytes(C.byref(p)) == 0
    a = _capi.FwdParams()
    a.p = p
    assert lib.fa2_fwd(C.byref(a), None) == _capi.FA2_ERR_UNSUPPORTED
    assert b"too large" in lib.fa2_last_error()


def test_stale_library_version_is_refused(monkeypatch):
    """The binding refuses a library whose ABI version differs from the one it was written for."""
    monkeypatch.setattr(_capi, "_lib", None)
    monkeypatch.setattr(_capi, "FA2_ABI_VERSION", 4000)
    with pytest.raises(ImportError, match="ABI version"):
        _capi.load()
    monkeypatch.setattr(_capi, "FA2_ABI_VERSION", 3000)
    assert _capi.load().fa2_version() == 3000


def test_forward_scratch_is_only_asked_for_low_occupancy_problems():
    lib = _capi.load()
    p = _capi.Problem()
    p.dtype, p.softmax_scale = _capi.FA2_BF16, 1.0
    def need(batch, sq, sk, hq, hkv, d):
        p.batch, p.seqlen_q, p.seqlen_k, p.heads_q, p.heads_kv, p.head_dim = batch, sq, sk, hq, hkv, d
        p.heads_q_global = hq
        return lib.fa2_fwd_workspace_bytes(C.byref(p))
    assert need(8, 4096, 4096, 32, 8, 128) == 0          # training shape: plenty of items
    assert need(1, 1, 32768, 32, 8, 128) > 0             # decode step: split along the keys
    assert need(1, 1, 512, 32, 8, 128) == 0              # too few keys to share out
    assert need(1, 1, 32768, 8, 8, 256) > 0              # the head dim 256 kernel splits as well
    assert lib.fa2_fwd_workspace_bytes(None) == 0
    # partial outputs + partial lse of every split, each rounded up to 256 bytes
    n = need(1, 256, 4096, 2, 2, 128)
    assert n > 0 and n % 256 == 0


def test_config_defaults_and_pairs():
    cfg = J.AttentionConfig(backend=J.Backend.GPU)
    assert cfg.platform == J.Platform.TRITON and cfg.blocksize_q == 128 and cfg.blocksize_k == 128
    assert J.AttentionConfig(backend=J.Backend.CPU).platform == J.Platform.JAX
    assert J.AttentionConfig(backend=J.Backend.TPU).platform == J.Platform.PALLAS
    with pytest.raises(ValueError):
        J.FlashAttention(J.AttentionConfig(backend=J.Backend.CPU, platform=J.Platform.TRITON))
    fa = J.create_flash_attention("gpu", "triton", softmax_scale=0.5)
    assert fa.config.softmax_scale == 0.5
    assert "triton" in repr(fa).lower() or "TRITON" in repr(fa)
    assert J.FlashAttention.forward is J.FlashAttention.__call__


def test_head_and_bias_rules():
    fa = J.create_flash_attention("gpu", "triton")
    q = torch.zeros(1, 8, 6, 64, dtype=torch.bfloat16)
    k = torch.zeros(1, 8, 4, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="divisible"):
        fa(q, k, k)
    # a bias with one head per key/value head is passed through (the kernels index it by
    # query head // group size instead of repeating it as the reference does)
    kv_bias = torch.zeros(1, 2, 8, 8)
    assert fa._handle_bias(kv_bias, 4, 2) is kv_bias
    assert fa._handle_bias(torch.zeros(1, 1, 8, 8), 4, 2).shape == (1, 1, 8, 8)
    with pytest.raises(ValueError, match="Incompatible bias shape"):
        fa._handle_bias(torch.zeros(1, 3, 8, 8), 4, 2)
    t, _ = _score_term(kv_bias, 1, 4, 8, 8, "bias", 2)
    assert t.head_div == 2 and t.stride_h == 64
    t, _ = _score_term(torch.zeros(1, 4, 8, 8), 1, 4, 8, 8, "bias", 2)
    assert t.head_div == 1
    with pytest.raises(NotImplementedError):
        J.FlashAttention(J.AttentionConfig(backend=J.Backend.CPU))(q, q, q)


def test_score_term_broadcast_rules():
    t, _ = _score_term(torch.zeros(1, 1, 16, 32), 2, 4, 16, 32, "bias")
    assert (t.stride_b, t.stride_h, t.stride_q) == (0, 0, 32)
    t, _ = _score_term(torch.zeros(2, 4, 16, 32), 2, 4, 16, 32, "bias")
    assert (t.stride_b, t.stride_h, t.stride_q) == (4 * 16 * 32, 16 * 32, 32)
    t, _ = _score_term(torch.zeros(2, 1, 1, 32), 2, 4, 16, 32, "mask")
    assert t.stride_q == 0
    for bad in ((3, 1, 16, 32), (2, 3, 16, 32), (2, 4, 15, 32), (2, 4, 16, 31)):
        with pytest.raises(ValueError):
            _score_term(torch.zeros(*bad), 2, 4, 16, 32, "bias")


def test_mask_normalisation():
    add, rows = normalise_attention_mask(torch.tensor([[1, 1, 0], [1, 0, 0]]), torch.bfloat16, 3, 3)
    assert add.shape == (2, 1, 1, 3) and rows.tolist() == [[True, True, False], [True, False, False]]
    assert add[0, 0, 0].tolist() == [0.0, 0.0, float("-inf")]
    m4 = torch.ones(1, 1, 3, 3, dtype=torch.bool).tril()
    add, rows = normalise_attention_mask(m4, torch.float16, 3, 3)
    assert rows is None and add.dtype == torch.float16 and add[0, 0, 0, 1] == float("-inf")
    fm = torch.zeros(1, 1, 3, 3)
    assert normalise_attention_mask(fm, torch.float16, 3, 3)[0] is fm
    with pytest.raises(AssertionError):
        normalise_attention_mask(torch.ones(2, 3), torch.float16, 3, 4)


@pytest.mark.parametrize("batch,hkv", [(2, 4), (8, 8), (4, 16), (1, 8), (4, 8)])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shard_plan_covers_every_unit_once(batch, hkv, world):
    seen = set()
    for rank in range(world):
        s = sharding.plan(batch, hkv, world, rank)
        assert s.units == batch * hkv // world
        for b in range(s.batch_start, s.batch_stop):
            for h in range(s.kv_head_start, s.kv_head_stop):
                assert (b, h) not in seen
                seen.add((b, h))
    assert len(seen) == batch * hkv


def test_shard_plan_rejects_uneven_split():
    with pytest.raises(ValueError):
        sharding.plan(1, 6, 4, 0)


def test_cuda_path_refuses_cpu_tensors():
    q = torch.zeros(1, 128, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        J.fwd_attention_kernel_call(q, q, q)
