"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header declares, and its
host-only entry points (version, status strings, workspace sizes, argument validation) behave."""

import ctypes
import os
import re

import pytest

from helpers import ext


def _declared_symbols():
    syms = set()
    for path in (ext.HEADER_PATH, ext.DEBUG_HEADER_PATH):   # the drop-in surface and the diagnostics header
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        syms |= set(re.findall(r"\b(corope_[a-z0-9_]+)\s*\(", text))
    return sorted(syms)


def test_library_is_built_and_exports_every_declared_symbol():
    ext.build()
    assert os.path.exists(ext.LIB_PATH)
    L = ctypes.CDLL(ext.LIB_PATH)
    syms = _declared_symbols()
    assert "corope_rope_attn_fwd" in syms and "corope_gqa_bwd" in syms and "corope_debug_expire_wait" in syms and len(syms) >= 12
    for s in syms:
        assert hasattr(L, s), s


def test_host_only_entry_points():
    L = ext.lib()
    assert L.corope_abi_version() == 1
    assert L.corope_status_string(0) == b"ok"
    assert b"head dimension" in L.corope_status_string(-3)
    # backward workspace of the Llama-7B-4K shape: packed tables + delta + fp32 dQ accumulator
    nbytes = L.corope_workspace_bytes(ext.OP_ROPE_BWD, 2, 32, 32, 4096, 128, 1)
    assert nbytes >= 2 * 32 * 4096 * 128 * 4 + 2 * 32 * 4096 * 4 + 4096 * 64 * 4
    assert nbytes % 256 == 0
    assert L.corope_workspace_bytes(ext.OP_GQA_BWD, 2, 32, 8, 2048, 128, 1) >= 2 * 2 * 8 * 2048 * 128 * 4
    assert L.corope_workspace_bytes(99, 1, 1, 1, 1, 64, 0) == 0
    # rotated fp16 operand copies of the tensor-core paths: forward = table + 2 bytes per element of k (16-bit, D = 128 only)
    elems = 2 * 32 * 4096 * 128
    fwd16 = L.corope_workspace_bytes(ext.OP_ROPE_FWD, 2, 32, 32, 4096, 128, 1)
    fwd32 = L.corope_workspace_bytes(ext.OP_ROPE_FWD, 2, 32, 32, 4096, 128, 0)
    assert fwd16 - fwd32 == 2 * elems and fwd32 < 4096 * 64 * 4 + 1024
    assert nbytes >= 6 * elems                                                      # backward: fp16 Q copy + fp32 dQ accumulator
    # D = 64, 16-bit, N % 128 == 0 runs zero-padded to D = 128: rotated K + padded q, v, o (four padded tensors); other D = 64 cases need only the table
    assert L.corope_workspace_bytes(ext.OP_ROPE_FWD, 2, 32, 32, 4096, 64, 1) >= 4 * elems * 2
    assert L.corope_workspace_bytes(ext.OP_ROPE_FWD, 2, 32, 32, 4000, 64, 1) < 4000 * 32 * 4 + 1024
    assert L.corope_workspace_bytes(ext.OP_ROPE_FWD, 2, 32, 32, 4096, 64, 0) < 4096 * 32 * 4 + 1024
    # Co-RoPE: fp16 copies of K and V for the tensor-core kernels (16-bit, D = 128, N % 64 == 0), none otherwise
    kv = 2 * 8 * 2048 * 128
    assert L.corope_workspace_bytes(ext.OP_GQA_FWD, 2, 32, 8, 2048, 128, 1) == 4 * kv
    assert L.corope_workspace_bytes(ext.OP_GQA_FWD, 2, 32, 8, 2048, 128, 0) == 256
    assert L.corope_workspace_bytes(ext.OP_GQA_FWD, 2, 32, 8, 2000, 128, 1) == 256


def test_argument_validation_happens_on_the_host():
    L = ext.lib()
    one = ctypes.c_void_p(256)  # never dereferenced: validation fails first
    rc = L.corope_rope_attn_fwd(None, None, None, None, None, 0, None, None, 1, 1, 1, 64, 0, 1, 1.0, None, 0, None, None)
    assert rc == -1
    rc = L.corope_rope_attn_fwd(one, one, one, one, one, 64, one, one, 1, 1, 16, 48, 0, 1, 1.0, one, 1 << 20, None, None)
    assert rc == -3
    rc = L.corope_rope_attn_fwd(one, one, one, one, one, 64, one, one, 1, 1, 0, 64, 0, 1, 1.0, one, 1 << 20, None, None)
    assert rc == -2
    rc = L.corope_rope_attn_fwd(one, one, one, one, one, 64, one, one, 1, 1, 16, 64, 7, 1, 1.0, one, 1 << 20, None, None)
    assert rc == -4
    rc = L.corope_rope_attn_fwd(one, one, one, one, one, 64, one, one, 1, 1, 16, 64, 0, 1, 1.0, one, 8, None, None)
    assert rc == -5
    rc = L.corope_gqa_fwd(one, one, one, one, one, one, 1, 6, 4, 16, 64, 0, 1.0, 1e4, one, 1 << 20, None, None)
    assert rc == -6
    rc = L.corope_gqa_fwd(one, one, one, one, one, one, 1, 16, 1, 16, 64, 0, 1.0, 1e4, one, 1 << 20, None, None)
    assert rc == -6


def test_entry_points_refuse_cpu_tensors():
    import torch
    from helpers import fused_attention, corope_attention

    q = torch.zeros(1, 1, 8, 64)
    t = torch.zeros(8, 64)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fused_attention(q, q, q, True, 1.0, t, t)
    with pytest.raises(RuntimeError, match="no CPU path"):
        corope_attention(q, q, q, True, 1.0, 1e4)


def test_corope_entry_point_raises_the_reference_errors():
    import torch
    from helpers import corope_attention

    q = torch.zeros(1, 4, 8, 64)
    k = torch.zeros(1, 2, 8, 64)
    with pytest.raises(ValueError, match="causal=True only"):
        corope_attention(q, k, k, False, 1.0, 1e4)
    with pytest.raises(ValueError, match="same shape"):
        corope_attention(q, k, torch.zeros(1, 2, 8, 32), True, 1.0, 1e4)
    with pytest.raises(ValueError, match="divisible"):
        corope_attention(torch.zeros(1, 3, 8, 64), k, k, True, 1.0, 1e4)
    with pytest.raises(ValueError, match="group_size <= 8"):
        corope_attention(torch.zeros(1, 32, 8, 64), k, k, True, 1.0, 1e4)
    with pytest.raises(ValueError, match="shape"):
        corope_attention(q[0], k, k, True, 1.0, 1e4)


def test_fused_entry_point_asserts_head_dim_like_the_reference():
    import torch
    from helpers import fused_attention

    q = torch.zeros(1, 1, 8, 48)
    t = torch.zeros(8, 48)
    with pytest.raises(AssertionError):
        fused_attention(q, q, q, True, 1.0, t, t)
