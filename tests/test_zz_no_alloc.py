"""The allocation-free forward entry point (corope_rope_attn_fwd_noalloc), called through the C ABI.

It serves callers that cannot allocate device memory where they call the library (a fixed, fully planned memory
arena; a hard memory budget; a point where an allocation would stall the device), so its scratch is a fixed array
inside the library.  The test checks calls in a row against the regular entry point (which takes a caller
workspace) and against the CPU oracle: each call uses a different length, different tables, dtype or mask, so it would
fail if anything left in the shared array by an earlier call were read.  This file sorts last so that a run stopping at the first failure has
already run every other test.
"""

import pytest
import torch

import oracle
from helpers import ext, rope_inputs

pytestmark = pytest.mark.gpu


def _call(fn_noalloc, q, k, v, cos, sin, causal, sm_scale):
    B, H, N, D = q.shape
    lib = ext.lib()
    dev = q.device
    o = torch.full_like(q, float("nan"))
    lse = torch.full((B, H, N), float("nan"), device=dev, dtype=torch.float32)
    code = ext.DTYPE_CODES[q.dtype]
    stream = ext.stream_ptr(dev)
    status = ext.status_word(dev).data_ptr()
    if fn_noalloc:
        rc = lib.corope_rope_attn_fwd_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(), cos.stride(0),
                                              o.data_ptr(), lse.data_ptr(), B, H, N, D, code, int(causal), sm_scale, status, stream)
    else:
        ws, nbytes = ext.workspace(ext.OP_ROPE_FWD, B, H, H, N, D, q.dtype, dev)
        rc = lib.corope_rope_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(), cos.stride(0),
                                      o.data_ptr(), lse.data_ptr(), B, H, N, D, code, int(causal), sm_scale, ws.data_ptr(), nbytes,
                                      status, stream)
    assert rc == 0, lib.corope_status_string(rc)
    torch.cuda.synchronize()
    ext.check_status()
    return o, lse


def test_noalloc_forward_matches_regular_entry_point_twice():
    dev = torch.device("cuda", 0)
    lib = ext.lib()
    # all take the tensor-core kernel (which needs the table); successive calls differ in length, tables, dtype and mask, so
    # anything read from what an earlier call left in the shared array would show
    cases = [((1, 2, 512, 128), 10000.0, 3, torch.bfloat16, True), ((2, 1, 256, 128), 500.0, 4, torch.bfloat16, True),
             ((1, 2, 384, 128), 10000.0, 5, torch.float16, True), ((1, 1, 256, 128), 2000.0, 6, torch.bfloat16, False)]
    for shape, theta, seed, dtype, causal in cases:
        B, H, N, D = shape
        hq, hk, hv, _ = rope_inputs(B, H, N, D, dtype, seed=seed)
        q, k, v = (t.to(dev) for t in (hq, hk, hv))
        hcos, hsin = oracle.precompute_freqs_cis(D, N, theta)
        cos, sin = hcos.to(dev), hsin.to(dev)
        o_ref, lse_ref = _call(False, q, k, v, cos, sin, causal, D ** -0.5)
        assert lib.corope_last_kernel_family(ext.OP_ROPE_FWD) == 1
        # make the general kernels the last family on record, so that the assertion below is about the call that follows
        prev = lib.corope_set_kernel_policy(1)
        _call(False, q, k, v, cos, sin, causal, D ** -0.5)
        lib.corope_set_kernel_policy(prev)
        assert lib.corope_last_kernel_family(ext.OP_ROPE_FWD) == 0
        o_new, lse_new = _call(True, q, k, v, cos, sin, causal, D ** -0.5)
        assert lib.corope_last_kernel_family(ext.OP_ROPE_FWD) == 1   # recorded by the allocation-free entry point itself
        assert not torch.isnan(o_new).any() and not torch.isnan(lse_new).any()
        assert (o_new.float() - o_ref.float()).abs().max().item() <= 1e-2
        assert (lse_new - lse_ref).abs().max().item() <= 1e-3
        # and against the CPU oracle, so that a fault shared by both entry points cannot hide
        ro, rlse2, _ = oracle.rope_attn_fwd(hq, hk, hv, causal, D ** -0.5, hcos, hsin, return_aux=True)
        assert (o_new.float().cpu() - ro).abs().max().item() <= 1e-2
        assert (lse_new.cpu() - rlse2).abs().max().item() <= 2e-2


def test_noalloc_follows_the_kernel_policy():
    dev = torch.device("cuda", 0)
    lib = ext.lib()
    B, H, N, D = 1, 1, 256, 128
    hq, hk, hv, _ = rope_inputs(B, H, N, D, torch.bfloat16, seed=7)
    q, k, v = (t.to(dev) for t in (hq, hk, hv))
    hcos, hsin = oracle.precompute_freqs_cis(D, N, 10000.0)
    prev = lib.corope_set_kernel_policy(1)
    try:
        o, _ = _call(True, q, k, v, hcos.to(dev), hsin.to(dev), True, D ** -0.5)
    finally:
        lib.corope_set_kernel_policy(prev)
    assert lib.corope_last_kernel_family(ext.OP_ROPE_FWD) == 0
    ro = oracle.rope_attn_fwd(hq, hk, hv, True, D ** -0.5, hcos, hsin)
    assert (o.float().cpu() - ro).abs().max().item() <= 1e-2


def test_noalloc_rejects_sizes_beyond_the_fixed_array():
    dev = torch.device("cuda", 0)
    t = torch.zeros(8, device=dev)
    p = t.data_ptr()
    lib = ext.lib()
    # N * D/2 = 16384 * 64 > 524288: refused on the host before anything is launched or dereferenced
    rc = lib.corope_rope_attn_fwd_noalloc(p, p, p, p, p, 64, p, p, 1, 1, 16384, 128, 1, 1, 0.1, None, None)
    assert rc == -10
    assert b"maximum" in lib.corope_status_string(rc)
