"""GPU parity tests: the CUDA kernels, called through the drop-in entry points (which call the C ABI),
against the CPU oracle on the same seeded inputs and against the committed golden vectors.

Tolerances are the ones the reference's verification uses for this path and the targets state:
bf16 / fp16: max-abs <= 1e-2 forward, <= 2e-2 gradients; fp32: <= 1e-4.
"""

import pytest
import torch

import oracle
import os

from helpers import (check16, corope_attention, draw, excess, ext, fused_attention, load_gold, maxdiff, rope_inputs, run_corope, run_fused)

pytestmark = pytest.mark.gpu

TOL_FWD_16, TOL_BWD_16, TOL_32 = 1e-2, 2e-2, 1e-4


def _label():
    """Name of the running test case, for the parity report."""
    return os.environ.get("PYTEST_CURRENT_TEST", "?").split("::")[-1].split(" ")[0]


@pytest.mark.parametrize("name", ["rope_a", "rope_b", "rope_c"])
def test_fused_rope_golden_fp32(name):
    g = load_gold(name)
    B, H, N, D, causal, _ = g["meta"].tolist()
    sm_scale, theta = g["scal"].tolist()
    q, k, v, do = (torch.from_numpy(g[x]).float() for x in ("q", "k", "v", "do"))
    cos, sin = torch.from_numpy(g["cos"]), torch.from_numpy(g["sin"])
    o, dq, dk, dv = run_fused(q, k, v, do, bool(causal), sm_scale, cos, sin)
    assert maxdiff(o, torch.from_numpy(g["o"])) < TOL_32
    assert maxdiff(dq, torch.from_numpy(g["dq"])) < TOL_32
    assert maxdiff(dk, torch.from_numpy(g["dk"])) < TOL_32
    assert maxdiff(dv, torch.from_numpy(g["dv"])) < TOL_32


@pytest.mark.parametrize("name", ["corope_a", "corope_b", "corope_c"])
def test_corope_golden_fp32(name):
    g = load_gold(name)
    sm_scale, theta = g["scal"].tolist()
    q, k, v, do = (torch.from_numpy(g[x]).float() for x in ("q", "k", "v", "do"))
    o, dq, dk, dv = run_corope(q, k, v, do, sm_scale, theta)
    assert maxdiff(o, torch.from_numpy(g["o"])) < TOL_32
    assert maxdiff(dq, torch.from_numpy(g["dq"])) < 2 * TOL_32
    assert maxdiff(dk, torch.from_numpy(g["dk"])) < 2 * TOL_32
    assert maxdiff(dv, torch.from_numpy(g["dv"])) < TOL_32


def test_fused_rope_config1_fp32():
    # B=4, H=8, N=512, D=64, fp32, causal, sm_scale = 1/sqrt(D)
    B, H, N, D = 4, 8, 512, 64
    q, k, v, do = rope_inputs(B, H, N, D, torch.float32, seed=1)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    ro = oracle.rope_attn_fwd(q, k, v, True, D ** -0.5, cos, sin)
    rdq, rdk, rdv = oracle.rope_attn_bwd(q, k, v, do, True, D ** -0.5, cos, sin)
    assert maxdiff(o, ro) < TOL_32
    assert maxdiff(dq, rdq) < TOL_32 and maxdiff(dk, rdk) < TOL_32 and maxdiff(dv, rdv) < TOL_32


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,causal", [((1, 2, 200, 64), True), ((2, 1, 96, 32), False), ((1, 2, 130, 128), False),
                                          ((1, 1, 384, 128), True)])
def test_fused_rope_general_kernels_16bit(dtype, shape, causal):
    # ragged N, non-causal, D = 32 / 64: shapes the tensor-core kernels do not take
    B, H, N, D = shape
    q, k, v, do = rope_inputs(B, H, N, D, dtype, seed=2)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    s = D ** -0.5
    o, dq, dk, dv = run_fused(q, k, v, do, causal, s, cos[:, : D // 2].contiguous(), sin[:, : D // 2].contiguous())
    ro = oracle.rope_attn_fwd(q, k, v, causal, s, cos, sin)
    rdq, rdk, rdv = oracle.rope_attn_bwd(q, k, v, do, causal, s, cos, sin)
    check16(_label() + " O", o, ro, TOL_FWD_16, dtype, strict=True)
    for got, ref in ((dq, rdq), (dk, rdk), (dv, rdv)):
        check16(_label() + " grad", got, ref, TOL_BWD_16, dtype)


@pytest.mark.parametrize("shape", [(2, 4, 512, 64), (1, 8, 1024, 128), (4, 16, 2048, 64)])
@pytest.mark.parametrize("causal", [False, True])
def test_fused_rope_reference_verification_cases_fp16(shape, causal):
    # The reference's verification script, case for case (fused-rope/verification.py:153-161): same shapes, fp16,
    # sm_scale 0.5, theta 1e4, and inputs drawn the way it draws them -- torch.manual_seed(42), then q, k, v with
    # torch.randn on the device (:32-38) and the output gradient with randn_like (:74).  Thresholds are its own:
    # forward max-abs < 1e-2 (:67); gradients max-abs < 0.15 and mean-abs < 5e-3 (:116).
    B, H, N, D = shape
    torch.manual_seed(42)
    q, k, v = (torch.randn(shape, dtype=torch.float16, device="cuda") for _ in range(3))
    do = torch.randn(shape, dtype=torch.float16, device="cuda")
    q, k, v, do = (t.cpu() for t in (q, k, v, do))
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, causal, 0.5, cos, sin)
    if N <= 1024:
        ro = oracle.rope_attn_fwd(q, k, v, causal, 0.5, cos, sin)
        refs = oracle.rope_attn_bwd(q, k, v, do, causal, 0.5, cos, sin)
    else:
        ro, _, rdq, rdk, rdv = oracle.rope_attn_fwd_bwd_chunked(q, k, v, do, causal, 0.5, cos, sin, rows=512)
        refs = (rdq, rdk, rdv)
    assert maxdiff(o, ro) < 1e-2
    for got, ref in zip((dq, dk, dv), refs):
        assert maxdiff(got, ref) < 0.15
        assert (got - ref).abs().mean().item() < 5e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 2, 256, 128), (2, 3, 1024, 128), (1, 2, 128, 128), (2, 3, 640, 128)])
def test_fused_rope_tensor_core_forward(dtype, shape):
    B, H, N, D = shape
    q, k, v, _ = rope_inputs(B, H, N, D, dtype, seed=3)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, _, _, _ = run_fused(q, k, v, None, True, D ** -0.5, cos, sin)
    assert ext.lib().corope_last_kernel_family(ext.OP_ROPE_FWD) == 1
    ro, lse2, _ = oracle.rope_attn_fwd(q, k, v, True, D ** -0.5, cos, sin, return_aux=True)
    check16(_label() + " O", o, ro, TOL_FWD_16, dtype, strict=True)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 2, 256, 128), (2, 3, 1024, 128), (1, 1, 384, 128)])
def test_fused_rope_tensor_core_backward(dtype, shape):
    B, H, N, D = shape
    q, k, v, do = rope_inputs(B, H, N, D, dtype, seed=5)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    assert ext.lib().corope_last_kernel_family(ext.OP_ROPE_FWD) == 1
    assert ext.lib().corope_last_kernel_family(ext.OP_ROPE_BWD) == 1
    ro = oracle.rope_attn_fwd(q, k, v, True, D ** -0.5, cos, sin)
    check16(_label() + " O", o, ro, TOL_FWD_16, dtype, strict=True)
    for name, got, ref in zip("qkv", (dq, dk, dv), oracle.rope_attn_bwd(q, k, v, do, True, D ** -0.5, cos, sin)):
        check16(_label() + " d" + name, got, ref, TOL_BWD_16, dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 2, 256, 128), (2, 3, 1024, 128), (1, 2, 2048, 128), (2, 2, 384, 128)])
def test_fused_rope_tensor_core_non_causal(dtype, shape):
    # full (non-causal) attention on the tensor-core kernels: every Q tile sees every K tile, no mask
    B, H, N, D = shape
    q, k, v, do = rope_inputs(B, H, N, D, dtype, seed=6)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, False, D ** -0.5, cos, sin)
    assert ext.lib().corope_last_kernel_family(ext.OP_ROPE_FWD) == 1
    assert ext.lib().corope_last_kernel_family(ext.OP_ROPE_BWD) == 1
    if N <= 1024:
        ro = oracle.rope_attn_fwd(q, k, v, False, D ** -0.5, cos, sin)
        refs = oracle.rope_attn_bwd(q, k, v, do, False, D ** -0.5, cos, sin)
    else:
        ro, _, rdq, rdk, rdv = oracle.rope_attn_fwd_bwd_chunked(q, k, v, do, False, D ** -0.5, cos, sin, rows=512)
        refs = (rdq, rdk, rdv)
    check16(_label() + " O", o, ro, TOL_FWD_16, dtype, strict=True)
    for name, got, ref in zip("qkv", (dq, dk, dv), refs):
        check16(_label() + " d" + name, got, ref, TOL_BWD_16, dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,causal", [((2, 3, 256, 64), True), ((1, 2, 1024, 64), True), ((2, 2, 384, 64), False)])
def test_fused_rope_head_dim_64_on_tensor_cores(dtype, shape, causal):
    # D = 64 with N % 128 == 0 runs zero-padded to D = 128 on the tensor-core kernels
    B, H, N, D = shape
    q, k, v, do = rope_inputs(B, H, N, D, dtype, seed=8)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, causal, D ** -0.5, cos, sin)
    assert ext.lib().corope_last_kernel_family(ext.OP_ROPE_FWD) == 1
    assert ext.lib().corope_last_kernel_family(ext.OP_ROPE_BWD) == 1
    ro = oracle.rope_attn_fwd(q, k, v, causal, D ** -0.5, cos, sin)
    check16(_label() + " O", o, ro, TOL_FWD_16, dtype, strict=True)
    for name, got, ref in zip("qkv", (dq, dk, dv), oracle.rope_attn_bwd(q, k, v, do, causal, D ** -0.5, cos, sin)):
        check16(_label() + " d" + name, got, ref, TOL_BWD_16, dtype)


def test_fused_rope_llama7b_4k_heads_bf16():
    # two heads of the Llama-7B-4K configuration at full sequence length, forward and backward
    B, H, N, D = 1, 2, 4096, 128
    q, k, v, do = rope_inputs(B, H, N, D, torch.bfloat16, seed=6)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    ro, lse2, rdq, rdk, rdv = oracle.rope_attn_fwd_bwd_chunked(q, k, v, do, True, D ** -0.5, cos, sin, rows=1024)
    check16(_label() + " O", o, ro, TOL_FWD_16, torch.bfloat16, strict=True)
    for name, got, ref in zip("qkv", (dq, dk, dv), (rdq, rdk, rdv)):
        check16(_label() + " d" + name, got, ref, TOL_BWD_16, torch.bfloat16)


def test_fused_rope_identity_tables_and_first_row():
    # the reference's own test_op uses cos = 1, sin = 0 (fused_rope_attn.py:803-804)
    B, H, N, D = 1, 2, 512, 128
    q, k, v, _ = rope_inputs(B, H, N, D, torch.bfloat16, seed=4)
    q, k, v = q * 0.5, k * 0.5, v * 0.5
    cos, sin = torch.ones(N, D), torch.zeros(N, D)
    o, _, _, _ = run_fused(q, k, v, None, True, 0.5, cos, sin)
    p = torch.matmul(q.float(), k.float().transpose(2, 3)) * 0.5
    p = p.masked_fill(torch.triu(torch.ones(N, N, dtype=torch.bool), 1), float("-inf"))
    ref = torch.matmul(torch.softmax(p, dim=-1), v.float())
    assert maxdiff(o, ref) < TOL_FWD_16
    assert maxdiff(o[..., 0, :], v[..., 0, :]) < 1e-6


@pytest.mark.parametrize("dtype,tolf,tolb", [(torch.bfloat16, TOL_FWD_16, TOL_BWD_16), (torch.float32, TOL_32, 2 * TOL_32)])
@pytest.mark.parametrize("cfg", [(1, 4, 1, 160, 64), (2, 4, 2, 96, 128), (1, 8, 1, 64, 64), (1, 3, 1, 40, 32)])
def test_corope_general_kernels(dtype, tolf, tolb, cfg):
    B, Hq, Hkv, N, D = cfg
    q = draw((B, Hq, N, D), 11, dtype)
    k = draw((B, Hkv, N, D), 12, dtype)
    v = draw((B, Hkv, N, D), 13, dtype)
    do = draw((B, Hq, N, D), 14, dtype)
    o, dq, dk, dv = run_corope(q, k, v, do, D ** -0.5, 10000.0)
    ro = oracle.corope_gqa_fwd(q, k, v, True, D ** -0.5, 10000.0)
    rdq, rdk, rdv = oracle.corope_gqa_bwd(q, k, v, do, True, D ** -0.5, 10000.0)
    assert excess(o, ro, tolf, dtype) <= 0
    for got, ref in ((dq, rdq), (dk, rdk), (dv, rdv)):
        assert excess(got, ref, tolb, dtype) <= 0


def test_fused_rope_llama70b_1k_heads_bf16():
    # heads of the Llama-70B-1K configuration (B=2, H=64, N=1024, D=128): 8 heads, the per-GPU share at 8 GPUs
    B, H, N, D = 1, 8, 1024, 128
    q, k, v, do = rope_inputs(B, H, N, D, torch.bfloat16, seed=7)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    ro = oracle.rope_attn_fwd(q, k, v, True, D ** -0.5, cos, sin)
    check16(_label() + " O", o, ro, TOL_FWD_16, torch.bfloat16, strict=True)
    for name, got, ref in zip("qkv", (dq, dk, dv), oracle.rope_attn_bwd(q, k, v, do, True, D ** -0.5, cos, sin)):
        check16(_label() + " d" + name, got, ref, TOL_BWD_16, torch.bfloat16)


def test_fused_rope_long_context_16k_full_gradients():
    # one head at N = 16384: every output row and all three gradients against the row-blocked oracle
    B, H, N, D = 1, 1, 16384, 128
    q, k, v, do = rope_inputs(B, H, N, D, torch.bfloat16, seed=8)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    ro, _, rdq, rdk, rdv = oracle.rope_attn_fwd_bwd_chunked(q, k, v, do, True, D ** -0.5, cos, sin, rows=1024)
    check16(_label() + " O", o, ro, TOL_FWD_16, torch.bfloat16, strict=True)
    for name, got, ref in zip("qkv", (dq, dk, dv), (rdq, rdk, rdv)):
        check16(_label() + " d" + name, got, ref, TOL_BWD_16, torch.bfloat16)


def test_fused_rope_long_context_64k_full_head():
    # one head of the Long-64K configuration (N = 65536): every row of O and all three gradients (dK and dV over every key
    # block) against the row-blocked oracle
    B, H, N, D = 1, 1, 65536, 128
    q, k, v, do = rope_inputs(B, H, N, D, torch.bfloat16, seed=9)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    ro, _, rdq, rdk, rdv = oracle.rope_attn_fwd_bwd_chunked(q, k, v, do, True, D ** -0.5, cos, sin, rows=1024)
    check16(_label() + " O", o, ro, TOL_FWD_16, torch.bfloat16, strict=True)
    for name, got, ref in zip("qkv", (dq, dk, dv), (rdq, rdk, rdv)):
        check16(_label() + " d" + name, got, ref, TOL_BWD_16, torch.bfloat16)


def test_fused_rope_llama7b_4k_full_launch_heads_across_chunks():
    # the whole Llama-7B-4K launch (B = 2, H = 32: 64 heads, i.e. 8 head chunks of the forward scheduler and 16 of the
    # backward's) with four heads from different chunks and both batch entries checked against the oracle
    B, H, N, D = 2, 32, 4096, 128
    q, k, v, do = rope_inputs(B, H, N, D, torch.bfloat16, seed=16)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    for t in (o, dq, dk, dv):
        assert torch.isfinite(t).all()
    for b, h in ((0, 0), (0, 13), (1, 7), (1, 31)):
        sl = (slice(b, b + 1), slice(h, h + 1))
        ro, _, rdq, rdk, rdv = oracle.rope_attn_fwd_bwd_chunked(q[sl], k[sl], v[sl], do[sl], True, D ** -0.5, cos, sin, rows=1024)
        tag = "%s b%d h%d" % (_label(), b, h)
        check16(tag + " O", o[sl], ro, TOL_FWD_16, torch.bfloat16, strict=True)
        for name, got, ref in zip("qkv", (dq[sl], dk[sl], dv[sl]), (rdq, rdk, rdv)):
            check16(tag + " d" + name, got, ref, TOL_BWD_16, torch.bfloat16)


def test_corope_config4_units_bf16():
    # (batch, KV head) units of the Co-RoPE configuration (groups of 4 query heads, D = 128): one unit at N = 512, and a
    # launch of two units at the configured N = 2048 -- O, dQ, dK and dV of both units in full (the oracle runs every
    # block of 32 query rows, so dK / dV are complete sums)
    D, G = 128, 4
    for N, units in ((512, 1), (2048, 2)):
        q = draw((1, G * units, N, D), 21, torch.bfloat16)
        k = draw((1, units, N, D), 22, torch.bfloat16)
        v = draw((1, units, N, D), 23, torch.bfloat16)
        do = draw((1, G * units, N, D), 24, torch.bfloat16)
        o, dq, dk, dv = run_corope(q, k, v, do, D ** -0.5, 10000.0)
        assert ext.lib().corope_last_kernel_family(ext.OP_GQA_FWD) == 1 and ext.lib().corope_last_kernel_family(ext.OP_GQA_BWD) == 1
        for u in range(units):
            hq, hk = slice(u * G, (u + 1) * G), slice(u, u + 1)
            ro, _, _, rdq, rdk, rdv = oracle.corope_gqa_fwd_bwd_chunked(q[:, hq], k[:, hk], v[:, hk], do[:, hq], D ** -0.5, 10000.0, rows=32)
            tag = "%s N%d unit%d" % (_label(), N, u)
            check16(tag + " O", o[:, hq], ro, TOL_FWD_16, torch.bfloat16, strict=True)
            check16(tag + " dQ", dq[:, hq], rdq, TOL_BWD_16, torch.bfloat16)
            check16(tag + " dK", dk[:, hk], rdk, TOL_BWD_16, torch.bfloat16)
            check16(tag + " dV", dv[:, hk], rdv, TOL_BWD_16, torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cfg", [(1, 1, 1, 128), (1, 2, 1, 192), (1, 3, 1, 64), (2, 8, 2, 256), (1, 8, 1, 320), (1, 5, 1, 128)])
def test_corope_tensor_core_groups(dtype, cfg):
    # the mma kernels (16-bit, D = 128, N % 64 == 0) for every group-size path, forward and all gradients, against the
    # oracle on the same values
    B, Hq, Hkv, N = cfg
    D = 128
    q = draw((B, Hq, N, D), 31, dtype)
    k = draw((B, Hkv, N, D), 32, dtype)
    v = draw((B, Hkv, N, D), 33, dtype)
    do = draw((B, Hq, N, D), 34, dtype)
    o, dq, dk, dv = run_corope(q, k, v, do, D ** -0.5, 10000.0)
    assert ext.lib().corope_last_kernel_family(ext.OP_GQA_FWD) == 1
    assert ext.lib().corope_last_kernel_family(ext.OP_GQA_BWD) == 1
    ro = oracle.corope_gqa_fwd(q, k, v, True, D ** -0.5, 10000.0)
    check16(_label() + " O", o, ro, TOL_FWD_16, dtype, strict=True)
    for name, got, ref in zip("qkv", (dq, dk, dv), oracle.corope_gqa_bwd(q, k, v, do, True, D ** -0.5, 10000.0)):
        check16(_label() + " d" + name, got, ref, TOL_BWD_16, dtype)


def test_host_pipeline_matches_direct_call():
    # the chunked host-to-host call must give what one call on the whole tensors gives (units are independent)
    import importlib
    pkg = importlib.import_module("co-rope_b200")
    B, H, N, D = 2, 6, 512, 128
    q, k, v, do = rope_inputs(B, H, N, D, torch.bfloat16, seed=41)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    hq, hk, hv, hdo = (t.pin_memory() for t in (q, k, v, do))
    ho, hdq, hdk, hdv = pkg.attention_fwd_bwd_host(hq, hk, hv, hdo, D ** -0.5, freqs_cos=cos.cuda(), freqs_sin=sin.cuda(), chunks=5)
    torch.cuda.synchronize()
    ext.check_status()
    assert torch.equal(ho.float(), o) and torch.equal(hdk.float(), dk) and torch.equal(hdv.float(), dv)
    assert maxdiff(hdq, dq) < 1e-2   # dQ is summed with floating-point reductions in an order that varies
    # Co-RoPE: groups of query heads stay with their KV head
    q = draw((2, 8, 128, D), 42, torch.bfloat16)
    k = draw((2, 2, 128, D), 43, torch.bfloat16)
    v = draw((2, 2, 128, D), 44, torch.bfloat16)
    do = draw((2, 8, 128, D), 45, torch.bfloat16)
    o, dq, dk, dv = run_corope(q, k, v, do, D ** -0.5, 10000.0)
    outs = pkg.attention_fwd_bwd_host(*(t.pin_memory() for t in (q, k, v, do)), D ** -0.5, theta=10000.0, chunks=3)
    torch.cuda.synchronize()
    ext.check_status()
    for got, ref in zip(outs, (o, dq, dk, dv)):
        assert maxdiff(got, ref) < 2e-2


@pytest.mark.parametrize("op", ["fused_rope", "corope"])
def test_calls_capture_into_cuda_graphs(op):
    # The library's calls are stream-ordered and allocate nothing: a forward + backward captured once as a CUDA graph and
    # replayed on new input values must give what the eager calls give (O, dK, dV of the fused-RoPE op bit for bit).
    import importlib
    pkg = importlib.import_module("co-rope_b200")
    rope_mod = importlib.import_module("co-rope_b200.fused_rope_attn")
    gqa_mod = importlib.import_module("co-rope_b200.flash_attn_co_rope_gqa_triton")
    B, Hq, Hkv, N, D = (2, 4, 4, 512, 128) if op == "fused_rope" else (1, 8, 2, 256, 128)
    dev = torch.device("cuda")
    sq, sk, sv, sdo = (torch.zeros(shape, dtype=torch.bfloat16, device=dev) for shape in
                       ((B, Hq, N, D), (B, Hkv, N, D), (B, Hkv, N, D), (B, Hq, N, D)))
    cos, sin = (t.cuda() for t in oracle.precompute_freqs_cis(D, N, 10000.0))

    def fwd_bwd(q, k, v, do):
        if op == "fused_rope":
            saved = rope_mod._forward(q, k, v, True, D ** -0.5, cos, sin)
            return (saved[3],) + tuple(rope_mod._backward(*saved, do, True, D ** -0.5))
        saved = gqa_mod._forward(q, k, v, True, D ** -0.5, 10000.0)
        return (saved[3],) + tuple(gqa_mod._backward(*saved, do, D ** -0.5, 10000.0))

    fwd_bwd(sq, sk, sv, sdo)   # workspaces and lazy initialisation happen outside the capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with pkg._ext.batched_status(dev):
        with torch.cuda.graph(g, capture_error_mode="relaxed"):
            outs = fwd_bwd(sq, sk, sv, sdo)
    for seed in (51, 52):
        vals = [draw(t.shape, seed + 10 * i, torch.bfloat16).cuda() for i, t in enumerate((sq, sk, sv, sdo))]
        for dst, src in zip((sq, sk, sv, sdo), vals):
            dst.copy_(src)
        g.replay()
        torch.cuda.synchronize()
        ext.check_status()
        got = [t.clone() for t in outs]
        ref = fwd_bwd(*vals)
        torch.cuda.synchronize()
        ext.check_status()
        if op == "fused_rope":
            assert torch.equal(got[0], ref[0]) and torch.equal(got[2], ref[2]) and torch.equal(got[3], ref[3])
            assert maxdiff(got[1], ref[1]) < 1e-2
        else:
            assert torch.equal(got[0], ref[0])
            for a, b in zip(got[1:], ref[1:]):
                assert maxdiff(a, b) <= TOL_BWD_16


def test_fused_rope_tensor_core_results_are_reproducible():
    # O, dK and dV are accumulated in a fixed order (TMEM accumulators), so repeated calls must agree bit for bit; a
    # difference means a race between the warp-specialised roles.  dQ is summed with floating-point reductions whose
    # order is free, so it may differ in the last bits only.
    B, H, N, D = 2, 4, 2048, 128
    q, k, v, do = rope_inputs(B, H, N, D, torch.bfloat16, seed=12)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    first = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    for _ in range(5):
        again = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
        assert torch.equal(first[0], again[0]), "O differs between runs"
        assert torch.equal(first[2], again[2]), "dK differs between runs"
        assert torch.equal(first[3], again[3]), "dV differs between runs"
        assert maxdiff(first[1], again[1]) < 1e-2


def test_fused_rope_head_dim_64_half_tables_with_poisoned_surroundings():
    # D = 64 on the tensor-core path with [N, D/2] tables that are the tail of a larger NaN-filled buffer: nothing outside
    # the tables' own [N, 32] columns may be read (a read past the end of a row would pull NaN into the results)
    B, H, N, D = 1, 2, 512, 64
    dtype = torch.bfloat16
    q, k, v, do = rope_inputs(B, H, N, D, dtype, seed=18)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    bufs = []
    for t in (cos, sin):
        buf = torch.full((3 * N * 32,), float("nan"), device="cuda")
        buf[N * 32: 2 * N * 32] = t[:, :32].contiguous().reshape(-1).cuda()
        bufs.append(buf[N * 32: 2 * N * 32].view(N, 32))
    o, dq, dk, dv = run_fused(q, k, v, do, True, D ** -0.5, bufs[0], bufs[1])
    assert ext.lib().corope_last_kernel_family(ext.OP_ROPE_FWD) == 1 and ext.lib().corope_last_kernel_family(ext.OP_ROPE_BWD) == 1
    for t in (o, dq, dk, dv):
        assert torch.isfinite(t).all()
    ro = oracle.rope_attn_fwd(q, k, v, True, D ** -0.5, cos, sin)
    check16(_label() + " O", o, ro, TOL_FWD_16, dtype, strict=True)
    for name, got, ref in zip("qkv", (dq, dk, dv), oracle.rope_attn_bwd(q, k, v, do, True, D ** -0.5, cos, sin)):
        check16(_label() + " d" + name, got, ref, TOL_BWD_16, dtype)


@pytest.mark.parametrize("policy", [0, 2])
def test_fused_rope_in_kernel_rotation_policy(policy):
    # policy 2: the tensor-core kernels rotate K (forward) and Q (backward) tiles in shared memory themselves -- no rotated
    # copy is written to the workspace; results must match the oracle like the default variant's
    B, H, N, D = 2, 3, 1024, 128
    q, k, v, do = rope_inputs(B, H, N, D, torch.bfloat16, seed=19)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    prev = ext.lib().corope_set_kernel_policy(policy)
    try:
        n0 = ext.lib().corope_launch_count()
        o, dq, dk, dv = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
        launches = ext.lib().corope_launch_count() - n0
    finally:
        ext.lib().corope_set_kernel_policy(prev)
    assert ext.lib().corope_last_kernel_family(ext.OP_ROPE_FWD) == 1 and ext.lib().corope_last_kernel_family(ext.OP_ROPE_BWD) == 1
    if policy == 2:   # forward: table pack + main kernel; backward: delta + table pack + main kernel + dQ finalize -- no pre-rotation kernels
        assert launches == 6, launches
    ro = oracle.rope_attn_fwd(q, k, v, True, D ** -0.5, cos, sin)
    check16(_label() + " O", o, ro, TOL_FWD_16, torch.bfloat16, strict=True)
    for name, got, ref in zip("qkv", (dq, dk, dv), oracle.rope_attn_bwd(q, k, v, do, True, D ** -0.5, cos, sin)):
        check16(_label() + " d" + name, got, ref, TOL_BWD_16, torch.bfloat16)


@pytest.mark.parametrize("qk_scale,v_scale,do_scale", [(1.0, 16.0, 16.0), (1.0, 64.0, 64.0), (1.0, 1.0, 256.0), (1.0, 1.0, 1024.0), (2.0, 16.0, 16.0)])
def test_fused_rope_scaled_inputs_bf16(qk_scale, v_scale, do_scale):
    # inputs far from N(0,1).  v and dO (the linear paths: P V, dV = P^T dO, dP = dO V^T) multiplied by 16 and 64, dO alone by
    # 256 and 1024 -- the magnitudes a loss-scaled training step produces -- and q, k by 2 (scores x 4).  O scales with v, dV
    # with dO, dQ / dK with both, so each tolerance is relative to the magnitude of its reference tensor; everything must stay
    # finite.  The limit is the fp16 operand dS = P (dP - delta) of the dK / dQ products: |dO| |v| sqrt(D) has to stay below
    # 65504, which v, dO x 1024 together would not.
    # (Scores far beyond that are outside what 16-bit operands can resolve: the error of a score grows as |score| * 2^-11,
    # for this kernel as for the reference's fp16 Triton kernels; see the value-range note in the C header.)
    B, H, N, D = 1, 2, 512, 128
    q, k, v, do = rope_inputs(B, H, N, D, torch.bfloat16, seed=20)
    q, k, v, do = q * qk_scale, k * qk_scale, v * v_scale, do * do_scale
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    outs = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    ro = oracle.rope_attn_fwd(q, k, v, True, D ** -0.5, cos, sin)
    refs = (ro,) + tuple(oracle.rope_attn_bwd(q, k, v, do, True, D ** -0.5, cos, sin))
    for name, got, ref, tol in zip(("O", "dQ", "dK", "dV"), outs, refs, (TOL_FWD_16, TOL_BWD_16, TOL_BWD_16, TOL_BWD_16)):
        assert torch.isfinite(got).all(), name
        mag = max(1.0, ref.abs().max().item())
        check16("%s qk x%g v x%g dO x%g %s (tolerance x %.0f)" % (_label(), qk_scale, v_scale, do_scale, name, mag), got, ref, tol * mag, torch.bfloat16)


@pytest.mark.parametrize("scale", [16.0, 1024.0])
def test_corope_scaled_gradients_bf16(scale):
    # output gradients as a loss-scaled fp16 / bf16 training step produces them (dO x 16, x 1024): dK of the tensor-core
    # backward is summed in fixed point with a range-safe slow path, so either the gradients are within (magnitude-relative)
    # tolerance or the status word reports that a term was clamped -- never a silently wrapped sum
    B, Hq, Hkv, N, D = 1, 4, 1, 256, 128
    q = draw((B, Hq, N, D), 51, torch.bfloat16)
    k = draw((B, Hkv, N, D), 52, torch.bfloat16)
    v = draw((B, Hkv, N, D), 53, torch.bfloat16)
    do = draw((B, Hq, N, D), 54, torch.bfloat16) * scale
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = corope_attention(qd, kd, vd, True, D ** -0.5, 10000.0)
    o.backward(do.cuda())
    assert ext.lib().corope_last_kernel_family(ext.OP_GQA_BWD) == 1
    try:
        ext.check_status()
        reported = False
    except RuntimeError as e:
        assert "0x2000" in str(e)
        reported = True
    refs = oracle.corope_gqa_bwd(q, k, v, do, True, D ** -0.5, 10000.0)
    for name, got, ref in zip(("dQ", "dK", "dV"), (qd.grad, kd.grad, vd.grad), refs):
        got = got.float().cpu()
        assert torch.isfinite(got).all(), name
        if not reported:
            mag = max(1.0, ref.abs().max().item())
            check16("%s x%d %s (tolerance x %.0f)" % (_label(), int(scale), name, mag), got, ref, TOL_BWD_16 * mag, torch.bfloat16)


def test_bounded_wait_expiry_is_reported_and_cleared():
    # the failure-detection path of the kernels: a wait that runs out records COROPE_DEV_WAIT_EXPIRED | id in the status
    # word and the kernel returns.  A test-only kernel waits (bounded, 2000 polls) on a barrier nobody arrives at.
    dev = torch.device("cuda", 0)
    lib = ext.lib()
    ext.check_status(dev)
    word = ext.status_word(dev)
    rc = lib.corope_debug_expire_wait(word.data_ptr(), 2000, torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(word.item()) == 0x1000 | 0x7e
    # a launch that is handed a set word returns without computing (outputs keep their previous contents) ...
    B, H, N, D = 1, 1, 256, 128
    q, k, v, _ = (t.cuda() for t in rope_inputs(B, H, N, D, torch.bfloat16, seed=21))
    cos, sin = (t.cuda() for t in oracle.precompute_freqs_cis(D, N, 10000.0))
    ext.post_call(dev)          # what every entry point does after its launch: refresh the host mirror of the word
    torch.cuda.synchronize()
    # ... and the next call through the drop-in entry point raises before launching anything, and clears the word
    with pytest.raises(RuntimeError, match="0x107e"):
        fused_attention(q, k, v, True, D ** -0.5, cos, sin)
    torch.cuda.synchronize()
    assert int(word.item()) == 0
    o = fused_attention(q, k, v, True, D ** -0.5, cos, sin)
    ext.check_status(dev)
    ro = oracle.rope_attn_fwd(q.cpu(), k.cpu(), v.cpu(), True, D ** -0.5, cos.cpu(), sin.cpu())
    check16(_label() + " O after clearing", o.float().cpu(), ro, TOL_FWD_16, torch.bfloat16, strict=True)
    # check_status() itself: synchronising form of the same report
    lib.corope_debug_expire_wait(word.data_ptr(), 100, torch.cuda.current_stream(dev).cuda_stream)
    with pytest.raises(RuntimeError, match="bounded"):
        ext.check_status(dev)
    ext.check_status(dev)
