"""GPU parity tests: the CUDA kernels, called through the drop-in entry points (which call the C ABI),
against the CPU oracle on the same seeded inputs and against the committed golden vectors.

Tolerances are the ones the reference's verification uses for this path and the targets state:
bf16 / fp16: max-abs <= 1e-2 forward, <= 2e-2 gradients; fp32: <= 1e-4.
"""

import pytest
import torch

import oracle
from helpers import (corope_attention, draw, excess, ext, fused_attention, load_gold, maxdiff, rope_inputs, run_corope, run_fused)

pytestmark = pytest.mark.gpu

TOL_FWD_16, TOL_BWD_16, TOL_32 = 1e-2, 2e-2, 1e-4


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
    assert excess(o, ro, TOL_FWD_16, dtype) <= 0
    for got, ref in ((dq, rdq), (dk, rdk), (dv, rdv)):
        assert excess(got, ref, TOL_BWD_16, dtype) <= 0


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
    assert excess(o, ro, TOL_FWD_16, dtype) <= 0


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
    assert excess(o, ro, TOL_FWD_16, dtype) <= 0
    for name, got, ref in zip("qkv", (dq, dk, dv), oracle.rope_attn_bwd(q, k, v, do, True, D ** -0.5, cos, sin)):
        assert excess(got, ref, TOL_BWD_16, dtype) <= 0, "d" + name


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
    assert excess(o, ro, TOL_FWD_16, dtype) <= 0
    for name, got, ref in zip("qkv", (dq, dk, dv), refs):
        assert excess(got, ref, TOL_BWD_16, dtype) <= 0, "d" + name


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
    assert excess(o, ro, TOL_FWD_16, dtype) <= 0
    for name, got, ref in zip("qkv", (dq, dk, dv), oracle.rope_attn_bwd(q, k, v, do, causal, D ** -0.5, cos, sin)):
        assert excess(got, ref, TOL_BWD_16, dtype) <= 0, "d" + name


def test_fused_rope_llama7b_4k_heads_bf16():
    # two heads of the Llama-7B-4K configuration at full sequence length, forward and backward
    B, H, N, D = 1, 2, 4096, 128
    q, k, v, do = rope_inputs(B, H, N, D, torch.bfloat16, seed=6)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    ro, lse2, rdq, rdk, rdv = oracle.rope_attn_fwd_bwd_chunked(q, k, v, do, True, D ** -0.5, cos, sin, rows=1024)
    assert excess(o, ro, TOL_FWD_16, torch.bfloat16) <= 0
    for name, got, ref in zip("qkv", (dq, dk, dv), (rdq, rdk, rdv)):
        assert excess(got, ref, TOL_BWD_16, torch.bfloat16) <= 0, "d" + name


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
    assert excess(o, ro, TOL_FWD_16, torch.bfloat16) <= 0
    for name, got, ref in zip("qkv", (dq, dk, dv), oracle.rope_attn_bwd(q, k, v, do, True, D ** -0.5, cos, sin)):
        assert excess(got, ref, TOL_BWD_16, torch.bfloat16) <= 0, "d" + name


def test_fused_rope_long_context_16k_full_gradients():
    # one head at N = 16384: every output row and all three gradients against the row-blocked oracle
    B, H, N, D = 1, 1, 16384, 128
    q, k, v, do = rope_inputs(B, H, N, D, torch.bfloat16, seed=8)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, dk, dv = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    ro, _, rdq, rdk, rdv = oracle.rope_attn_fwd_bwd_chunked(q, k, v, do, True, D ** -0.5, cos, sin, rows=1024)
    assert excess(o, ro, TOL_FWD_16, torch.bfloat16) <= 0
    for name, got, ref in zip("qkv", (dq, dk, dv), (rdq, rdk, rdv)):
        assert excess(got, ref, TOL_BWD_16, torch.bfloat16) <= 0, "d" + name


def test_fused_rope_long_context_64k_sampled_rows():
    # one head of the Long-64K configuration (N = 65536): O and dQ on the first, a middle and the last block of 1024 rows
    B, H, N, D = 1, 1, 65536, 128
    q, k, v, do = rope_inputs(B, H, N, D, torch.bfloat16, seed=9)
    cos, sin = oracle.precompute_freqs_cis(D, N, 10000.0)
    o, dq, _, _ = run_fused(q, k, v, do, True, D ** -0.5, cos, sin)
    blocks = [0, 37, 63]
    ro, _, rdq, _, _ = oracle.rope_attn_fwd_bwd_chunked(q, k, v, do, True, D ** -0.5, cos, sin, rows=1024, row_blocks=blocks)
    for b in blocks:
        sl = slice(b * 1024, (b + 1) * 1024)
        assert excess(o[:, :, sl], ro[:, :, sl], TOL_FWD_16, torch.bfloat16) <= 0
        assert excess(dq[:, :, sl], rdq[:, :, sl], TOL_BWD_16, torch.bfloat16) <= 0


def test_corope_config4_unit_bf16():
    # one (batch, KV head) unit of the Co-RoPE configuration (group of 4 query heads, D = 128): full check at N = 512,
    # O / dQ on sampled row blocks at the full N = 2048
    D, G = 128, 4
    for N, blocks in ((512, None), (2048, [0, 31, 63])):
        q = draw((1, G, N, D), 21, torch.bfloat16)
        k = draw((1, 1, N, D), 22, torch.bfloat16)
        v = draw((1, 1, N, D), 23, torch.bfloat16)
        do = draw((1, G, N, D), 24, torch.bfloat16)
        o, dq, dk, dv = run_corope(q, k, v, do, D ** -0.5, 10000.0)
        ro, _, _, rdq, rdk, rdv = oracle.corope_gqa_fwd_bwd_chunked(q, k, v, do, D ** -0.5, 10000.0, rows=32, row_blocks=blocks)
        if blocks is None:
            assert excess(o, ro, TOL_FWD_16, torch.bfloat16) <= 0
            for name, got, ref in zip("qkv", (dq, dk, dv), (rdq, rdk, rdv)):
                assert excess(got, ref, TOL_BWD_16, torch.bfloat16) <= 0, "d" + name
        else:
            for b in blocks:
                sl = slice(b * 32, (b + 1) * 32)
                assert excess(o[:, :, sl], ro[:, :, sl], TOL_FWD_16, torch.bfloat16) <= 0
                assert excess(dq[:, :, sl], rdq[:, :, sl], TOL_BWD_16, torch.bfloat16) <= 0


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
    assert excess(o, ro, TOL_FWD_16, dtype) <= 0
    for name, got, ref in zip("qkv", (dq, dk, dv), oracle.corope_gqa_bwd(q, k, v, do, True, D ** -0.5, 10000.0)):
        assert excess(got, ref, TOL_BWD_16, dtype) <= 0, "d" + name


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
