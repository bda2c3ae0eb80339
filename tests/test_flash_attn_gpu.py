"""GPU parity tests of the two widened entry points: plain flash attention with grouped K / V heads (the reference's
flash_attn_v2_triton.attention signature) and fused-RoPE attention with the tables synthesized from frequencies.
Everything goes through the drop-in Python modules, i.e. through the C ABI.  Tolerances as in test_gpu_parity.py."""

import os

import pytest
import torch

import oracle
from helpers import check16, draw, ext, load_gold, maxdiff, pkg

pytestmark = pytest.mark.gpu

TOL_FWD_16, TOL_BWD_16, TOL_32 = 1e-2, 2e-2, 1e-4
flash_attention = pkg.flash_attention
attention_theta = pkg.fused_rope_attention_theta


def _label():
    return os.environ.get("PYTEST_CURRENT_TEST", "?").split("::")[-1].split(" ")[0]


def run_flash(q, k, v, do, causal, sm_scale):
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = flash_attention(qd, kd, vd, causal, sm_scale)
    o.backward(do.cuda())
    ext.check_status()
    return tuple(t.detach().float().cpu() for t in (o, qd.grad, kd.grad, vd.grad))


@pytest.mark.parametrize("name", ["attn_gqa_a", "attn_gqa_b", "attn_gqa_c"])
def test_flash_attention_golden_fp32(name):
    g = load_gold(name)
    B, Hq, Hkv, N, D, causal, _ = g["meta"].tolist()
    (sm_scale,) = g["scal"].tolist()
    q, k, v, do = (torch.from_numpy(g[x]).float() for x in ("q", "k", "v", "do"))
    o, dq, dk, dv = run_flash(q, k, v, do, bool(causal), sm_scale)
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert got.shape == g[key].shape
        assert maxdiff(got, torch.from_numpy(g[key])) < TOL_32, key


def _inputs(B, Hq, Hkv, N, D, dtype, seed):
    return (draw((B, Hq, N, D), seed, dtype), draw((B, Hkv, N, D), seed + 1, dtype), draw((B, Hkv, N, D), seed + 2, dtype),
            draw((B, Hq, N, D), seed + 3, dtype))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cfg,causal", [((1, 4, 2, 200, 64), True), ((2, 6, 2, 96, 32), False), ((1, 8, 1, 130, 128), True)])
def test_flash_attention_general_kernels_16bit(dtype, cfg, causal):
    # ragged N and D = 32: the CUDA-core kernels, groups of 2, 3 and 8 query heads per K / V head
    B, Hq, Hkv, N, D = cfg
    q, k, v, do = _inputs(B, Hq, Hkv, N, D, dtype, 60)
    outs = run_flash(q, k, v, do, causal, D ** -0.5)
    assert ext.lib().corope_last_kernel_family(ext.OP_ROPE_FWD) == 0
    refs = (oracle.attn_gqa_fwd(q, k, v, causal, D ** -0.5),) + tuple(oracle.attn_gqa_bwd(q, k, v, do, causal, D ** -0.5))
    check16(_label() + " O", outs[0], refs[0], TOL_FWD_16, dtype, strict=True)
    for name, got, ref in zip(("dQ", "dK", "dV"), outs[1:], refs[1:]):
        check16(_label() + " " + name, got, ref, TOL_BWD_16, dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cfg,causal", [((1, 2, 2, 256, 128), True), ((2, 8, 2, 512, 128), True), ((1, 6, 2, 384, 128), False),
                                        ((1, 8, 1, 1024, 128), True), ((2, 4, 2, 256, 64), True), ((1, 6, 3, 384, 64), False)])
def test_flash_attention_tensor_core_groups(dtype, cfg, causal):
    # the tcgen05 kernels with the rotation off: group sizes 1, 2, 3, 4 and 8; D = 64 runs zero-padded on them
    B, Hq, Hkv, N, D = cfg
    q, k, v, do = _inputs(B, Hq, Hkv, N, D, dtype, 70)
    outs = run_flash(q, k, v, do, causal, D ** -0.5)
    assert ext.lib().corope_last_kernel_family(ext.OP_ROPE_FWD) == 1 and ext.lib().corope_last_kernel_family(ext.OP_ROPE_BWD) == 1
    refs = (oracle.attn_gqa_fwd(q, k, v, causal, D ** -0.5),) + tuple(oracle.attn_gqa_bwd(q, k, v, do, causal, D ** -0.5))
    check16(_label() + " O", outs[0], refs[0], TOL_FWD_16, dtype, strict=True)
    for name, got, ref in zip(("dQ", "dK", "dV"), outs[1:], refs[1:]):
        check16(_label() + " " + name, got, ref, TOL_BWD_16, dtype)


def test_flash_attention_llama70b_like_gqa_bf16():
    # a Llama-70B-like group shape: 8 query heads per K / V head, N = 2048
    B, Hq, Hkv, N, D = 1, 16, 2, 2048, 128
    q, k, v, do = _inputs(B, Hq, Hkv, N, D, torch.bfloat16, 80)
    outs = run_flash(q, k, v, do, True, D ** -0.5)
    ro, _, rdq, rdk, rdv = oracle.attn_gqa_fwd_bwd_chunked(q, k, v, do, True, D ** -0.5, rows=512)
    check16(_label() + " O", outs[0], ro, TOL_FWD_16, torch.bfloat16, strict=True)
    for name, got, ref in zip(("dQ", "dK", "dV"), outs[1:], (rdq, rdk, rdv)):
        check16(_label() + " " + name, got, ref, TOL_BWD_16, torch.bfloat16)


def test_flash_attention_rejects_bad_groups():
    q = torch.zeros(1, 3, 64, 64, device="cuda", dtype=torch.bfloat16)
    k = torch.zeros(1, 2, 64, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        flash_attention(q, k, k, True, 0.1)
    rc = ext.lib().corope_flash_attn_fwd(q.data_ptr(), k.data_ptr(), k.data_ptr(), q.data_ptr(), q.data_ptr(), 1, 3, 2, 64, 64, 1, 1, 0.1,
                                         None, 0, None, None)
    assert rc == -6


# ---------------------------------------------------------------------------------------------------------------------
def test_synthesized_tables_equal_precompute_freqs_cis():
    # element-by-element: the tables the frequency entry points build on the device against precompute_freqs_cis evaluated
    # by torch on the same device (the reference's default, rope_attn_pytorch.py:11)
    import importlib
    fr = importlib.import_module("co-rope_b200.fused_rope_attn")
    for D, N, theta in ((128, 4096, 10000.0), (64, 1000, 500000.0), (32, 65536, 10000.0)):
        inv = fr.inv_freq_of(theta, D, "cuda")
        cos = torch.empty((N, D // 2), device="cuda")
        sin = torch.empty_like(cos)
        rc = ext.lib().corope_debug_synth_tables(inv.data_ptr(), cos.data_ptr(), sin.data_ptr(), N, D // 2, None)
        assert rc == 0
        torch.cuda.synchronize()
        ang = torch.outer(torch.arange(N, device="cuda", dtype=torch.float32), inv)
        rc_, rs_ = torch.cos(ang), torch.sin(ang)
        # same angles bit for bit (one fp32 multiply); cos / sin may differ by a rounding of the last place between two
        # correctly-working implementations
        assert (cos - rc_).abs().max().item() <= 2.4e-7 and (sin - rs_).abs().max().item() <= 2.4e-7
        frac = ((cos != rc_) | (sin != rs_)).float().mean().item()
        assert frac < 0.05, frac
        # and against the CPU oracle's tables (what the parity tests use): angles above 2^24 ulp apart cannot occur here
        oc, os_ = oracle.precompute_freqs_cis(D, N, theta)
        assert (cos.cpu() - oc[:, : D // 2]).abs().max().item() < 5e-4 * max(1.0, N / 4096)


@pytest.mark.parametrize("dtype,shape", [(torch.bfloat16, (2, 3, 1024, 128)), (torch.float16, (1, 2, 512, 64)), (torch.float32, (1, 2, 200, 64)),
                                         (torch.bfloat16, (1, 2, 130, 32))])
def test_attention_theta_matches_table_path_and_oracle(dtype, shape):
    B, H, N, D = shape
    theta = 10000.0
    q, k, v, do = (draw(shape, 90 + i, dtype) for i in range(4))
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = attention_theta(qd, kd, vd, True, D ** -0.5, theta)
    o.backward(do.cuda())
    ext.check_status()
    got = tuple(t.detach().float().cpu() for t in (o, qd.grad, kd.grad, vd.grad))
    # against the table path fed with precompute_freqs_cis evaluated on the device
    import importlib
    fr = importlib.import_module("co-rope_b200.fused_rope_attn")
    ang = torch.outer(torch.arange(N, device="cuda", dtype=torch.float32), fr.inv_freq_of(theta, D, "cuda"))
    q2, k2, v2 = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o2 = pkg.fused_rope_attention(q2, k2, v2, True, D ** -0.5, torch.cos(ang), torch.sin(ang))
    o2.backward(do.cuda())
    ext.check_status()
    tab = tuple(t.detach().float().cpu() for t in (o2, q2.grad, k2.grad, v2.grad))
    tol = 1e-5 if dtype == torch.float32 else 2 ** -6   # 16-bit: a table entry on a rounding boundary may flip one output bit
    for a, b in zip(got, tab):
        assert maxdiff(a, b) <= tol
        assert (a != b).float().mean().item() < 0.02
    # and against the oracle
    cos, sin = oracle.precompute_freqs_cis(D, N, theta)
    refs = (oracle.rope_attn_fwd(q, k, v, True, D ** -0.5, cos, sin),) + tuple(oracle.rope_attn_bwd(q, k, v, do, True, D ** -0.5, cos, sin))
    if dtype == torch.float32:
        for a, b in zip(got, refs):
            assert maxdiff(a, b) < 2 * TOL_32
    else:
        check16(_label() + " O", got[0], refs[0], TOL_FWD_16, dtype, strict=True)
        for name, a, b in zip(("dQ", "dK", "dV"), got[1:], refs[1:]):
            check16(_label() + " " + name, a, b, TOL_BWD_16, dtype)
