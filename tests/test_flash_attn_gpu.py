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


# ---------------------------------------------------------------------------------------------------------------------
# strided tensors: the kernels take every tensor's own {batch, head, row} strides
# ---------------------------------------------------------------------------------------------------------------------
def _as_bnhd_view(t):
    """The same values held in a [B, N, H, D] buffer and viewed as [B, H, N, D] (what a projection followed by
    .view(B, N, H, D).transpose(1, 2) gives a model)."""
    return t.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)


def _padded_rows_view(t, pad):
    """The same values with `pad` unused elements behind every row (row stride D + pad)."""
    B, H, N, D = t.shape
    buf = torch.zeros((B, H, N, D + pad), dtype=t.dtype, device=t.device)
    buf[..., :D] = t
    return buf[..., :D]


@pytest.mark.parametrize("dtype,shape,causal", [(torch.bfloat16, (2, 4, 512, 128), True), (torch.float16, (1, 3, 256, 64), False),
                                                (torch.float32, (2, 2, 100, 64), True), (torch.bfloat16, (1, 2, 200, 32), True)])
@pytest.mark.parametrize("layout", ["bnhd", "padded8", "padded2"])
def test_fused_rope_strided_views_need_no_copies(dtype, shape, causal, layout):
    # Transposed and row-padded views through the drop-in entry point: same results as contiguous tensors, the outputs
    # come back in the inputs' layout (o = empty_like(q), fused_rope_attn.py:662), and the library launches exactly the
    # kernels it launches for contiguous tensors -- no copy kernels of its own, and torch makes none either.
    # "padded2" (row stride D + 2) is not a multiple of 16 bytes for 16-bit types: those run on the CUDA-core kernels.
    B, H, N, D = shape
    q, k, v, do = (draw(shape, 100 + i, dtype).cuda() for i in range(4))
    cos, sin = (t.cuda() for t in oracle.precompute_freqs_cis(D, N, 10000.0))
    view = {"bnhd": _as_bnhd_view, "padded8": lambda t: _padded_rows_view(t, 8), "padded2": lambda t: _padded_rows_view(t, 2)}[layout]

    def run(make):
        qq, kk, vv = (make(t).detach().requires_grad_(True) for t in (q, k, v))
        n0 = ext.lib().corope_launch_count()
        o = pkg.fused_rope_attention(qq, kk, vv, causal, D ** -0.5, cos, sin)
        o.backward(make(do))
        ext.check_status()
        return (o, qq.grad, kk.grad, vv.grad), (qq, kk, vv), ext.lib().corope_launch_count() - n0

    ref, _, launches_contig = run(lambda t: t.clone())
    fam_contig = (ext.lib().corope_last_kernel_family(ext.OP_ROPE_FWD), ext.lib().corope_last_kernel_family(ext.OP_ROPE_BWD))
    got, (qq, kk, vv), launches = run(view)
    fam = (ext.lib().corope_last_kernel_family(ext.OP_ROPE_FWD), ext.lib().corope_last_kernel_family(ext.OP_ROPE_BWD))
    assert not qq.is_contiguous()
    # outputs and gradients are laid out as torch.empty_like lays them out: the input's own strides for a dense view (the
    # transposed buffer), contiguous for a view with gaps (the padded rows)
    want = torch.empty_like(qq).stride()
    assert got[0].stride() == want and got[1].stride() == want and got[2].stride() == torch.empty_like(kk).stride()
    if layout == "bnhd":
        assert want == qq.stride() and not got[0].is_contiguous()
    aligned = dtype == torch.float32 or layout != "padded2"
    if aligned:
        assert fam == fam_contig and launches == launches_contig
        assert torch.equal(got[0], ref[0]) and torch.equal(got[2], ref[2]) and torch.equal(got[3], ref[3])   # fixed summation order
        assert maxdiff(got[1], ref[1]) < 1e-2
    else:
        assert fam == (0, 0)
        for a, b, tol in zip(got, ref, (TOL_FWD_16, TOL_BWD_16, TOL_BWD_16, TOL_BWD_16)):
            assert maxdiff(a, b) <= 2 * tol


def test_flash_attention_strided_gqa_views():
    B, Hq, Hkv, N, D = 2, 8, 2, 384, 128
    q, k, v, do = (t.cuda() for t in _inputs(B, Hq, Hkv, N, D, torch.bfloat16, 110))
    qq, kk, vv = (_as_bnhd_view(t).detach().requires_grad_(True) for t in (q, k, v))
    o = flash_attention(qq, kk, vv, True, D ** -0.5)
    o.backward(_as_bnhd_view(do))
    ext.check_status()
    assert ext.lib().corope_last_kernel_family(ext.OP_ROPE_FWD) == 1 and ext.lib().corope_last_kernel_family(ext.OP_ROPE_BWD) == 1
    assert o.stride() == qq.stride() and kk.grad.stride() == kk.stride()
    qc, kc, vc, dc = (t.float().cpu() for t in (q, k, v, do))
    refs = (oracle.attn_gqa_fwd(qc, kc, vc, True, D ** -0.5),) + tuple(oracle.attn_gqa_bwd(qc, kc, vc, dc, True, D ** -0.5))
    check16(_label() + " O", o.detach().float().cpu(), refs[0], TOL_FWD_16, torch.bfloat16, strict=True)
    for name, got, ref in zip(("dQ", "dK", "dV"), (qq.grad, kk.grad, vv.grad), refs[1:]):
        check16(_label() + " " + name, got.float().cpu(), ref, TOL_BWD_16, torch.bfloat16)


@pytest.mark.parametrize("dtype,cfg", [(torch.bfloat16, (2, 8, 2, 256, 128)), (torch.float16, (1, 3, 1, 192, 128)),
                                       (torch.float32, (1, 4, 2, 100, 64)), (torch.bfloat16, (1, 2, 1, 96, 64))])
@pytest.mark.parametrize("layout", ["bnhd", "padded8", "padded2"])
def test_corope_strided_views_need_no_copies(dtype, cfg, layout):
    # Co-RoPE through its drop-in entry point on transposed and row-padded views: the results of contiguous tensors, the
    # same kernel family and launch count (no copy kernels), outputs laid out like the inputs.  A K / V row stride that
    # is not a multiple of 16 bytes ("padded2" in 16 bits) keeps D = 128 off the tensor-core kernels, whose pre-pass
    # reads 16-byte vectors.
    from helpers import corope_attention
    B, Hq, Hkv, N, D = cfg
    q, do = (draw((B, Hq, N, D), 120 + i, dtype).cuda() for i in range(2))
    k, v = (draw((B, Hkv, N, D), 122 + i, dtype).cuda() for i in range(2))
    view = {"bnhd": _as_bnhd_view, "padded8": lambda t: _padded_rows_view(t, 8), "padded2": lambda t: _padded_rows_view(t, 2)}[layout]

    def run(make):
        qq, kk, vv = (make(t).detach().requires_grad_(True) for t in (q, k, v))
        n0 = ext.lib().corope_launch_count()
        o = corope_attention(qq, kk, vv, True, D ** -0.5, 10000.0)
        o.backward(make(do))
        ext.check_status()
        fam = (ext.lib().corope_last_kernel_family(ext.OP_GQA_FWD), ext.lib().corope_last_kernel_family(ext.OP_GQA_BWD))
        return (o, qq.grad, kk.grad, vv.grad), (qq, kk, vv), ext.lib().corope_launch_count() - n0, fam

    ref, _, launches_contig, fam_contig = run(lambda t: t.clone())
    got, (qq, kk, vv), launches, fam = run(view)
    assert not qq.is_contiguous()
    assert got[0].stride() == torch.empty_like(qq).stride() and got[2].stride() == torch.empty_like(kk).stride()
    if layout == "bnhd":
        assert got[0].stride() == qq.stride() and not got[0].is_contiguous()
    tolf, tolb = (1e-4, 1e-3) if dtype == torch.float32 else (TOL_FWD_16, TOL_BWD_16)
    if dtype == torch.float32 or D != 128 or layout != "padded2":
        assert fam == fam_contig and launches == launches_contig
        assert torch.equal(got[0], ref[0])
        for a, b in zip(got[1:], ref[1:]):      # dK / dV are summed with atomics: order varies from run to run
            assert maxdiff(a, b) <= tolb
    else:
        assert fam_contig == (1, 1) and fam == (0, 0)   # the CUDA-core kernels: compared with the oracle below
    # and against the oracle on the same values
    qc, kc, vc, dc = (t.float().cpu() for t in (q, k, v, do))
    refs = (oracle.corope_gqa_fwd(qc, kc, vc, True, D ** -0.5, 10000.0),) + tuple(oracle.corope_gqa_bwd(qc, kc, vc, dc, True, D ** -0.5, 10000.0))
    for name, a, b, tol in zip(("O", "dQ", "dK", "dV"), got, refs, (tolf, tolb, tolb, tolb)):
        if dtype == torch.float32:
            assert maxdiff(a.float().cpu(), b) <= tol, name
        else:
            check16(_label() + " " + name, a.float().cpu(), b, tol, dtype, strict=(name == "O"))


def test_strided_entry_point_rejects_bad_strides():
    lib = ext.lib()
    t = torch.zeros(1, 1, 128, 128, device="cuda", dtype=torch.bfloat16)
    st = ext.strides_of(q=t, k=t, v=t, o=t)
    st.q[2] = 64   # row stride smaller than D
    f = torch.zeros(128, 64, device="cuda")
    ws, nbytes = ext.workspace(ext.OP_ROPE_FWD, 1, 1, 1, 128, 128, torch.bfloat16, t.device)
    rc = lib.corope_rope_attn_fwd_strided(t.data_ptr(), t.data_ptr(), t.data_ptr(), f.data_ptr(), f.data_ptr(), 64, t.data_ptr(), f.data_ptr(),
                                          1, 1, 128, 128, 1, 1, 0.1, ws.data_ptr(), nbytes, None, None, st)
    assert rc == -11 and b"stride" in lib.corope_status_string(rc)
    ws, nbytes = ext.workspace(ext.OP_GQA_FWD, 1, 1, 1, 128, 128, torch.bfloat16, t.device)
    g = torch.zeros(128, device="cuda")
    rc = lib.corope_gqa_fwd_strided(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), g.data_ptr(), g.data_ptr(), 1, 1, 1, 128, 128, 1,
                                    0.1, 10000.0, ws.data_ptr(), nbytes, None, None, st)
    assert rc == -11
