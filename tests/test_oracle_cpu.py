"""Pins the CPU oracle: against the committed golden vectors (outputs of the reference's
own PyTorch functions), against the reference itself when a checkout is present, and
against the known-answer properties the reference's tests use."""

import glob
import importlib.util
import os

import numpy as np
import pytest
import torch

import oracle

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
# a checkout of the reference: COROPE_REFERENCE_ROOT, else a directory named "reference" beside this repository
REF = os.environ.get("COROPE_REFERENCE_ROOT",
                     os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))


def _t(a):
    return torch.from_numpy(np.asarray(a)).float()


@pytest.mark.parametrize("name", ["rope_a", "rope_b", "rope_c"])
def test_rope_oracle_matches_golden(name):
    g = np.load(os.path.join(GOLD, name + ".npz"))
    B, H, N, D, causal, _ = g["meta"].tolist()
    sm_scale, theta = g["scal"].tolist()
    q, k, v, do = (_t(g[x]) for x in ("q", "k", "v", "do"))
    cos, sin = oracle.precompute_freqs_cis(D, N, theta)
    assert torch.equal(cos, _t(g["cos"])) and torch.equal(sin, _t(g["sin"]))
    o = oracle.rope_attn_fwd(q, k, v, bool(causal), sm_scale, cos, sin)
    dq, dk, dv = oracle.rope_attn_bwd(q, k, v, do, bool(causal), sm_scale, cos, sin)
    assert (o - _t(g["o"])).abs().max() < 1e-6
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert (got - _t(g[key])).abs().max() < 2e-6, key
    # half-width tables are accepted and equivalent
    o2 = oracle.rope_attn_fwd(q, k, v, bool(causal), sm_scale, cos[:, : D // 2], sin[:, : D // 2])
    assert torch.equal(o, o2)
    # the row-blocked form is the same arithmetic
    oc, lse2, dqc, dkc, dvc = oracle.rope_attn_fwd_bwd_chunked(q, k, v, do, bool(causal), sm_scale, cos, sin, rows=32)
    assert (oc - _t(g["o"])).abs().max() < 2e-6
    for got, key in ((dqc, "dq"), (dkc, "dk"), (dvc, "dv")):
        assert (got - _t(g[key])).abs().max() < 5e-6, key
    _, lse_d, _ = oracle.rope_attn_fwd(q, k, v, bool(causal), sm_scale, cos, sin, return_aux=True)
    assert (lse2 - lse_d).abs().max() < 1e-5


@pytest.mark.parametrize("name", ["corope_a", "corope_b", "corope_c"])
def test_corope_oracle_matches_golden(name):
    g = np.load(os.path.join(GOLD, name + ".npz"))
    B, Hq, Hkv, N, D, _ = g["meta"].tolist()
    sm_scale, theta = g["scal"].tolist()
    q, k, v, do = (_t(g[x]) for x in ("q", "k", "v", "do"))
    o = oracle.corope_gqa_fwd(q, k, v, True, sm_scale, theta)
    dq, dk, dv = oracle.corope_gqa_bwd(q, k, v, do, True, sm_scale, theta)
    assert (o - _t(g["o"])).abs().max() < 2e-6
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert (got - _t(g[key])).abs().max() < 1e-5, key
    oc, lse2, ad, dqc, dkc, dvc = oracle.corope_gqa_fwd_bwd_chunked(q, k, v, do, sm_scale, theta, rows=16)
    assert (oc - _t(g["o"])).abs().max() < 5e-6
    for got, key in ((dqc, "dq"), (dkc, "dk"), (dvc, "dv")):
        assert (got - _t(g[key])).abs().max() < 2e-5, key
    _, lse_d, ad_d, _ = oracle.corope_gqa_fwd(q, k, v, True, sm_scale, theta, return_aux=True)
    assert (lse2 - lse_d).abs().max() < 1e-5 and (ad - ad_d).abs().max() < 1e-5


def test_every_golden_file_is_covered():
    names = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLD, "*.npz")))
    assert names == ["attn_gqa_a", "attn_gqa_b", "attn_gqa_c", "corope_a", "corope_b", "corope_c", "rope_a", "rope_b", "rope_c"]


def test_corope_manual_backward_equals_autograd():
    # the reference's own self-check (corope_attn_gqa_pytorch.py:305-363): B=2, Hq=4, Hkv=2, N=64, D=32, loss = out.sum()
    torch.manual_seed(42)
    B, H, N, D = 2, 4, 64, 32
    q = torch.randn(B, H, N, D, requires_grad=True)
    k = torch.randn(B, H // 2, N, D, requires_grad=True)
    v = torch.randn(B, H // 2, N, D, requires_grad=True)
    o = oracle.corope_gqa_fwd(q, k, v, True, D ** -0.5, 10000.0)
    o.sum().backward()
    dq, dk, dv = oracle.corope_gqa_bwd(q.detach(), k.detach(), v.detach(), torch.ones_like(o), True, D ** -0.5, 10000.0)
    assert (dq - q.grad).abs().max() < 1e-5
    assert (dk - k.grad).abs().max() < 1e-5
    assert (dv - v.grad).abs().max() < 1e-5


def test_rope_identity_tables_give_plain_attention():
    # the reference's test_op (fused_rope_attn.py:785-851) uses cos=1, sin=0
    torch.manual_seed(20)
    q, k, v = (torch.randn(1, 2, 128, 64) * 0.5 for _ in range(3))
    cos, sin = torch.ones(128, 64), torch.zeros(128, 64)
    o = oracle.rope_attn_fwd(q, k, v, True, 0.5, cos, sin)
    p = torch.matmul(q, k.transpose(2, 3)) * 0.5
    p = p.masked_fill(torch.triu(torch.ones(128, 128, dtype=torch.bool), 1), float("-inf"))
    ref = torch.matmul(torch.softmax(p, dim=-1), v)
    assert (o - ref).abs().max() < 1e-6
    assert torch.allclose(o[..., 0, :], v[..., 0, :])


def test_rope_is_relative():
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 1, 64, 32) for _ in range(3))
    cos, sin = oracle.precompute_freqs_cis(32, 64 + 7, 10000.0)
    o0 = oracle.rope_attn_fwd(q, k, v, True, 0.3, cos[:64], sin[:64])
    o1 = oracle.rope_attn_fwd(q, k, v, True, 0.3, cos[7:], sin[7:])
    assert (o0 - o1).abs().max() < 1e-5


def test_corope_rejects_non_causal_and_bad_groups():
    q = torch.zeros(1, 3, 8, 16)
    k = torch.zeros(1, 2, 8, 16)
    with pytest.raises(ValueError):
        oracle.corope_gqa_fwd(q, k, k, False, 1.0, 10000.0)
    with pytest.raises(ValueError):
        oracle.corope_gqa_fwd(q, k, k, True, 1.0, 10000.0)


def _load_ref(rel, name):
    path = os.path.join(REF, rel)
    if not os.path.exists(path):
        pytest.skip("reference checkout not present")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_rope_oracle_matches_live_reference():
    ref = _load_ref("fused-rope/rope_attn_pytorch.py", "ref_rope_live")
    torch.manual_seed(7)
    B, H, N, D = 2, 3, 200, 64
    q, k, v, do = (torch.randn(B, H, N, D) for _ in range(4))
    cos, sin = ref.precompute_freqs_cis(D, N, 10000.0, device="cpu")
    for causal in (True, False):
        qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = ref.attention_pytorch(qq, kk, vv, causal, 0.125, cos, sin)
        o.backward(do)
        oo = oracle.rope_attn_fwd(q, k, v, causal, 0.125, cos, sin)
        dq, dk, dv = oracle.rope_attn_bwd(q, k, v, do, causal, 0.125, cos, sin)
        assert (oo - o).abs().max() < 1e-6
        assert (dq - qq.grad).abs().max() < 5e-6
        assert (dk - kk.grad).abs().max() < 5e-6
        assert (dv - vv.grad).abs().max() < 5e-6


def test_corope_oracle_matches_live_reference():
    ref = _load_ref("corope-exp/corope_attn_gqa_pytorch.py", "ref_corope_live")
    torch.manual_seed(9)
    B, Hq, Hkv, N, D = 1, 8, 2, 80, 32
    q = torch.randn(B, Hq, N, D)
    k, v = torch.randn(B, Hkv, N, D), torch.randn(B, Hkv, N, D)
    do = torch.randn(B, Hq, N, D)
    qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
    o = ref.attention_pytorch(qq, kk, vv, True, D ** -0.5, 10000.0)
    o.backward(do)
    oo = oracle.corope_gqa_fwd(q, k, v, True, D ** -0.5, 10000.0)
    dq, dk, dv = oracle.corope_gqa_bwd(q, k, v, do, True, D ** -0.5, 10000.0)
    assert (oo - o).abs().max() < 2e-6
    assert (dq - qq.grad).abs().max() < 1e-5
    assert (dk - kk.grad).abs().max() < 1e-5
    assert (dv - vv.grad).abs().max() < 1e-5


@pytest.mark.parametrize("name", ["attn_gqa_a", "attn_gqa_b", "attn_gqa_c"])
def test_plain_gqa_oracle_matches_golden(name):
    # plain attention with grouped K / V heads: outputs of the reference's assets/flashattn-gqa/attn_gqa_pytorch.py
    g = np.load(os.path.join(GOLD, name + ".npz"))
    B, Hq, Hkv, N, D, causal, _ = g["meta"].tolist()
    (sm_scale,) = g["scal"].tolist()
    q, k, v, do = (_t(g[x]) for x in ("q", "k", "v", "do"))
    o = oracle.attn_gqa_fwd(q, k, v, bool(causal), sm_scale)
    dq, dk, dv = oracle.attn_gqa_bwd(q, k, v, do, bool(causal), sm_scale)
    assert (o - _t(g["o"])).abs().max() < 1e-6
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert got.shape == _t(g[key]).shape
        assert (got - _t(g[key])).abs().max() < 5e-6, key
    oc, lse2, dqc, dkc, dvc = oracle.attn_gqa_fwd_bwd_chunked(q, k, v, do, bool(causal), sm_scale, rows=16)
    assert (oc - _t(g["o"])).abs().max() < 2e-6
    for got, key in ((dqc, "dq"), (dkc, "dk"), (dvc, "dv")):
        assert (got - _t(g[key])).abs().max() < 1e-5, key
    # with the rotation by identity tables the fused-RoPE oracle must give the same (group size 1 only)
    if Hq == Hkv:
        o2 = oracle.rope_attn_fwd(q, k, v, bool(causal), sm_scale, torch.ones(N, D), torch.zeros(N, D))
        assert (o2 - o).abs().max() < 1e-6


def test_plain_gqa_oracle_matches_live_reference():
    path = os.path.join(REF, "assets", "flashattn-gqa", "attn_gqa_pytorch.py")
    if not os.path.exists(path):
        pytest.skip("no reference checkout")
    spec = importlib.util.spec_from_file_location("ref_attn_gqa_pytorch_live", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    gen = torch.Generator().manual_seed(77)
    q = torch.randn((2, 8, 48, 64), generator=gen)
    k, v = (torch.randn((2, 2, 48, 64), generator=gen) for _ in range(2))
    do = torch.randn((2, 8, 48, 64), generator=gen)
    for causal in (True, False):
        qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = ref.attention_pytorch(qq, kk, vv, causal, 0.3)
        o.backward(do)
        assert (oracle.attn_gqa_fwd(q, k, v, causal, 0.3) - o.detach()).abs().max() < 1e-6
        for got, want in zip(oracle.attn_gqa_bwd(q, k, v, do, causal, 0.3), (qq.grad, kk.grad, vv.grad)):
            assert (got - want).abs().max() < 5e-6
