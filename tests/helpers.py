"""Shared helpers for the parity tests: package import, seeded inputs, oracle calls."""

import importlib
import os

import numpy as np
import torch

import oracle

pkg = importlib.import_module("co-rope_b200")
ext = pkg._ext
fused_attention = pkg.fused_rope_attention
corope_attention = pkg.corope_gqa_attention

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_gold(name):
    g = np.load(os.path.join(GOLD, name + ".npz"))
    return {k: g[k] for k in g.files}


def draw(shape, seed, dtype):
    """Seeded N(0,1) drawn in fp32 on the CPU, then cast to the test dtype (returned on the CPU)."""
    gen = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=gen, dtype=torch.float32).to(dtype)


def rope_inputs(B, H, N, D, dtype, seed=0):
    q, k, v, do = (draw((B, H, N, D), seed * 4 + i, dtype) for i in range(4))
    return q, k, v, do


def run_fused(q, k, v, do, causal, sm_scale, cos, sin, device="cuda"):
    """Forward (+ backward when do is given) through the drop-in entry point; results on the CPU in fp32."""
    qd, kd, vd = (t.to(device).requires_grad_(True) for t in (q, k, v))
    o = fused_attention(qd, kd, vd, causal, sm_scale, cos.to(device), sin.to(device))
    if do is None:
        ext.check_status()
        return o.detach().float().cpu(), None, None, None
    o.backward(do.to(device))
    ext.check_status()
    return tuple(t.detach().float().cpu() for t in (o, qd.grad, kd.grad, vd.grad))


def run_corope(q, k, v, do, sm_scale, theta, device="cuda"):
    qd, kd, vd = (t.to(device).requires_grad_(True) for t in (q, k, v))
    o = corope_attention(qd, kd, vd, True, sm_scale, theta)
    if do is None:
        ext.check_status()
        return o.detach().float().cpu(), None, None, None
    o.backward(do.to(device))
    ext.check_status()
    return tuple(t.detach().float().cpu() for t in (o, qd.grad, kd.grad, vd.grad))


def maxdiff(a, b):
    return (a.float() - b.float()).abs().max().item()


_ULP = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -23}


def excess(got, ref, abs_tol, dtype):
    """Largest amount by which |got - ref| exceeds the allowed error, over all elements (<= 0 means pass).

    The allowed error is `abs_tol`, or one unit in the last place of the output dtype at the reference
    value where that is larger: a bf16 result of magnitude >= 4 cannot be closer than 2^-7 to an arbitrary
    fp32 reference value, so a pure absolute bound below that is unattainable there by any kernel."""
    ref = ref.float()
    allowed = torch.clamp(ref.abs() * _ULP[dtype], min=abs_tol)
    return ((got.float() - ref).abs() - allowed).max().item()
