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


_MANT_BITS = {torch.bfloat16: 7, torch.float16: 10, torch.float32: 23}   # stored significand bits


def excess(got, ref, abs_tol, dtype):
    """Largest amount by which |got - ref| exceeds the allowed error, over all elements (<= 0 means pass).

    The allowed error is `abs_tol`, or one unit in the last place of the output dtype at the reference value where that
    is larger: ulp(x) = 2^(floor(log2 |x|) - stored significand bits).  For bf16 that is 2^-5 = 0.031 for |x| in [4, 8), the
    first binade in which it exceeds the gradients' 2e-2 (rounding the exact result to bf16 alone costs up to half of
    it), so only outputs of magnitude >= 4 (>= 2 for the forward's 1e-2) ever get the allowance."""
    ref = ref.float()
    ulp = torch.exp2(torch.floor(torch.log2(ref.abs().clamp_min(1e-30))) - _MANT_BITS[dtype])
    allowed = torch.clamp(ulp, min=abs_tol)
    return ((got.float() - ref).abs() - allowed).max().item()

REPORT_PATH = os.environ.get("COROPE_PARITY_REPORT", os.path.join(os.path.dirname(os.path.abspath(__file__)), "_report", "parity_report.jsonl"))


def check16(label, got, ref, abs_tol, dtype, strict=False):
    """Parity check of a 16-bit result that also puts the plain numbers on record.

    Always measured: the strict max-abs error and how many elements exceed the absolute tolerance (i.e. needed the
    one-ulp allowance of `excess`).  With strict=True the strict max-abs itself must be within `abs_tol`; otherwise the
    bound is `excess`'s (absolute tolerance, or one ulp of the output dtype where that is larger).  One JSON line per
    call is appended to REPORT_PATH so that a run leaves the strict figures behind, not only pass / fail."""
    import json

    d = (got.float() - ref.float()).abs()
    strict_max = d.max().item()
    n_over = int((d > abs_tol).sum().item())
    exc = excess(got, ref, abs_tol, dtype)
    try:
        os.makedirs(os.path.dirname(REPORT_PATH), exist_ok=True)
        with open(REPORT_PATH, "a") as f:
            f.write(json.dumps({"case": label, "dtype": str(dtype).replace("torch.", ""), "abs_tol": abs_tol, "strict_max_abs": strict_max,
                                "n_over_abs_tol": n_over, "numel": d.numel(), "max_abs_ref": ref.float().abs().max().item(),
                                "asserted": "strict" if strict else "abs_tol_or_one_ulp"}) + "\n")
    except OSError:
        pass
    if strict:
        assert strict_max <= abs_tol, "%s: strict max-abs %.5f > %.5f" % (label, strict_max, abs_tol)
    else:
        assert exc <= 0, "%s: max-abs %.5f, %d elements beyond %.0e and beyond one ulp by up to %.5f" % (label, strict_max, n_over, abs_tol, exc)


def check16_all(label, outs, refs, tol_fwd, tol_bwd, dtype):
    """O strictly within tol_fwd; dQ, dK, dV within tol_bwd or one ulp.  `outs` / `refs` = (o, dq, dk, dv)."""
    check16(label + " O", outs[0], refs[0], tol_fwd, dtype, strict=True)
    for name, got, ref in zip(("dQ", "dK", "dV"), outs[1:], refs[1:]):
        check16(label + " " + name, got, ref, tol_bwd, dtype)
