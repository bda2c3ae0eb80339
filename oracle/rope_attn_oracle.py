"""CPU oracle: fused RoPE (half layout) attention, forward and backward, fp32.

TEST INFRASTRUCTURE ONLY -- never imported by the shipped package.

Restates fused-rope/rope_attn_pytorch.py of the reference:
  precompute_freqs_cis   <- rope_attn_pytorch.py:10-49
  apply_rotary_emb       <- rope_attn_pytorch.py:52-84
  rope_attn_fwd          <- rope_attn_pytorch.py:94-162  (_attention_pytorch.forward)
  rope_attn_bwd          <- rope_attn_pytorch.py:165-224 (_attention_pytorch.backward)
  rope_attn_fwd_bwd_chunked : the same arithmetic evaluated one block of query
      rows at a time (rows x all keys), so that N = 65536 needs O(rows * N)
      memory instead of O(N^2).

All inputs are upcast to fp32 first: the protocol is "same seeded values,
reference arithmetic in fp32".  Side output `lse2` is the row log-sum-exp of
the scaled scores in log2 units, the quantity the reference's fused kernel
keeps as `M` (fused_rope_attn.py:316).
"""

import math

import torch

LOG2E = 1.4426950408889634


def precompute_freqs_cis(dim, seq_len, theta, device="cpu"):
    """cos/sin tables in the "cat" layout [N, D] = [c | c]  (rope_attn_pytorch.py:26-49)."""
    assert dim % 2 == 0, f"dim must be even, got {dim}"
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, device=device).float() / dim))
    t = torch.arange(seq_len, device=device, dtype=torch.float32)
    ang = torch.outer(t, inv)
    c, s = torch.cos(ang), torch.sin(ang)
    return torch.cat([c, c], dim=-1), torch.cat([s, s], dim=-1)


def _full_tables(cos, sin, D):
    """Accept [N, D] (cat layout) or [N, D/2] tables; only columns [0, D/2) carry information."""
    cos = cos.float()
    sin = sin.float()
    h = D // 2
    c, s = cos[:, :h], sin[:, :h]
    return torch.cat([c, c], dim=-1), torch.cat([s, s], dim=-1)


def apply_rotary_emb(x, cos, sin):
    """x*cos + rotate_half(x)*sin with rotate_half([x1|x2]) = [-x2|x1]  (rope_attn_pytorch.py:52-84)."""
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    return x * cos + torch.cat((-x2, x1), dim=-1) * sin


def _softmax_rows(scores, causal_mask):
    """Safe softmax exactly as rope_attn_pytorch.py:124-151; returns (weights, lse_natural)."""
    if causal_mask is not None:
        scores = scores.masked_fill(causal_mask, float("-inf"))
    mx = scores.max(dim=-1, keepdim=True).values
    mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    ex = torch.exp(scores - mx)
    if causal_mask is not None:
        ex = ex.masked_fill(causal_mask, 0.0)
    sm = ex.sum(dim=-1, keepdim=True)
    w = ex / sm
    if causal_mask is not None:
        w = w.masked_fill(causal_mask, 0.0)
    return w, (mx + torch.log(sm)).squeeze(-1)


def rope_attn_fwd(q, k, v, causal, sm_scale, cos, sin, return_aux=False):
    """O = softmax(rot(Q) rot(K)^T * sm_scale [+ causal mask]) V in fp32  (rope_attn_pytorch.py:108-155)."""
    q, k, v = q.float(), k.float(), v.float()
    D = q.shape[-1]
    cos, sin = _full_tables(cos, sin, D)
    qr = apply_rotary_emb(q, cos, sin)
    kr = apply_rotary_emb(k, cos, sin)
    scores = torch.einsum("bhqd,bhkd->bhqk", qr, kr) * sm_scale
    mask = None
    if causal:
        N = q.shape[2]
        mask = torch.triu(torch.ones(N, N, dtype=torch.bool), diagonal=1)[None, None]
    w, lse = _softmax_rows(scores, mask)
    o = torch.einsum("bhqk,bhkd->bhqd", w, v)
    if return_aux:
        return o, lse * LOG2E, (qr, kr, w)
    return o


def rope_attn_bwd(q, k, v, do, causal, sm_scale, cos, sin):
    """dQ, dK, dV in fp32  (rope_attn_pytorch.py:187-222)."""
    D = q.shape[-1]
    _, _, (qr, kr, w) = rope_attn_fwd(q, k, v, causal, sm_scale, cos, sin, return_aux=True)
    cos, sin = _full_tables(cos, sin, D)
    v, do = v.float(), do.float()
    dv = torch.einsum("bhqk,bhqd->bhkd", w, do)
    dw = torch.einsum("bhqd,bhkd->bhqk", do, v)
    delta = (dw * w).sum(dim=-1, keepdim=True)
    ds = w * (dw - delta)
    if causal:
        N = q.shape[2]
        mask = torch.triu(torch.ones(N, N, dtype=torch.bool), diagonal=1)[None, None]
        ds = ds.masked_fill(mask, 0.0)
    dq = torch.einsum("bhqk,bhkd->bhqd", ds, kr) * sm_scale
    dk = torch.einsum("bhqk,bhqd->bhkd", ds, qr) * sm_scale
    dq = apply_rotary_emb(dq, cos, -sin)
    dk = apply_rotary_emb(dk, cos, -sin)
    return dq, dk, dv


def rope_attn_fwd_bwd_chunked(q, k, v, do, causal, sm_scale, cos, sin, rows=1024, row_blocks=None):
    """Row-blocked evaluation of the same arithmetic (rope_attn_pytorch.py:108-155, 187-222).

    Processes `rows` query rows at a time against the keys they can see.  When
    `row_blocks` (a list of block indices) is given, only those blocks are
    evaluated: O, lse2 and dQ are then valid for those rows only (others are
    NaN) and dK/dV are the partial sums over those rows.  `do` may be None
    (forward only).  Returns (o, lse2, dq, dk, dv).
    """
    q, k, v = q.float(), k.float(), v.float()
    B, H, N, D = q.shape
    cos, sin = _full_tables(cos, sin, D)
    qr = apply_rotary_emb(q, cos, sin)
    kr = apply_rotary_emb(k, cos, sin)
    o = torch.full_like(q, float("nan"))
    lse2 = torch.full((B, H, N), float("nan"))
    want_bwd = do is not None
    if want_bwd:
        do = do.float()
        dqr = torch.full_like(q, float("nan"))
        dkr = torch.zeros_like(k)
        dv = torch.zeros_like(v)
    nblk = (N + rows - 1) // rows
    blocks = range(nblk) if row_blocks is None else row_blocks
    for ib in blocks:
        r0, r1 = ib * rows, min(N, (ib + 1) * rows)
        kend = r1 if causal else N
        s = torch.einsum("bhqd,bhkd->bhqk", qr[:, :, r0:r1], kr[:, :, :kend]) * sm_scale
        mask = None
        if causal:
            ii = torch.arange(r0, r1)[:, None]
            jj = torch.arange(kend)[None, :]
            mask = (jj > ii)[None, None]
        w, lse = _softmax_rows(s, mask)
        o[:, :, r0:r1] = torch.einsum("bhqk,bhkd->bhqd", w, v[:, :, :kend])
        lse2[:, :, r0:r1] = lse * LOG2E
        if want_bwd:
            g = do[:, :, r0:r1]
            dv[:, :, :kend] += torch.einsum("bhqk,bhqd->bhkd", w, g)
            dw = torch.einsum("bhqd,bhkd->bhqk", g, v[:, :, :kend])
            delta = (dw * w).sum(dim=-1, keepdim=True)
            ds = w * (dw - delta)
            if mask is not None:
                ds = ds.masked_fill(mask, 0.0)
            dqr[:, :, r0:r1] = torch.einsum("bhqk,bhkd->bhqd", ds, kr[:, :, :kend]) * sm_scale
            dkr[:, :, :kend] += torch.einsum("bhqk,bhqd->bhkd", ds, qr[:, :, r0:r1]) * sm_scale
    if not want_bwd:
        return o, lse2, None, None, None
    dq = apply_rotary_emb(dqr, cos, -sin)
    dk = apply_rotary_emb(dkr, cos, -sin)
    return o, lse2, dq, dk, dv


def attention_flops(B, H, N, D, mode="fwd", causal=True):
    """FLOP convention of the reference's benchmark driver (bench_compare.py:61-86)."""
    f = 4.0 * B * H * N * N * D
    if causal:
        f *= 0.5
    if mode == "bwd":
        f *= 2.5
    elif mode == "fwd+bwd":
        f *= 3.5
    return f


def default_sm_scale(D):
    return 1.0 / math.sqrt(D)
