"""CPU oracle: plain (no RoPE) attention with grouped K / V heads, forward and backward, fp32.

TEST INFRASTRUCTURE ONLY -- never imported by the shipped package.

Restates assets/flashattn-gqa/attn_gqa_pytorch.py of the reference:
  attn_gqa_fwd   <- attn_gqa_pytorch.py:17-116  (_attention_pytorch.forward: K / V heads expanded over their group :29-46,
                    fp32 scores :50-54, triu -inf mask :57-61, safe softmax :65-95, fp32 P V :99-103)
  attn_gqa_bwd   <- attn_gqa_pytorch.py:118-190 (dV :154-158, dP :162, softmax backward :166-176, dQ :180, dK :184,
                    group sums :189-190)
  attn_gqa_fwd_bwd_chunked : the same arithmetic one block of query rows at a time.

Inputs are upcast to fp32 first ("same seeded values, reference arithmetic in fp32").  Query head h of a batch entry
reads K / V head h // group_size -- the heads of a group are adjacent, as in flash_attn_v2_triton.py:194-196.
"""

import torch

from .rope_attn_oracle import LOG2E, _softmax_rows


def _expand(x, G):
    """[B, Hkv, N, D] -> [B, Hkv * G, N, D] with every K / V head repeated for its group (attn_gqa_pytorch.py:40-46)."""
    if G == 1:
        return x
    B, Hkv, N, D = x.shape
    return x.view(B, Hkv, 1, N, D).expand(B, Hkv, G, N, D).reshape(B, Hkv * G, N, D)


def _group_sum(x, G):
    if G == 1:
        return x
    B, H, N, D = x.shape
    return x.view(B, H // G, G, N, D).sum(dim=2)


def attn_gqa_fwd(q, k, v, causal, sm_scale, return_aux=False):
    q, k, v = q.float(), k.float(), v.float()
    Hq, Hkv = q.shape[1], k.shape[1]
    if Hq % Hkv != 0:
        raise ValueError(f"Number of Q heads ({Hq}) must be divisible by KV heads ({Hkv}).")
    G = Hq // Hkv
    ke, ve = _expand(k, G), _expand(v, G)
    scores = torch.einsum("bhqd,bhkd->bhqk", q, ke) * sm_scale
    mask = None
    if causal:
        N = q.shape[2]
        mask = torch.triu(torch.ones(N, N, dtype=torch.bool), diagonal=1)[None, None]
    w, lse = _softmax_rows(scores, mask)
    o = torch.einsum("bhqk,bhkd->bhqd", w, ve)
    if return_aux:
        return o, lse * LOG2E, w
    return o


def attn_gqa_bwd(q, k, v, do, causal, sm_scale):
    q, k, v, do = q.float(), k.float(), v.float(), do.float()
    G = q.shape[1] // k.shape[1]
    _, _, w = attn_gqa_fwd(q, k, v, causal, sm_scale, return_aux=True)
    ke, ve = _expand(k, G), _expand(v, G)
    dv = torch.einsum("bhqk,bhqd->bhkd", w, do)
    dw = torch.einsum("bhqd,bhkd->bhqk", do, ve)
    delta = (dw * w).sum(dim=-1, keepdim=True)
    ds = w * (dw - delta)
    if causal:
        N = q.shape[2]
        ds = ds.masked_fill(torch.triu(torch.ones(N, N, dtype=torch.bool), diagonal=1)[None, None], 0.0)
    dq = torch.einsum("bhqk,bhkd->bhqd", ds, ke) * sm_scale
    dk = torch.einsum("bhqk,bhqd->bhkd", ds, q) * sm_scale
    return dq, _group_sum(dk, G), _group_sum(dv, G)


def attn_gqa_fwd_bwd_chunked(q, k, v, do, causal, sm_scale, rows=1024):
    """Row-blocked evaluation of the same arithmetic for lengths whose N x N matrices do not fit.  Returns (o, lse2, dq, dk, dv)."""
    q, k, v = q.float(), k.float(), v.float()
    B, Hq, N, D = q.shape
    G = Hq // k.shape[1]
    ke, ve = _expand(k, G), _expand(v, G)
    o = torch.empty_like(q)
    lse2 = torch.empty((B, Hq, N))
    want_bwd = do is not None
    if want_bwd:
        do = do.float()
        dq, dke, dve = torch.empty_like(q), torch.zeros_like(ke), torch.zeros_like(ve)
    for r0 in range(0, N, rows):
        r1 = min(N, r0 + rows)
        kend = r1 if causal else N
        s = torch.einsum("bhqd,bhkd->bhqk", q[:, :, r0:r1], ke[:, :, :kend]) * sm_scale
        mask = None
        if causal:
            mask = (torch.arange(kend)[None, :] > torch.arange(r0, r1)[:, None])[None, None]
        w, lse = _softmax_rows(s, mask)
        o[:, :, r0:r1] = torch.einsum("bhqk,bhkd->bhqd", w, ve[:, :, :kend])
        lse2[:, :, r0:r1] = lse * LOG2E
        if want_bwd:
            g = do[:, :, r0:r1]
            dve[:, :, :kend] += torch.einsum("bhqk,bhqd->bhkd", w, g)
            dw = torch.einsum("bhqd,bhkd->bhqk", g, ve[:, :, :kend])
            ds = w * (dw - (dw * w).sum(dim=-1, keepdim=True))
            if mask is not None:
                ds = ds.masked_fill(mask, 0.0)
            dq[:, :, r0:r1] = torch.einsum("bhqk,bhkd->bhqd", ds, ke[:, :, :kend]) * sm_scale
            dke[:, :, :kend] += torch.einsum("bhqk,bhqd->bhkd", ds, q[:, :, r0:r1]) * sm_scale
    if not want_bwd:
        return o, lse2, None, None, None
    return o, lse2, dq, _group_sum(dke, G), _group_sum(dve, G)
