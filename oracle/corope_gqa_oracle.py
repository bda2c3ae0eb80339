"""CPU oracle: context-aware Co-RoPE GQA attention, forward and backward, fp32.

TEST INFRASTRUCTURE ONLY -- never imported by the shipped package.

Restates corope-exp/corope_attn_gqa_pytorch.py of the reference:
  corope_gqa_fwd  <- corope_attn_gqa_pytorch.py:16-134  (_attention_pytorch.forward)
  corope_gqa_bwd  <- corope_attn_gqa_pytorch.py:138-300 (_attention_pytorch.backward)
  corope_gqa_fwd_bwd_chunked : the same arithmetic one block of query rows at a
      time, so the [Hq, N, N, D/2] temporaries become [rows, N, D/2].

Definition (line numbers of corope_attn_gqa_pytorch.py):
  G = Hq / Hkv, the leader of KV head g is query head g*G             (58)
  w_d   = theta^(-2d/D), d < D/2                                       (35)
  z_ik  = sigmoid(qL_i . k_k * s)                                      (59)
  a_ij  = sum_{k<=j} z_ik                                              (60)
  D_ij  = a_ii - a_ij                                                  (64)
  E_A   = q1 k1 + q2 k2,  E_B = q2 k1 - q1 k2   per (h, i, j, d)       (71-72)
  S_hij = s * sum_d (E_A cos(D_ij w_d) - E_B sin(D_ij w_d))            (74-78)
  causal mask, safe softmax, O = P V with V of the group's KV head     (81-124)
Inputs are upcast to fp32 first.
"""

import torch

LOG2E = 1.4426950408889634


def corope_inv_freq(D, theta):
    return 1.0 / (theta ** (torch.arange(0, D, 2).float() / D))


def _softmax_rows(scores, mask):
    scores = scores.masked_fill(mask, float("-inf"))
    mx = scores.max(dim=-1, keepdim=True).values
    mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    ex = torch.exp(scores - mx).masked_fill(mask, 0.0)
    sm = ex.sum(dim=-1, keepdim=True)
    w = (ex / sm).masked_fill(mask, 0.0)
    return w, (mx + torch.log(sm)).squeeze(-1)


def _dense_parts(q, k, sm_scale, theta):
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    if Hq % Hkv != 0:
        raise ValueError(f"Number of Q heads ({Hq}) must be divisible by KV heads ({Hkv}).")
    G = Hq // Hkv
    inv_freq = corope_inv_freq(D, theta)
    k_e = k.repeat_interleave(G, dim=1)
    qL = q[:, ::G]
    z = torch.sigmoid(torch.einsum("bhqd,bhkd->bhqk", qL, k) * sm_scale)
    a_leader = torch.cumsum(z, dim=-1)
    a = a_leader.repeat_interleave(G, dim=1)
    delta_a = torch.diagonal(a, dim1=-2, dim2=-1).unsqueeze(-1) - a
    h = D // 2
    q1, q2 = q[..., :h], q[..., h:]
    k1, k2 = k_e[..., :h], k_e[..., h:]
    E_A = q1.unsqueeze(3) * k1.unsqueeze(2) + q2.unsqueeze(3) * k2.unsqueeze(2)
    E_B = q2.unsqueeze(3) * k1.unsqueeze(2) - q1.unsqueeze(3) * k2.unsqueeze(2)
    phi = delta_a.unsqueeze(-1) * inv_freq.view(1, 1, 1, 1, -1)
    return G, inv_freq, z, a_leader, E_A, E_B, torch.cos(phi), torch.sin(phi)


def corope_gqa_fwd(q, k, v, causal, sm_scale, theta, return_aux=False):
    """Dense forward (corope_attn_gqa_pytorch.py:28-124).  q [B,Hq,N,D]; k, v [B,Hkv,N,D]."""
    if not causal:
        raise ValueError("CoRoPE PyTorch implementation supports causal=True only.")
    q, k, v = q.float(), k.float(), v.float()
    N = q.shape[2]
    G, inv_freq, z, a_leader, E_A, E_B, c, s = _dense_parts(q, k, sm_scale, theta)
    scores = (E_A * c - E_B * s).sum(dim=-1) * sm_scale
    mask = torch.triu(torch.ones(N, N, dtype=torch.bool), diagonal=1)[None, None]
    w, lse = _softmax_rows(scores, mask)
    o = torch.einsum("bhqk,bhkd->bhqd", w, v.repeat_interleave(G, dim=1))
    if return_aux:
        a_diag = torch.diagonal(a_leader, dim1=-2, dim2=-1)
        return o, lse * LOG2E, a_diag, w
    return o


def corope_gqa_bwd(q, k, v, do, causal, sm_scale, theta):
    """Dense backward (corope_attn_gqa_pytorch.py:161-298).  Returns dq [B,Hq,N,D], dk, dv [B,Hkv,N,D]."""
    if not causal:
        raise ValueError("CoRoPE PyTorch implementation supports causal=True only.")
    q, k, v, do = q.float(), k.float(), v.float(), do.float()
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    h = D // 2
    G, inv_freq, z, a_leader, E_A, E_B, c, s = _dense_parts(q, k, sm_scale, theta)
    mask = torch.triu(torch.ones(N, N, dtype=torch.bool), diagonal=1)[None, None]
    scores = (E_A * c - E_B * s).sum(dim=-1) * sm_scale
    w, _ = _softmax_rows(scores, mask)
    v_e = v.repeat_interleave(G, dim=1)
    k_e = k.repeat_interleave(G, dim=1)
    dw = torch.einsum("bhqd,bhkd->bhqk", do, v_e)
    dv_e = torch.einsum("bhqk,bhqd->bhkd", w, do)
    dsum = (dw * w).sum(dim=-1, keepdim=True)
    dp = (w * (dw - dsum)).masked_fill(mask, 0.0)
    gT = (dp * sm_scale).unsqueeze(-1)
    gEA = gT * c
    gEB = gT * (-s)
    gphi = gT * (-E_A * s - E_B * c)
    q1, q2 = q[..., :h], q[..., h:]
    k1, k2 = k_e[..., :h], k_e[..., h:]
    dq1 = torch.einsum("bhqkd,bhkd->bhqd", gEA, k1) + torch.einsum("bhqkd,bhkd->bhqd", -gEB, k2)
    dq2 = torch.einsum("bhqkd,bhkd->bhqd", gEA, k2) + torch.einsum("bhqkd,bhkd->bhqd", gEB, k1)
    dk1 = torch.einsum("bhqkd,bhqd->bhkd", gEA, q1) + torch.einsum("bhqkd,bhqd->bhkd", gEB, q2)
    dk2 = torch.einsum("bhqkd,bhqd->bhkd", gEA, q2) + torch.einsum("bhqkd,bhqd->bhkd", -gEB, q1)
    g_delta = (gphi * inv_freq.view(1, 1, 1, 1, -1)).sum(dim=-1)
    g_a = torch.diag_embed(g_delta.sum(dim=-1)) - g_delta
    g_aL = g_a.view(B, Hkv, G, N, N).sum(dim=2)
    g_z = torch.cumsum(g_aL.flip(-1), dim=-1).flip(-1)
    g_raw = g_z * z * (1.0 - z) * sm_scale
    qL = q[:, ::G]
    dq = torch.zeros_like(q)
    dq[:, ::G] = torch.einsum("bhqk,bhkd->bhqd", g_raw, k)
    dk_raw = torch.einsum("bhqk,bhqd->bhkd", g_raw, qL)
    dq[..., :h] += dq1
    dq[..., h:] += dq2
    dk_e = torch.cat([dk1, dk2], dim=-1)
    dk = dk_raw + dk_e.view(B, Hkv, G, N, D).sum(dim=2)
    dv = dv_e.view(B, Hkv, G, N, D).sum(dim=2)
    return dq, dk, dv


def corope_gqa_fwd_bwd_chunked(q, k, v, do, sm_scale, theta, rows=64, row_blocks=None):
    """Row-blocked evaluation of corope_attn_gqa_pytorch.py:56-124 and 182-298.

    One (batch, KV head) unit and one block of `rows` query rows at a time;
    temporaries are [G, rows, keys, D/2].  With `row_blocks` only those blocks
    are evaluated (O / lse2 / a_diag / dQ valid on those rows, NaN elsewhere;
    dK / dV are partial sums over those rows).  `do` may be None.
    Returns (o, lse2, a_diag, dq, dk, dv).
    """
    q, k, v = q.float(), k.float(), v.float()
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    if Hq % Hkv != 0:
        raise ValueError(f"Number of Q heads ({Hq}) must be divisible by KV heads ({Hkv}).")
    G = Hq // Hkv
    h = D // 2
    w_d = corope_inv_freq(D, theta)
    o = torch.full_like(q, float("nan"))
    lse2 = torch.full((B, Hq, N), float("nan"))
    a_diag = torch.full((B, Hkv, N), float("nan"))
    want_bwd = do is not None
    if want_bwd:
        do = do.float()
        dq = torch.full_like(q, float("nan"))
        dk = torch.zeros_like(k)
        dv = torch.zeros_like(v)
    nblk = (N + rows - 1) // rows
    blocks = range(nblk) if row_blocks is None else row_blocks
    for b in range(B):
        for g in range(Hkv):
            kk, vv = k[b, g], v[b, g]
            k1, k2 = kk[:, :h], kk[:, h:]
            for ib in blocks:
                r0, r1 = ib * rows, min(N, (ib + 1) * rows)
                ke = r1
                ii = torch.arange(r0, r1)
                mask = torch.arange(ke)[None, :] > ii[:, None]
                qg = q[b, g * G:(g + 1) * G, r0:r1]                       # [G, R, D]
                qL = qg[0]
                z = torch.sigmoid(qL @ kk[:ke].T * sm_scale)               # [R, ke]
                a = torch.cumsum(z, dim=-1)
                ad = a[torch.arange(r1 - r0), ii]
                a_diag[b, g, r0:r1] = ad
                dlt = ad[:, None] - a                                      # [R, ke]
                phi = dlt[:, :, None] * w_d[None, None, :]
                c, s = torch.cos(phi), torch.sin(phi)                      # [R, ke, h]
                q1, q2 = qg[..., :h], qg[..., h:]                          # [G, R, h]
                E_A = q1[:, :, None, :] * k1[None, None, :ke] + q2[:, :, None, :] * k2[None, None, :ke]
                E_B = q2[:, :, None, :] * k1[None, None, :ke] - q1[:, :, None, :] * k2[None, None, :ke]
                sc = (E_A * c[None] - E_B * s[None]).sum(dim=-1) * sm_scale  # [G, R, ke]
                w, lse = _softmax_rows(sc, mask[None])
                o[b, g * G:(g + 1) * G, r0:r1] = w @ vv[:ke]
                lse2[b, g * G:(g + 1) * G, r0:r1] = lse * LOG2E
                if not want_bwd:
                    continue
                gO = do[b, g * G:(g + 1) * G, r0:r1]                       # [G, R, D]
                dv[b, g, :ke] += torch.einsum("grk,grd->kd", w, gO)
                dw = gO @ vv[:ke].T
                dsum = (dw * w).sum(dim=-1, keepdim=True)
                dp = (w * (dw - dsum)).masked_fill(mask[None], 0.0)
                gT = (dp * sm_scale)[..., None]                            # [G, R, ke, 1]
                gEA = gT * c[None]
                gEB = gT * (-s[None])
                gphi = gT * (-E_A * s[None] - E_B * c[None])
                dq1 = torch.einsum("grkd,kd->grd", gEA, k1[:ke]) - torch.einsum("grkd,kd->grd", gEB, k2[:ke])
                dq2 = torch.einsum("grkd,kd->grd", gEA, k2[:ke]) + torch.einsum("grkd,kd->grd", gEB, k1[:ke])
                dk1 = torch.einsum("grkd,grd->kd", gEA, q1) + torch.einsum("grkd,grd->kd", gEB, q2)
                dk2 = torch.einsum("grkd,grd->kd", gEA, q2) - torch.einsum("grkd,grd->kd", gEB, q1)
                g_delta = (gphi * w_d.view(1, 1, 1, -1)).sum(dim=-1).sum(dim=0)  # [R, ke], group-summed
                g_a = -g_delta
                g_a[torch.arange(r1 - r0), ii] += g_delta.sum(dim=-1)
                g_z = torch.cumsum(g_a.flip(-1), dim=-1).flip(-1)
                g_raw = g_z * z * (1.0 - z) * sm_scale
                dqb = torch.cat([dq1, dq2], dim=-1)
                dqb[0] += g_raw @ kk[:ke]
                dq[b, g * G:(g + 1) * G, r0:r1] = dqb
                dk[b, g, :ke] += torch.cat([dk1, dk2], dim=-1) + g_raw.T @ qL
    if not want_bwd:
        return o, lse2, a_diag, None, None, None
    return o, lse2, a_diag, dq, dk, dv
