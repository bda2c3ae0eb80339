"""Drop-in for the reference's Co-RoPE GQA entry point
(corope-exp/flash_attn_co_rope_gqa_triton.py:403-580; the module keeps the reference's name so its scripts
can import this one unchanged).

    attention(q, k, v, causal, sm_scale, theta, warp_specialize=False) -> o

q: [B, Hq, N, D]; k, v: [B, Hkv, N, D]; Hq % Hkv == 0 and group size <= 8; causal must be True.
The math is that of corope-exp/corope_attn_gqa_pytorch.py; forward and backward are CUDA kernels reached
through the C ABI in include/corope_b200.h (the reference's backward is dense PyTorch).

Device-side errors (an expired bounded wait; a gradient term beyond the value range of the 16-bit backward) set a
per-device status word; every call first looks at a pinned host mirror of it and raises RuntimeError if an earlier
call set it (see fused_rope_attn.py).
"""

import torch

try:
    from . import _ext
except ImportError:
    import _ext


def _forward(q, k, v, causal, sm_scale, theta):
    """Checks + one corope_gqa_fwd call.  Returns what the backward needs: (q, k, v, o, lse2, a_diag)."""
    # same checks and messages as flash_attn_co_rope_gqa_triton.py:407-425
    if not causal:
        raise ValueError("CoRoPE fused kernel supports causal=True only.")
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("Expected q, k, v to have shape (batch, heads, seqlen, dim).")
    if k.shape != v.shape:
        raise ValueError("k and v must share the same shape in GQA.")
    if q.shape[0] != k.shape[0] or q.shape[2] != k.shape[2] or q.shape[3] != k.shape[3]:
        raise ValueError("k must align with q along batch/sequence/head_dim.")
    BATCH, H_Q, N_CTX, HEAD_DIM = q.shape
    H_KV = k.shape[1]
    if H_Q % H_KV != 0:
        raise ValueError("Number of query heads must be divisible by KV heads.")
    group_size = H_Q // H_KV
    if group_size > 8:
        raise ValueError(f"CoRoPE backbone currently limits group_size <= 8 (got {group_size}).")
    if not (q.dtype == k.dtype == v.dtype) or q.dtype not in _ext.DTYPE_CODES:
        raise ValueError("q, k, v must share one dtype out of float32, bfloat16, float16.")
    for t in (q, k, v):
        _ext.require_cuda(t)
    qc, kc, vc = _ext.kernel_layout(q), _ext.kernel_layout(k), _ext.kernel_layout(v)   # own strides, no copies
    o = torch.empty_like(qc)
    lse2 = torch.empty((BATCH, H_Q, N_CTX), device=q.device, dtype=torch.float32)
    a_diag = torch.empty((BATCH, H_KV, N_CTX), device=q.device, dtype=torch.float32)
    ws, ws_bytes = _ext.workspace(_ext.OP_GQA_FWD, BATCH, H_Q, H_KV, N_CTX, HEAD_DIM, q.dtype, q.device)
    st = _ext.strides_of(q=qc, k=kc, v=vc, o=o)
    _ext.pre_call(q.device)
    with torch.cuda.device(q.device):
        rc = _ext.lib().corope_gqa_fwd_strided(
            qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), lse2.data_ptr(), a_diag.data_ptr(),
            BATCH, H_Q, H_KV, N_CTX, HEAD_DIM, _ext.DTYPE_CODES[q.dtype], float(sm_scale), float(theta),
            ws.data_ptr(), ws_bytes, _ext.status_word(q.device).data_ptr(), _ext.stream_ptr(q.device), st)
    _ext.raise_for_status(rc, "corope_gqa_fwd")
    _ext.post_call(q.device)
    return qc, kc, vc, o, lse2, a_diag


def _backward(q, k, v, o, lse2, a_diag, grad_output, sm_scale, theta):
    """One corope_gqa_bwd call on what _forward returned.  Returns (dq, dk, dv); dk / dv are summed over each group."""
    grad_output = _ext.kernel_layout(grad_output)
    BATCH, H_Q, N_CTX, HEAD_DIM = q.shape
    H_KV = k.shape[1]
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    ws, ws_bytes = _ext.workspace(_ext.OP_GQA_BWD, BATCH, H_Q, H_KV, N_CTX, HEAD_DIM, q.dtype, q.device)
    st = _ext.strides_of(q=q, k=k, v=v, o=o, d_o=grad_output, dq=dq, dk=dk, dv=dv)
    _ext.pre_call(q.device)
    with torch.cuda.device(q.device):
        rc = _ext.lib().corope_gqa_bwd_strided(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), grad_output.data_ptr(), lse2.data_ptr(),
            a_diag.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            BATCH, H_Q, H_KV, N_CTX, HEAD_DIM, _ext.DTYPE_CODES[q.dtype], float(sm_scale), float(theta),
            ws.data_ptr(), ws_bytes, _ext.status_word(q.device).data_ptr(), _ext.stream_ptr(q.device), st)
    _ext.raise_for_status(rc, "corope_gqa_bwd")
    _ext.post_call(q.device)
    return dq, dk, dv


class _attention(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, theta, warp_specialize=False):
        qc, kc, vc, o, lse2, a_diag = _forward(q, k, v, causal, sm_scale, theta)
        ctx.save_for_backward(qc, kc, vc, o, lse2, a_diag)
        ctx.group_size = q.shape[1] // k.shape[1]
        ctx.sm_scale = sm_scale
        ctx.theta = theta
        ctx.causal = causal
        return o

    @staticmethod
    def backward(ctx, grad_output):
        q, k, v, o, lse2, a_diag = ctx.saved_tensors
        dq, dk, dv = _backward(q, k, v, o, lse2, a_diag, grad_output, ctx.sm_scale, ctx.theta)
        return dq, dk, dv, None, None, None, None


attention = _attention.apply
