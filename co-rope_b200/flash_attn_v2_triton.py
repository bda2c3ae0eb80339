"""Drop-in for the reference's un-fused flash attention entry point
(fused-rope/flash_attn_v2_triton.py:513-631; the module keeps the reference's name so its scripts can import this one).

    attention(q, k, v, causal, sm_scale, warp_specialize=True) -> o

q: [B, Hq, N, D]; k, v: [B, Hkv, N, D] with Hq % Hkv == 0 -- query head h reads K / V head h // (Hq // Hkv), as the
reference's kernel maps them (:194-196).  No RoPE: callers rotate q / k themselves (the reference's baselines do,
fused-rope/baseline.py).  The backward also takes Hq != Hkv and returns dk / dv summed over each group (the reference's
backward asserts equal strides, i.e. Hq == Hkv, :560); the math is that of assets/flashattn-gqa/attn_gqa_pytorch.py.
The kernels are the fused-RoPE kernels with the rotation switched off, reached through corope_flash_attn_fwd / _bwd of
the C ABI in include/corope_b200.h.  Device-side errors are reported as in fused_rope_attn.py.
"""

import torch

try:
    from . import _ext
except ImportError:  # imported as a top-level module (directory on sys.path, the way the reference's scripts import it)
    import _ext

SUPPORTED_HEAD_DIMS = (32, 64, 128)


def _forward(q, k, v, causal, sm_scale):
    """Checks + one corope_flash_attn_fwd call.  Returns what the backward needs: (q, k, v, o, M)."""
    # shape constraints, as flash_attn_v2_triton.py:517-521
    HEAD_DIM_Q, HEAD_DIM_K = q.shape[-1], k.shape[-1]
    HEAD_DIM_V = v.shape[-1]
    assert HEAD_DIM_Q == HEAD_DIM_K and HEAD_DIM_K == HEAD_DIM_V
    assert HEAD_DIM_K in {16, 32, 64, 128, 256}
    assert HEAD_DIM_K in SUPPORTED_HEAD_DIMS, "corope_b200 supports head dims %s" % (SUPPORTED_HEAD_DIMS,)
    assert q.dim() == 4 and k.shape == v.shape and k.dim() == 4
    assert q.shape[0] == k.shape[0] and q.shape[2] == k.shape[2]
    assert q.dtype == k.dtype == v.dtype and q.dtype in _ext.DTYPE_CODES
    B, H_Q, N, D = q.shape
    H_KV = k.shape[1]
    assert H_Q % H_KV == 0, "number of query heads must be a multiple of the number of K / V heads"
    for t in (q, k, v):
        _ext.require_cuda(t)
    qc, kc, vc = _ext.kernel_layout(q), _ext.kernel_layout(k), _ext.kernel_layout(v)   # own strides, no copies (as :601-603)
    o = torch.empty_like(qc)
    M = torch.empty((B, H_Q, N), device=q.device, dtype=torch.float32)
    ws, ws_bytes = _ext.workspace(_ext.OP_FLASH_FWD, B, H_Q, H_KV, N, D, q.dtype, q.device)
    st = _ext.strides_of(q=qc, k=kc, v=vc, o=o)
    _ext.pre_call(q.device)
    with torch.cuda.device(q.device):
        rc = _ext.lib().corope_flash_attn_fwd_strided(
            qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), M.data_ptr(), B, H_Q, H_KV, N, D,
            _ext.DTYPE_CODES[q.dtype], int(bool(causal)), float(sm_scale),
            ws.data_ptr(), ws_bytes, _ext.status_word(q.device).data_ptr(), _ext.stream_ptr(q.device), st)
    _ext.raise_for_status(rc, "corope_flash_attn_fwd")
    _ext.post_call(q.device)
    return qc, kc, vc, o, M


def _backward(q, k, v, o, M, do, causal, sm_scale):
    """One corope_flash_attn_bwd call on what _forward returned.  Returns (dq, dk, dv)."""
    do = _ext.kernel_layout(do)
    B, H_Q, N, D = q.shape
    H_KV = k.shape[1]
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    ws, ws_bytes = _ext.workspace(_ext.OP_FLASH_BWD, B, H_Q, H_KV, N, D, q.dtype, q.device)
    st = _ext.strides_of(q=q, k=k, v=v, o=o, d_o=do, dq=dq, dk=dk, dv=dv)
    _ext.pre_call(q.device)
    with torch.cuda.device(q.device):
        rc = _ext.lib().corope_flash_attn_bwd_strided(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), M.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, H_Q, H_KV, N, D, _ext.DTYPE_CODES[q.dtype], int(bool(causal)),
            float(sm_scale), ws.data_ptr(), ws_bytes, _ext.status_word(q.device).data_ptr(), _ext.stream_ptr(q.device), st)
    _ext.raise_for_status(rc, "corope_flash_attn_bwd")
    _ext.post_call(q.device)
    return dq, dk, dv


class _attention(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, warp_specialize=True):
        qc, kc, vc, o, M = _forward(q, k, v, causal, sm_scale)
        ctx.save_for_backward(qc, kc, vc, o, M)
        ctx.sm_scale = sm_scale
        ctx.HEAD_DIM = q.shape[-1]
        ctx.causal = causal
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, M = ctx.saved_tensors
        dq, dk, dv = _backward(q, k, v, o, M, do, ctx.causal, ctx.sm_scale)
        return dq, dk, dv, None, None, None


attention = _attention.apply
