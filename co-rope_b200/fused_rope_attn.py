"""Drop-in for the reference's `fused_rope_attn.attention` (fused-rope/fused_rope_attn.py:652-780).

    attention(q, k, v, causal, sm_scale, freqs_cos, freqs_sin, warp_specialize=True) -> o

q, k, v: [B, H, N, D] CUDA tensors of one dtype (bf16, fp16 or fp32).  freqs_cos / freqs_sin: [N, D]
("cat" layout of precompute_freqs_cis) or [N, D/2]; only columns [0, D/2) are read, as in the
reference (fused_rope_attn.py:88-93).  Positional-only, like torch.autograd.Function.apply.
The CUDA kernels are reached through the C ABI in include/corope_b200.h.

Device-side errors: kernels never trap; a bounded wait that runs out sets a per-device status word.  Every call
first looks at a pinned host mirror of that word (refreshed by a side stream after each call, no synchronisation)
and raises RuntimeError, clearing the word, if an earlier call set it; `_ext.check_status()` does the same with a
synchronisation.
"""

import torch

try:
    from . import _ext
except ImportError:  # imported as a top-level module (directory on sys.path, the way the reference's scripts import it)
    import _ext

SUPPORTED_HEAD_DIMS = (32, 64, 128)


def _tables(freqs_cos, freqs_sin, N, D, device):
    if freqs_cos.shape != freqs_sin.shape or freqs_cos.dim() != 2:
        raise ValueError("freqs_cos and freqs_sin must be 2-D tensors of the same shape")
    if freqs_cos.shape[0] < N or freqs_cos.shape[1] < D // 2:
        raise ValueError("RoPE tables must cover [N, D/2] = [%d, %d], got %s" % (N, D // 2, tuple(freqs_cos.shape)))
    out = []
    for t in (freqs_cos, freqs_sin):
        _ext.require_cuda(t)
        if t.dtype != torch.float32 or t.stride(1) != 1:
            t = t.float().contiguous()
        out.append(t)
    if out[0].stride(0) != out[1].stride(0):
        out = [t.contiguous() for t in out]
    return out[0], out[1], out[0].stride(0)


def _forward(q, k, v, causal, sm_scale, freqs_cos, freqs_sin):
    """Checks + one corope_rope_attn_fwd call.  Returns what the backward needs: (q, k, v, o, M, cos, sin, table stride)."""
    # shape constraints, as fused_rope_attn.py:657-661
    HEAD_DIM_Q, HEAD_DIM_K = q.shape[-1], k.shape[-1]
    HEAD_DIM_V = v.shape[-1]
    assert HEAD_DIM_Q == HEAD_DIM_K and HEAD_DIM_K == HEAD_DIM_V
    assert HEAD_DIM_K in {16, 32, 64, 128, 256}
    assert HEAD_DIM_K in SUPPORTED_HEAD_DIMS, "corope_b200 supports head dims %s" % (SUPPORTED_HEAD_DIMS,)
    assert q.shape == k.shape == v.shape and q.dim() == 4
    assert q.dtype == k.dtype == v.dtype and q.dtype in _ext.DTYPE_CODES
    for t in (q, k, v):
        _ext.require_cuda(t)
    B, H, N, D = q.shape
    # the kernels take the tensors' own strides, like the reference's (fused_rope_attn.py:709-710): a [B, N, H, D] buffer viewed
    # as [B, H, N, D] is not copied, and o = empty_like(q) has q's layout (:662)
    qc, kc, vc = _ext.kernel_layout(q), _ext.kernel_layout(k), _ext.kernel_layout(v)
    cos, sin, tstride = _tables(freqs_cos, freqs_sin, N, D, q.device)
    o = torch.empty_like(qc)
    M = torch.empty((B, H, N), device=q.device, dtype=torch.float32)
    ws, ws_bytes = _ext.workspace(_ext.OP_ROPE_FWD, B, H, H, N, D, q.dtype, q.device)
    st = _ext.strides_of(q=qc, k=kc, v=vc, o=o)
    _ext.pre_call(q.device)
    with torch.cuda.device(q.device):
        rc = _ext.lib().corope_rope_attn_fwd_strided(
            qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), cos.data_ptr(), sin.data_ptr(), tstride,
            o.data_ptr(), M.data_ptr(), B, H, N, D, _ext.DTYPE_CODES[q.dtype], int(bool(causal)), float(sm_scale),
            ws.data_ptr(), ws_bytes, _ext.status_word(q.device).data_ptr(), _ext.stream_ptr(q.device), st)
    _ext.raise_for_status(rc, "corope_rope_attn_fwd")
    _ext.post_call(q.device)
    return qc, kc, vc, o, M, cos, sin, tstride


def _backward(q, k, v, o, M, cos, sin, tstride, do, causal, sm_scale):
    """One corope_rope_attn_bwd call on what _forward returned.  Returns (dq, dk, dv)."""
    # the reference asserts a contiguous dO, equal strides and N % 128 == 0 (fused_rope_attn.py:727-728, 750); these kernels
    # take any N and every tensor's own strides
    do = _ext.kernel_layout(do)
    B, H, N, D = q.shape
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    ws, ws_bytes = _ext.workspace(_ext.OP_ROPE_BWD, B, H, H, N, D, q.dtype, q.device)
    st = _ext.strides_of(q=q, k=k, v=v, o=o, d_o=do, dq=dq, dk=dk, dv=dv)
    _ext.pre_call(q.device)
    with torch.cuda.device(q.device):
        rc = _ext.lib().corope_rope_attn_bwd_strided(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), M.data_ptr(),
            cos.data_ptr(), sin.data_ptr(), tstride, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            B, H, N, D, _ext.DTYPE_CODES[q.dtype], int(bool(causal)), float(sm_scale),
            ws.data_ptr(), ws_bytes, _ext.status_word(q.device).data_ptr(), _ext.stream_ptr(q.device), st)
    _ext.raise_for_status(rc, "corope_rope_attn_bwd")
    _ext.post_call(q.device)
    return dq, dk, dv


class _attention(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, freqs_cos, freqs_sin, warp_specialize=True):
        qc, kc, vc, o, M, cos, sin, tstride = _forward(q, k, v, causal, sm_scale, freqs_cos, freqs_sin)
        ctx.save_for_backward(qc, kc, vc, o, M, cos, sin)
        ctx.sm_scale = sm_scale
        ctx.HEAD_DIM = q.shape[-1]
        ctx.causal = causal
        ctx.tstride = tstride
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, M, cos, sin = ctx.saved_tensors
        dq, dk, dv = _backward(q, k, v, o, M, cos, sin, ctx.tstride, do, ctx.causal, ctx.sm_scale)
        return dq, dk, dv, None, None, None, None, None


attention = _attention.apply


# ---------------------------------------------------------------------------------------------------------------------
# The same attention with the tables left out of the interface: for callers whose cos / sin tables are the output of the
# reference's precompute_freqs_cis(D, N, theta) (fused-rope/rope_attn_pytorch.py:10-49) the angles can be formed on the
# device from D/2 frequencies, so no [N, D] tables have to exist at all.  The explicit-table entry point above stays the
# general case (other positions, scaled frequencies).
# ---------------------------------------------------------------------------------------------------------------------
def inv_freq_of(theta, D, device):
    """The D/2 frequencies exactly as precompute_freqs_cis computes them (rope_attn_pytorch.py:29), on `device`."""
    return 1.0 / (theta ** (torch.arange(0, D, 2, device=device).float() / D))


def _forward_freqs(q, k, v, causal, sm_scale, inv_freq):
    HEAD_DIM_K = q.shape[-1]
    assert HEAD_DIM_K in SUPPORTED_HEAD_DIMS, "corope_b200 supports head dims %s" % (SUPPORTED_HEAD_DIMS,)
    assert q.shape == k.shape == v.shape and q.dim() == 4
    assert q.dtype == k.dtype == v.dtype and q.dtype in _ext.DTYPE_CODES
    for t in (q, k, v, inv_freq):
        _ext.require_cuda(t)
    B, H, N, D = q.shape
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == D // 2 and inv_freq.is_contiguous()
    qc, kc, vc = q.contiguous(), k.contiguous(), v.contiguous()
    o = torch.empty_like(qc)
    M = torch.empty((B, H, N), device=q.device, dtype=torch.float32)
    ws, ws_bytes = _ext.workspace(_ext.OP_ROPE_FWD_FREQS, B, H, H, N, D, q.dtype, q.device)
    _ext.pre_call(q.device)
    with torch.cuda.device(q.device):
        rc = _ext.lib().corope_rope_attn_fwd_freqs(
            qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), inv_freq.data_ptr(), o.data_ptr(), M.data_ptr(), B, H, N, D,
            _ext.DTYPE_CODES[q.dtype], int(bool(causal)), float(sm_scale),
            ws.data_ptr(), ws_bytes, _ext.status_word(q.device).data_ptr(), _ext.stream_ptr(q.device))
    _ext.raise_for_status(rc, "corope_rope_attn_fwd_freqs")
    _ext.post_call(q.device)
    return qc, kc, vc, o, M


def _backward_freqs(q, k, v, o, M, inv_freq, do, causal, sm_scale):
    do = do.contiguous()
    B, H, N, D = q.shape
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ws, ws_bytes = _ext.workspace(_ext.OP_ROPE_BWD_FREQS, B, H, H, N, D, q.dtype, q.device)
    _ext.pre_call(q.device)
    with torch.cuda.device(q.device):
        rc = _ext.lib().corope_rope_attn_bwd_freqs(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), M.data_ptr(), inv_freq.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, H, N, D, _ext.DTYPE_CODES[q.dtype], int(bool(causal)), float(sm_scale),
            ws.data_ptr(), ws_bytes, _ext.status_word(q.device).data_ptr(), _ext.stream_ptr(q.device))
    _ext.raise_for_status(rc, "corope_rope_attn_bwd_freqs")
    _ext.post_call(q.device)
    return dq, dk, dv


class _attention_theta(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, theta):
        inv_freq = inv_freq_of(theta, q.shape[-1], q.device)
        qc, kc, vc, o, M = _forward_freqs(q, k, v, causal, sm_scale, inv_freq)
        ctx.save_for_backward(qc, kc, vc, o, M, inv_freq)
        ctx.sm_scale = sm_scale
        ctx.causal = causal
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, M, inv_freq = ctx.saved_tensors
        dq, dk, dv = _backward_freqs(q, k, v, o, M, inv_freq, do, ctx.causal, ctx.sm_scale)
        return dq, dk, dv, None, None, None


attention_theta = _attention_theta.apply   # attention_theta(q, k, v, causal, sm_scale, theta): positions 0 .. N-1, base theta
