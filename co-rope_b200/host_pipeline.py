"""Forward + backward for tensors that live in pinned host memory.

The unit of work -- one (batch, KV head) pair with its group of query heads -- is independent of all others, so a
call on host tensors does not have to wait for the whole input to cross PCIe: the units are cut into chunks and run
through three streams (host-to-device copies, the kernels, device-to-host copies).  Copying in chunk c + 1 and
copying out chunk c - 1 overlap the kernels of chunk c, and the two copy directions overlap each other, so the
call costs about one direction's copy time instead of both directions plus the kernels.
"""

import torch

from . import _ext
from . import fused_rope_attn as _rope
from . import flash_attn_co_rope_gqa_triton as _gqa


_side_streams = {}   # device index -> (copy-in stream, copy-out stream), created once: the caching allocator keeps one pool
                     # of blocks per stream, so fresh streams on every call would mean fresh cudaMallocs on every call


def _streams():
    dev = torch.cuda.current_device()
    if dev not in _side_streams:
        _side_streams[dev] = (torch.cuda.Stream(), torch.cuda.Stream())
    return _side_streams[dev]


def _unit_view(t, n_units):
    """[B, H, N, D] -> [B * Hkv, G, N, D] (no copy: the heads of a group are adjacent)."""
    B, H, N, D = t.shape
    return t.view(n_units, (B * H) // n_units, N, D)


def auto_chunks(total_bytes, n_units):
    """Chunk count of the pipeline when the caller names none: about 32 MB of traffic per chunk, between 2 and 16 chunks.  More
    chunks hide more of the first copy-in and the last copy-out behind the kernels, but every chunk costs about 0.1 ms of host
    work (two library calls and a dozen stream operations), which a small call would not earn back."""
    return max(1, min(n_units, 16, max(2, int(total_bytes // (32 << 20)))))


def attention_fwd_bwd_host(q, k, v, d_o, sm_scale, *, freqs_cos=None, freqs_sin=None, theta=None, out=None, chunks=None):
    """o, dq, dk, dv for pinned host tensors q [B,Hq,N,D], k / v [B,Hkv,N,D], d_o like q (causal attention).

    With `freqs_cos` / `freqs_sin` (device tensors) this is the fused-RoPE attention (Hq == Hkv); with `theta` it is
    the Co-RoPE GQA attention.  `out` = (o, dq, dk, dv) preallocated pinned host tensors, or None to allocate them.
    `chunks` = number of pipeline chunks (None: chosen from the size, see auto_chunks).
    Results are complete when the current stream has finished (the call does not synchronise).
    """
    if (theta is None) == (freqs_cos is None):
        raise ValueError("give either freqs_cos/freqs_sin (fused RoPE) or theta (Co-RoPE)")
    for t in (q, k, v, d_o):
        if t.is_cuda or not t.is_pinned() or not t.is_contiguous():
            raise ValueError("inputs must be contiguous pinned host tensors")
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    n_units = B * Hkv
    if chunks is None:
        chunks = auto_chunks(2 * sum(t.numel() * t.element_size() for t in (q, k, v, d_o)), n_units)
    chunks = max(1, min(int(chunks), n_units))
    if out is None:
        out = tuple(torch.empty_like(t).pin_memory() for t in (q, q, k, v))
    ho, hdq, hdk, hdv = out
    for t, like in zip(out, (q, q, k, v)):
        if t.is_cuda or not t.is_pinned() or not t.is_contiguous() or t.shape != like.shape or t.dtype != like.dtype:
            raise ValueError("outputs must be contiguous pinned host tensors shaped like q, q, k, v")
    uq, uk, uv, udo, uo, udq, udk, udv = (_unit_view(t, n_units) for t in (q, k, v, d_o, ho, hdq, hdk, hdv))
    G = Hq // Hkv

    cur = torch.cuda.current_stream()
    s_in, s_out = _streams()
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    bounds = [(n_units * c) // chunks for c in range(chunks + 1)]
    with _ext.batched_status(cur.device):
        _run_chunks(bounds, chunks, uq, uk, uv, udo, uo, udq, udk, udv, G, N, D, cur, s_in, s_out, sm_scale, freqs_cos, freqs_sin, theta)
    cur.wait_stream(s_out)
    return ho, hdq, hdk, hdv


def _run_chunks(bounds, chunks, uq, uk, uv, udo, uo, udq, udk, udv, G, N, D, cur, s_in, s_out, sm_scale, freqs_cos, freqs_sin, theta):
    for c in range(chunks):
        lo, hi = bounds[c], bounds[c + 1]
        n = hi - lo
        with torch.cuda.stream(s_in):
            dq_, dk_, dv_, ddo = (t[lo:hi].to("cuda", non_blocking=True) for t in (uq, uk, uv, udo))
            landed = s_in.record_event()
        for t in (dq_, dk_, dv_, ddo):
            t.record_stream(cur)
        cur.wait_event(landed)
        # a chunk is a batch of one with n KV heads; the two library calls are made directly (same checks as the autograd
        # entry points, none of the autograd engine's per-call cost, which a 16-chunk call would pay 32 times)
        qq, kk, vv, dd = dq_.view(1, n * G, N, D), dk_.view(1, n, N, D), dv_.view(1, n, N, D), ddo.view(1, n * G, N, D)
        if theta is None:
            saved = _rope._forward(qq, kk, vv, True, sm_scale, freqs_cos, freqs_sin)
            o = saved[3]
            gq, gk, gv = _rope._backward(*saved, dd, True, sm_scale)
        else:
            saved = _gqa._forward(qq, kk, vv, True, sm_scale, theta)
            o = saved[3]
            gq, gk, gv = _gqa._backward(*saved, dd, sm_scale, theta)
        done = cur.record_event()
        s_out.wait_event(done)
        with torch.cuda.stream(s_out):
            uo[lo:hi].copy_(o.view(n, G, N, D), non_blocking=True)
            udq[lo:hi].copy_(gq.view(n, G, N, D), non_blocking=True)
            udk[lo:hi].copy_(gk.view(n, 1, N, D), non_blocking=True)
            udv[lo:hi].copy_(gv.view(n, 1, N, D), non_blocking=True)
        for t in (o, gq, gk, gv):
            t.record_stream(s_out)
