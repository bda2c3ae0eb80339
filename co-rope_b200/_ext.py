"""Loader for the C-ABI library (libcorope_b200.so) and thin ctypes call helpers.

The library is built in-tree by `build()` (nvcc, sm_100a only).  There is no fallback:
if the library is missing or a CUDA device is absent, the attention entry points raise.
"""

import ctypes
import os
import subprocess
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "libcorope_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "corope_b200.h")
DEBUG_HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "corope_b200_debug.h")

SOURCES = ["abi.cu", "rope_general.cu", "rope_fwd_sm100.cu", "rope_bwd_sm100.cu", "corope_general.cu", "corope_fwd_mma.cu", "corope_bwd_mma.cu", "noalloc.cu",
           "debug.cu"]

DTYPE_CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
OP_ROPE_FWD, OP_ROPE_BWD, OP_GQA_FWD, OP_GQA_BWD = 0, 1, 2, 3
OP_ROPE_FWD_FREQS, OP_ROPE_BWD_FREQS, OP_FLASH_FWD, OP_FLASH_BWD = 4, 5, 6, 7

_lock = threading.Lock()
_lib = None
_status_words = {}


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def build(force=False, verbose=False):
    """Compile csrc/*.cu into libcorope_b200.so for sm_100a (cross-compiles without a GPU)."""
    srcs = [os.path.join(_CSRC, s) for s in SOURCES]
    deps = srcs + [os.path.join(_CSRC, "common.cuh"), os.path.join(_CSRC, "corope_mma.cuh"), HEADER_PATH, DEBUG_HEADER_PATH]
    if not force and os.path.exists(LIB_PATH) and all(os.path.getmtime(LIB_PATH) >= os.path.getmtime(d) for d in deps):
        return LIB_PATH
    objs = []
    procs = []
    for src in srcs:
        obj = src[:-3] + ".o"
        objs.append(obj)
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
               "-Xcompiler", "-fPIC", "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s" % (" ".join(cmd), out))
        if verbose and out:
            print(out)
    link = [_nvcc(), "-shared", "-o", LIB_PATH] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed: %s\n%s" % (" ".join(link), r.stdout))
    return LIB_PATH


def lib():
    """The loaded library.  Raises if it has not been built -- there is no other code path."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    "corope_b200: %s is missing; build it with `python -c \"import __graft_entry__ as g; g.build()\"` "
                    "(nvcc, sm_100a).  There is no CPU or PyTorch fallback." % LIB_PATH)
            L = ctypes.CDLL(LIB_PATH)
            vp, i32, i64, f32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t
            L.corope_abi_version.restype = i32
            L.corope_status_mirror_refresh.restype = i32
            L.corope_status_mirror_refresh.argtypes = [vp, vp, vp]
            L.corope_status_mirror_clear.restype = i32
            L.corope_status_mirror_clear.argtypes = [vp, vp, vp]
            L.corope_status_string.restype = ctypes.c_char_p
            L.corope_status_string.argtypes = [i32]
            L.corope_workspace_bytes.restype = sz
            L.corope_workspace_bytes.argtypes = [i32] * 7
            L.corope_launch_count.restype = ctypes.c_uint64
            L.corope_launch_count.argtypes = []
            L.corope_set_kernel_policy.restype = i32
            L.corope_set_kernel_policy.argtypes = [i32]
            L.corope_last_kernel_family.restype = i32
            L.corope_last_kernel_family.argtypes = [i32]
            if hasattr(L, "corope_debug_synth_tables"):
                L.corope_debug_synth_tables.restype = i32
                L.corope_debug_synth_tables.argtypes = [vp, vp, vp, i32, i32, vp]
            if hasattr(L, "corope_debug_expire_wait"):
                L.corope_debug_expire_wait.restype = i32
                L.corope_debug_expire_wait.argtypes = [vp, ctypes.c_uint, vp]
            L.corope_rope_attn_fwd.restype = i32
            L.corope_rope_attn_fwd.argtypes = [vp, vp, vp, vp, vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp, sz, vp, vp]
            L.corope_rope_attn_fwd_noalloc.restype = i32
            L.corope_rope_attn_fwd_noalloc.argtypes = [vp, vp, vp, vp, vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp, vp]
            L.corope_rope_attn_bwd.restype = i32
            L.corope_rope_attn_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i64, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32,
                                               vp, sz, vp, vp]
            sp = ctypes.POINTER(Strides)
            L.corope_rope_attn_fwd_strided.restype = i32
            L.corope_rope_attn_fwd_strided.argtypes = [vp, vp, vp, vp, vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp, sz, vp, vp, sp]
            L.corope_rope_attn_bwd_strided.restype = i32
            L.corope_rope_attn_bwd_strided.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i64, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32,
                                                       vp, sz, vp, vp, sp]
            L.corope_flash_attn_fwd_strided.restype = i32
            L.corope_flash_attn_fwd_strided.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp, sz, vp, vp, sp]
            L.corope_flash_attn_bwd_strided.restype = i32
            L.corope_flash_attn_bwd_strided.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp, sz,
                                                        vp, vp, sp]
            L.corope_rope_attn_fwd_freqs.restype = i32
            L.corope_rope_attn_fwd_freqs.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp, sz, vp, vp]
            L.corope_rope_attn_bwd_freqs.restype = i32
            L.corope_rope_attn_bwd_freqs.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp, sz, vp, vp]
            L.corope_flash_attn_fwd.restype = i32
            L.corope_flash_attn_fwd.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp, sz, vp, vp]
            L.corope_flash_attn_bwd.restype = i32
            L.corope_flash_attn_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp, sz, vp, vp]
            L.corope_gqa_fwd.restype = i32
            L.corope_gqa_fwd.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, f32, vp, sz, vp, vp]
            L.corope_gqa_bwd.restype = i32
            L.corope_gqa_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, f32, vp, sz, vp, vp]
            L.corope_gqa_fwd_strided.restype = i32
            L.corope_gqa_fwd_strided.argtypes = L.corope_gqa_fwd.argtypes + [ctypes.POINTER(Strides)]
            L.corope_gqa_bwd_strided.restype = i32
            L.corope_gqa_bwd_strided.argtypes = L.corope_gqa_bwd.argtypes + [ctypes.POINTER(Strides)]
            _lib = L
        return _lib


class Strides(ctypes.Structure):
    """corope_strides_t of the C header: {batch, head, row} strides in elements of q, k, v, o, d_o, dq, dk, dv."""
    _fields_ = [(name, ctypes.c_int64 * 3) for name in ("q", "k", "v", "o", "d_o", "dq", "dk", "dv")]


def strides_of(**tensors):
    """A Strides struct filled from the given [B, H, N, D] tensors (keyword = field name); other fields stay zero."""
    st = Strides()
    for name, t in tensors.items():
        getattr(st, name)[:] = list(t.stride()[:3])
    return st


def kernel_layout(t):
    """`t` itself when the kernels can take its layout directly (unit stride along the head dimension, no overlapping
    or broadcast strides), else a contiguous copy."""
    if t.stride(-1) == 1 and all(s > 0 for s in t.stride()) and t.stride(2) >= t.shape[3]:
        return t
    return t.contiguous()


def require_cuda(t):
    if not t.is_cuda:
        raise RuntimeError("corope_b200 runs on CUDA tensors only (got a %s tensor); there is no CPU path." % t.device.type)


class _DeviceStatus:
    """The device status word of one GPU with a pinned host mirror that the library's side stream refreshes after every call."""

    def __init__(self, index):
        dev = torch.device("cuda", index)
        self.index = index
        self.word = torch.zeros(1, dtype=torch.int32, device=dev)
        self.mirror = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.word_ptr = self.word.data_ptr()
        self.mirror_ptr = self.mirror.data_ptr()
        self.mirror_view = (ctypes.c_int * 1).from_address(self.mirror_ptr)   # a plain int read, no tensor indexing per call


def _status(device):
    key = device.index if isinstance(device, torch.device) else torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    st = _status_words.get(key)
    if st is None:
        with _lock:
            st = _status_words.get(key)
            if st is None:
                st = _DeviceStatus(key)
                _status_words[key] = st
    return st


def status_word(device):
    """Per-device int32 that kernels set when a bounded wait expires or a value leaves the supported range (0 = healthy)."""
    return _status(device).word


def _status_message(v):
    if v & 0x2000:
        return "a gradient term left the value range of the 16-bit Co-RoPE backward and was clamped (results of that call are inaccurate)"
    return "a bounded device-side wait expired (results of that call and of later calls are undefined)"


def pre_call(device):
    """Called by the attention entry points before they launch: raises if an EARLIER call on this device left the status
    word set.  Reads only the pinned host mirror (no synchronisation); the mirror is refreshed by post_call(), so the error
    surfaces at the first call after the failing one has finished on the GPU.  The word is cleared before raising."""
    if getattr(_batched, "depth", 0) > 0:
        return
    st = _status(device)
    v = st.mirror_view[0]
    if v != 0:
        with torch.cuda.device(st.index):
            lib().corope_status_mirror_clear(st.word_ptr, st.mirror_ptr, torch.cuda.current_stream(st.index).cuda_stream)
        raise RuntimeError("corope_b200: an earlier kernel reported device status 0x%x: %s" % (v, _status_message(v)))


_batched = threading.local()


class batched_status:
    """Context manager for callers that make many library calls in a row (the host pipeline): the per-call look at the
    mirror and its refresh are done once, on entry and on exit, instead of around every call."""

    def __init__(self, device):
        self.device = device

    def __enter__(self):
        pre_call(self.device)
        _batched.depth = getattr(_batched, "depth", 0) + 1
        return self

    def __exit__(self, *exc):
        _batched.depth -= 1
        if exc[0] is None:
            post_call(self.device)
        return False


def post_call(device, stream=None):
    """Called after a launch: the library's side stream copies the status word to its pinned mirror once the caller's stream
    gets there (the caller's stream itself only records an event).  The caller has the device current."""
    if getattr(_batched, "depth", 0) > 0:
        return
    if torch.cuda.is_current_stream_capturing():
        return
    st = _status(device)
    if stream is None:
        stream = torch.cuda.current_stream(st.index).cuda_stream
    if torch.cuda.current_device() == st.index:
        lib().corope_status_mirror_refresh(st.word_ptr, st.mirror_ptr, stream)
    else:   # the library's side stream belongs to the current device
        with torch.cuda.device(st.index):
            lib().corope_status_mirror_refresh(st.word_ptr, st.mirror_ptr, stream)


def check_status(device=None):
    """Synchronise and raise if any kernel on `device` has set the status word; clears it."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    st = _status(dev)
    v = int(st.word.item())
    if v != 0:
        with torch.cuda.device(st.index):
            lib().corope_status_mirror_clear(st.word_ptr, st.mirror_ptr, torch.cuda.current_stream(st.index).cuda_stream)
        torch.cuda.synchronize(st.index)
        raise RuntimeError("corope_b200 kernel reported device status 0x%x: %s" % (v, _status_message(v)))


def workspace(op, B, Hq, Hkv, N, D, dtype, device):
    nbytes = lib().corope_workspace_bytes(op, B, Hq, Hkv, N, D, DTYPE_CODES[dtype])
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device), int(nbytes)


def raise_for_status(code, what):
    if code == 0:
        return
    msg = lib().corope_status_string(code).decode()
    if code == -3:
        raise AssertionError("%s: %s" % (what, msg))
    if code in (-6,):
        raise ValueError("%s: %s" % (what, msg))
    raise RuntimeError("%s failed with status %d: %s" % (what, code, msg))


def stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream
