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

SOURCES = ["abi.cu", "rope_general.cu", "rope_fwd_sm100.cu", "rope_bwd_sm100.cu", "corope_general.cu", "corope_fwd_mma.cu", "corope_bwd_mma.cu", "noalloc.cu"]

DTYPE_CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
OP_ROPE_FWD, OP_ROPE_BWD, OP_GQA_FWD, OP_GQA_BWD = 0, 1, 2, 3

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
    deps = srcs + [os.path.join(_CSRC, "common.cuh"), HEADER_PATH]
    if not force and os.path.exists(LIB_PATH) and all(os.path.getmtime(LIB_PATH) >= os.path.getmtime(d) for d in deps):
        return LIB_PATH
    objs = []
    procs = []
    for src in srcs:
        obj = src[:-3] + ".o"
        objs.append(obj)
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
               "-Xcompiler", "-fPIC", "--use_fast_math" if False else "-DCOROPE_BUILD", "-c", src, "-o", obj]
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
            L.corope_rope_attn_fwd.restype = i32
            L.corope_rope_attn_fwd.argtypes = [vp, vp, vp, vp, vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp, sz, vp, vp]
            L.corope_rope_attn_fwd_noalloc.restype = i32
            L.corope_rope_attn_fwd_noalloc.argtypes = [vp, vp, vp, vp, vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp, vp]
            L.corope_rope_attn_bwd.restype = i32
            L.corope_rope_attn_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i64, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32,
                                               vp, sz, vp, vp]
            L.corope_gqa_fwd.restype = i32
            L.corope_gqa_fwd.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, f32, vp, sz, vp, vp]
            L.corope_gqa_bwd.restype = i32
            L.corope_gqa_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, f32, vp, sz, vp, vp]
            _lib = L
        return _lib


def require_cuda(t):
    if not t.is_cuda:
        raise RuntimeError("corope_b200 runs on CUDA tensors only (got a %s tensor); there is no CPU path." % t.device.type)


def status_word(device):
    """Per-device int32 that kernels set when a bounded wait expires (0 = healthy)."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    with _lock:
        w = _status_words.get(key)
        if w is None:
            w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
            _status_words[key] = w
        return w


def check_status(device=None):
    """Synchronise and raise if any kernel on `device` reported an expired wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = status_word(dev)
    v = int(w.item())
    if v != 0:
        w.zero_()
        raise RuntimeError("corope_b200 kernel reported device status 0x%x (bounded wait expired)" % v)


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
