"""Generate the golden vectors under tests/golden/ from the reference's own PyTorch code.

Run where a checkout of the reference is available (the tests themselves must not
depend on one, which is why the vectors are committed):

    TORCH_COMPILE_DISABLE=1 python tests/golden/make_golden.py /path/to/reference

For every case it draws seeded N(0,1) inputs, rounds them to fp16 (so they
are stored exactly in 2 bytes and are exact in fp32), upcasts to fp32, and
runs the reference's `attention_pytorch` forward and its hand-written backward
(fused-rope/rope_attn_pytorch.py:87-227, corope-exp/corope_attn_gqa_pytorch.py:9-303,
assets/flashattn-gqa/attn_gqa_pytorch.py:10-193).
Outputs are stored in fp32.
"""

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

ROPE_CASES = {
    # name: (B, H, N, D, causal, sm_scale, theta, seed)
    "rope_a": (1, 2, 64, 32, True, 32 ** -0.5, 10000.0, 1),
    "rope_b": (2, 1, 96, 64, False, 0.5, 10000.0, 2),
    "rope_c": (1, 1, 128, 128, True, 128 ** -0.5, 10000.0, 3),
}
COROPE_CASES = {
    # name: (B, Hq, Hkv, N, D, sm_scale, theta, seed)
    "corope_a": (2, 4, 2, 64, 32, 32 ** -0.5, 10000.0, 42),
    "corope_b": (1, 4, 1, 48, 64, 64 ** -0.5, 10000.0, 5),
    "corope_c": (1, 2, 2, 32, 128, 128 ** -0.5, 500.0, 6),
}


GQA_CASES = {
    # name: (B, Hq, Hkv, N, D, causal, sm_scale, seed)   -- plain attention with grouped K / V heads
    "attn_gqa_a": (2, 4, 2, 64, 32, True, 32 ** -0.5, 11),
    "attn_gqa_b": (1, 6, 2, 80, 64, False, 0.5, 12),
    "attn_gqa_c": (1, 2, 2, 128, 128, True, 128 ** -0.5, 13),
}


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _draw(shape, gen):
    return torch.randn(shape, generator=gen, dtype=torch.float32).to(torch.float16)


def main(ref_root):
    os.environ.setdefault("TORCH_COMPILE_DISABLE", "1")
    rope = _load(os.path.join(ref_root, "fused-rope", "rope_attn_pytorch.py"), "ref_rope_attn_pytorch")
    corope = _load(os.path.join(ref_root, "corope-exp", "corope_attn_gqa_pytorch.py"), "ref_corope_attn_gqa_pytorch")

    for name, (B, H, N, D, causal, sm_scale, theta, seed) in ROPE_CASES.items():
        gen = torch.Generator().manual_seed(seed)
        q16, k16, v16, do16 = (_draw((B, H, N, D), gen) for _ in range(4))
        q, k, v = (t.float().requires_grad_(True) for t in (q16, k16, v16))
        cos, sin = rope.precompute_freqs_cis(D, N, theta, device="cpu")
        o = rope.attention_pytorch(q, k, v, causal, sm_scale, cos, sin)
        o.backward(do16.float())
        np.savez(os.path.join(HERE, name + ".npz"),
                 meta=np.array([B, H, N, D, int(causal), seed], dtype=np.int64),
                 scal=np.array([sm_scale, theta], dtype=np.float64),
                 q=q16.numpy(), k=k16.numpy(), v=v16.numpy(), do=do16.numpy(),
                 cos=cos.numpy(), sin=sin.numpy(),
                 o=o.detach().numpy(), dq=q.grad.numpy(), dk=k.grad.numpy(), dv=v.grad.numpy())
        print(name, "ok", tuple(o.shape))

    for name, (B, Hq, Hkv, N, D, sm_scale, theta, seed) in COROPE_CASES.items():
        gen = torch.Generator().manual_seed(seed)
        q16 = _draw((B, Hq, N, D), gen)
        k16 = _draw((B, Hkv, N, D), gen)
        v16 = _draw((B, Hkv, N, D), gen)
        do16 = _draw((B, Hq, N, D), gen)
        q, k, v = (t.float().requires_grad_(True) for t in (q16, k16, v16))
        o = corope.attention_pytorch(q, k, v, True, sm_scale, theta)
        o.backward(do16.float())
        np.savez(os.path.join(HERE, name + ".npz"),
                 meta=np.array([B, Hq, Hkv, N, D, seed], dtype=np.int64),
                 scal=np.array([sm_scale, theta], dtype=np.float64),
                 q=q16.numpy(), k=k16.numpy(), v=v16.numpy(), do=do16.numpy(),
                 o=o.detach().numpy(), dq=q.grad.numpy(), dk=k.grad.numpy(), dv=v.grad.numpy())
        print(name, "ok", tuple(o.shape))


    gqa = _load(os.path.join(ref_root, "assets", "flashattn-gqa", "attn_gqa_pytorch.py"), "ref_attn_gqa_pytorch")
    for name, (B, Hq, Hkv, N, D, causal, sm_scale, seed) in GQA_CASES.items():
        gen = torch.Generator().manual_seed(seed)
        q16 = _draw((B, Hq, N, D), gen)
        k16 = _draw((B, Hkv, N, D), gen)
        v16 = _draw((B, Hkv, N, D), gen)
        do16 = _draw((B, Hq, N, D), gen)
        q, k, v = (t.float().requires_grad_(True) for t in (q16, k16, v16))
        o = gqa.attention_pytorch(q, k, v, causal, sm_scale)
        o.backward(do16.float())
        np.savez(os.path.join(HERE, name + ".npz"),
                 meta=np.array([B, Hq, Hkv, N, D, int(causal), seed], dtype=np.int64),
                 scal=np.array([sm_scale], dtype=np.float64),
                 q=q16.numpy(), k=k16.numpy(), v=v16.numpy(), do=do16.numpy(),
                 o=o.detach().numpy(), dq=q.grad.numpy(), dk=k.grad.numpy(), dv=v.grad.numpy())
        print(name, "ok", tuple(o.shape))


if __name__ == "__main__":
    # argument: path of a checkout of the reference (default: a directory named "reference" beside this repository)
    here = os.path.dirname(os.path.abspath(__file__))
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(here))), "reference"))
