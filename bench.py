"""Benchmark of the fused-RoPE attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--scaling strong|weak]

A step is one forward + backward pass of fused-RoPE causal attention over one synthetic batch of the
workload (default: the Llama-7B-4K shape, B=2 H=32 N=4096 D=128 bf16).  The metric is causal-adjusted
TFLOP/s with the FLOP convention of the reference's benchmark driver (fused-rope/bench_compare.py:61-86):
F_fwd = 4*B*H*N^2*D*0.5, F_bwd = 2.5*F_fwd.

With N > 1 GPUs (torchrun, one rank per GPU) the (batch, KV head) units of that ONE problem are divided among the
ranks (`sharding.unit_range`; strong scaling): every rank draws its own units from (seed, unit index), runs them with no
data-path collective, and `value` is the whole problem's FLOPs divided by the slowest rank's time.  Outside the timed
region the ranks' O, dQ, dK, dV are gathered with NCCL and rank 0 compares them with a single-GPU run of the whole
problem (`shard_check`).  `--scaling weak` gives every rank the whole problem instead.

One JSON line is printed by rank 0.  `--impl reference` times the reference's own PyTorch implementation on the host
cores instead (its unmodified files when the build step has staged them, else the CPU restatement under oracle/).
`--triton-baseline` (used by the default run as a child process) times the reference's Triton kernels on the GPU.
"""

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
os.environ.setdefault("TORCH_COMPILE_DISABLE", "1")

import torch  # noqa: E402

WORKLOADS = {
    # name: (kind, B, Hq, Hkv, N, D, dtype)
    "llama7b-4k": ("rope", 2, 32, 32, 4096, 128, "bf16"),
    "llama70b-1k": ("rope", 2, 64, 64, 1024, 128, "bf16"),
    "long-64k": ("rope", 1, 8, 8, 65536, 128, "bf16"),
    "small-512-fp32": ("rope", 4, 8, 8, 512, 64, "f32"),
    "corope-gqa-2k": ("corope", 2, 32, 8, 2048, 128, "bf16"),
}
DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}
THETA = 10000.0
REF_COPY = os.path.join(ROOT, "baseline", "_ref")

# DRAM bytes per launch of the two tensor-core kernels, from one ncu capture of both (dram__bytes_read.sum +
# dram__bytes_write.sum) at the Llama-7B-4K shape itself, B=2 H=32 N=4096 D=128 bf16 -- 251.8 MB forward, 628.6 MB backward
# (profiles/rope_fwd_bwd_sm100_llama7b_4k.md) -- expressed per byte of one [B,H,N,D] bf16 tensor (67.11 MB there).  Traffic of
# these kernels is proportional to the tensor bytes as long as a head's K/V (and, backward, its fp32 dQ rows) fit in L2, which
# holds for every workload here; for the default workload on one GPU the factor is exact.
NCU_DRAM_PER_TENSOR_BYTE = {"fused_rope_fwd": 251.8 / 67.11, "fused_rope_bwd": 628.6 / 67.11}


def flops_fwd(B, H, N, D):
    return 4.0 * B * H * N * N * D * 0.5


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"tflops": float(d["bf16_tflops"]), "tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi for the whole run; every sample carries the host time at which
    it was read, so that figures can be taken over any window (the timed region, the sustained leg)."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, device_index):
        self.rows = []
        self.proc = None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            ident = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            ident = str(device_index)
        self.cmd = ["nvidia-smi", "-i", ident, "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "50"]

    def start(self):
        try:
            self.proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is None:
            return
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()

    def window(self, t0, t1):
        """Median SM clock, power and the throttle reasons seen between host times t0 and t1 (a sample read up to 60 ms after
        t1 still describes the window: nvidia-smi reports with that delay)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        sm, mx, pw, reasons = [], [], [], set()
        for t, r in self.rows:
            if t < t0 or t > t1 + 0.06:
                continue
            parts = [x.strip() for x in r.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                pw.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(pw) if pw else None}


def unit_inputs(units, G, N, D, dtype, seed):
    """q [n*G, N, D], k, v [n, N, D], dO like q for the given (batch, KV head) unit indices: N(0,1) drawn in fp32 from a
    generator seeded by (seed, unit index) and cast to the test dtype, so a unit's values do not depend on which rank draws it."""
    qs, ks, vs, dos = [], [], [], []
    for u in units:
        gen = torch.Generator(device="cpu").manual_seed(seed * 1000003 + u)
        qs.append(torch.randn((G, N, D), generator=gen, dtype=torch.float32).to(dtype))
        ks.append(torch.randn((1, N, D), generator=gen, dtype=torch.float32).to(dtype))
        vs.append(torch.randn((1, N, D), generator=gen, dtype=torch.float32).to(dtype))
        dos.append(torch.randn((G, N, D), generator=gen, dtype=torch.float32).to(dtype))
    return tuple(torch.cat(x, dim=0) for x in (qs, ks, vs, dos))


# ------------------------------------------------------------------------------------------------------------------
# CPU reference arm
# ------------------------------------------------------------------------------------------------------------------
def _reference_modules():
    """The reference's own PyTorch modules from the staged copy, or None.  Its precompute_freqs_cis is decorated with
    torch.compile; TORCH_COMPILE_DISABLE (set above) makes that a no-op on hosts without a working inductor toolchain."""
    mods = {}
    for sub, name in (("fused-rope", "rope_attn_pytorch"), ("corope-exp", "corope_attn_gqa_pytorch")):
        path = os.path.join(REF_COPY, sub, name + ".py")
        if not os.path.exists(path):
            return None
        spec = importlib.util.spec_from_file_location("_staged_" + name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods


def cpu_reference_sample(kind, Hq, Hkv, N, D, n_units, threads=None):
    """Times the reference's PyTorch path (fwd + bwd, fp32) on `n_units` (batch, KV head) units of the workload on the host
    cores.  Uses the reference's own functions, one unit per call, where their dense N x N temporaries fit (fused RoPE up
    to N = 8192; Co-RoPE up to N = 512 per group); otherwise the row-blocked CPU restatement.  Returns seconds, FLOPs, kind."""
    import importlib.util  # noqa: F401

    if threads:
        torch.set_num_threads(threads)
    G = Hq // Hkv
    gen = torch.Generator().manual_seed(1234)
    mods = _reference_modules()
    dense_ok = mods is not None and ((kind == "rope" and N <= 8192) or (kind == "corope" and N <= 512))
    import oracle

    t0 = time.perf_counter()
    if kind == "rope":
        if dense_ok:
            ref = mods["rope_attn_pytorch"]
            cos, sin = ref.precompute_freqs_cis(D, N, THETA, device="cpu")
            for _ in range(n_units):
                q, k, v = (torch.randn((1, 1, N, D), generator=gen).requires_grad_(True) for _ in range(3))
                do = torch.randn((1, 1, N, D), generator=gen)
                o = ref.attention_pytorch(q, k, v, True, D ** -0.5, cos, sin)
                o.backward(do)
        else:
            cos, sin = oracle.precompute_freqs_cis(D, N, THETA)
            for _ in range(n_units):
                q, k, v, do = (torch.randn((1, 1, N, D), generator=gen) for _ in range(4))
                oracle.rope_attn_fwd_bwd_chunked(q, k, v, do, True, D ** -0.5, cos, sin, rows=1024 if N > 4096 else N)
        fl = 3.5 * flops_fwd(1, 1, N, D) * n_units
    else:
        for _ in range(n_units):
            q = torch.randn((1, G, N, D), generator=gen)
            k, v = (torch.randn((1, 1, N, D), generator=gen) for _ in range(2))
            do = torch.randn((1, G, N, D), generator=gen)
            if dense_ok:
                q, k, v = (t.requires_grad_(True) for t in (q, k, v))
                mods["corope_attn_gqa_pytorch"].attention_pytorch(q, k, v, True, D ** -0.5, THETA).backward(do)
            else:
                oracle.corope_gqa_fwd_bwd_chunked(q, k, v, do, D ** -0.5, THETA, rows=32)
        fl = 3.5 * flops_fwd(1, G, N, D) * n_units
    return time.perf_counter() - t0, fl, ("reference" if dense_ok else "port")


def run_reference_arm(args, wl, rank, world):
    kind, B, Hq, Hkv, N, D, dt = wl
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    units_per_step = args.ref_units
    for _ in range(args.warmup):
        cpu_reference_sample(kind, Hq, Hkv, N, D, 1)
    t_total, f_total, how = 0.0, 0.0, "port"
    for _ in range(args.steps):
        t, f, how = cpu_reference_sample(kind, Hq, Hkv, N, D, units_per_step)
        t_total += t
        f_total += f
    tf = f_total / t_total / 1e12
    sample = "%d of %d (batch, KV-head) units per step, fwd+bwd, fp32, %d torch threads, %s" % (
        units_per_step, B * Hkv, torch.get_num_threads(),
        "the reference's own attention_pytorch" if how == "reference" else "row-blocked CPU restatement of the reference")
    line = {
        "impl": "reference", "metric": metric_name(kind), "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_total / args.steps, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "Hq": Hq, "Hkv": Hkv, "N": N, "D": D, "causal": True, "sample": sample},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": how, "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def metric_name(kind):
    return "fused_rope_attn_fwd_bwd_causal_tflops" if kind == "rope" else "corope_gqa_attn_fwd_bwd_causal_tflops"


# ------------------------------------------------------------------------------------------------------------------
# timing helpers shared by the sweep and the Triton baseline
# ------------------------------------------------------------------------------------------------------------------
def timed_like_do_bench(fn, reps, flush):
    """The reference's method (triton.testing.do_bench, fused-rope/bench_compare.py:28-58): per repetition the L2 is flushed,
    then one call sits between two events; nothing synchronises until all repetitions are queued, so the host's launch work
    hides behind the flushes and the events see device time with a cold L2.  Returns the sorted times in ms."""
    for _ in range(3):
        fn()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    for a, b in ev:
        flush.zero_()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return sorted(a.elapsed_time(b) for a, b in ev)


# The 19 causal shapes of the reference's own comparison script (fused-rope/bench_compare.py:323-350): (B, H, N, D, name).
SWEEP_SHAPES = [
    (4, 8, 512, 64, "Small-512"), (4, 8, 1024, 64, "Small-1K"), (2, 8, 2048, 64, "Small-2K"), (2, 8, 4096, 64, "Small-4K"),
    (1, 8, 8192, 64, "Small-8K"),
    (4, 32, 512, 128, "Llama7B-512"), (4, 32, 1024, 128, "Llama7B-1K"), (2, 32, 2048, 128, "Llama7B-2K"), (2, 32, 4096, 128, "Llama7B-4K"),
    (1, 32, 8192, 128, "Llama7B-8K"), (1, 32, 16384, 128, "Llama7B-16K"),
    (2, 64, 512, 128, "Llama70B-512"), (2, 64, 1024, 128, "Llama70B-1K"), (1, 64, 2048, 128, "Llama70B-2K"), (1, 64, 4096, 128, "Llama70B-4K"),
    (1, 32, 8192, 128, "Llama70B-8K"),
    (1, 16, 32768, 128, "Long-32K"), (1, 8, 65536, 128, "Long-64K"), (1, 4, 131072, 128, "Long-128K"),
]


def _sweep_inputs(B, H, N, D, dev):
    gen = torch.Generator(device="cpu").manual_seed(7)
    q, k, v, do = (torch.randn((B, H, N, D), generator=gen, dtype=torch.float32).to(torch.float16).to(dev) for _ in range(4))
    import oracle
    cos, sin = oracle.precompute_freqs_cis(D, N, THETA)
    return q, k, v, do, cos.to(dev), sin.to(dev)


def run_sweep(args):
    """Forward / backward time and causal-adjusted TFLOP/s for the reference's shape list, one markdown row per shape
    (same FLOP convention as its report: 4 B H N^2 D / 2 forward, 2.5x that backward).  fp16 like the reference's run.
    With --sweep-triton the reference's Triton kernel (warp_specialize False, the setting of its own benchmark) is timed
    beside it on the same inputs by a child process per shape."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    pkg = importlib.import_module("co-rope_b200")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # larger than the 126 MB L2
    tri = args.sweep_triton
    # bring the GPU out of its idle clocks before the first (smallest) shape is timed
    wq, wk, wv, wdo, wcos, wsin = _sweep_inputs(2, 32, 2048, 128, dev)
    wcos, wsin = wcos[:, :64].contiguous(), wsin[:, :64].contiguous()
    t_w = time.time()
    while time.time() - t_w < 0.5:
        for _ in range(20):
            pkg.fused_rope_attention(wq, wk, wv, True, 0.5, wcos, wsin)
        torch.cuda.synchronize()
    del wq, wk, wv, wdo, wcos, wsin
    print("| configuration (B, H, N, D) | forward | backward | kernels |" + (" reference Triton forward | reference Triton backward | ours / Triton (fwd, bwd) |" if tri else ""))
    print("|---|---|---|---|" + ("---|---|---|" if tri else ""))
    for B, H, N, D, name in SWEEP_SHAPES:
        q, k, v, do, cos, sin = _sweep_inputs(B, H, N, D, dev)
        cos, sin = cos[:, : D // 2].contiguous(), sin[:, : D // 2].contiguous()
        reps = max(3, min(args.steps, 50))
        qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
        o = pkg.fused_rope_attention(qq, kk, vv, True, 0.5, cos, sin)
        f_ms = timed_like_do_bench(lambda: pkg.fused_rope_attention(qq, kk, vv, True, 0.5, cos, sin), reps, flush)
        b_ms = timed_like_do_bench(lambda: torch.autograd.grad(o, (qq, kk, vv), do, retain_graph=True), reps, flush)
        del o
        pkg.check_status()
        F = flops_fwd(B, H, N, D)
        f, b = f_ms[len(f_ms) // 2], b_ms[len(b_ms) // 2]
        fam = "tcgen05" if pkg._ext.lib().corope_last_kernel_family(0) == 1 else "cuda-core fp32"
        row = "| %s (%d, %d, %d, %d) | %.3f ms (%.1f TFLOP/s) | %.3f ms (%.1f TFLOP/s) | %s |" % (name, B, H, N, D, f, F / f / 1e9, b, 2.5 * F / b / 1e9, fam)
        del q, k, v, do, qq, kk, vv
        if tri:
            t = triton_baseline_child(["--shape", "%d,%d,%d,%d" % (B, H, N, D), "--steps", str(reps), "--ws", "0"], timeout=600)
            r = (t or {}).get("ws0") if isinstance(t, dict) else None
            if r and r.get("fwd_ms") and r.get("bwd_ms"):
                row += " %.3f ms (%.1f TFLOP/s) | %.3f ms (%.1f TFLOP/s) | %.2fx, %.2fx |" % (
                    r["fwd_ms"], F / r["fwd_ms"] / 1e9, r["bwd_ms"], 2.5 * F / r["bwd_ms"] / 1e9, r["fwd_ms"] / f, r["bwd_ms"] / b)
            else:
                why = (t or {}).get("unavailable") or (r or {}).get("error") or "no result"
                row += " unavailable: %s | | |" % str(why)[:120]
        print(row, flush=True)


# ------------------------------------------------------------------------------------------------------------------
# the reference's Triton kernels on this GPU (child process: Triton and its autotuner stay out of the product's process)
# ------------------------------------------------------------------------------------------------------------------
def run_triton_baseline(args):
    """Child mode: times the reference's unmodified Triton kernels (staged copy) at one shape, fp16 (the only dtype they
    take, fused_rope_attn.py:236, 379-380), sm_scale and timing method as in the sweep.  Prints one JSON object."""
    out = {}
    try:
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        reps = max(3, min(args.steps, 30))
        if args.shape:
            kind = "rope"
            B, H, N, D = [int(x) for x in args.shape.split(",")]
            Hkv = H
        else:
            kind, B, H, Hkv, N, D, _ = WORKLOADS[args.workload]
        F = flops_fwd(B, H, N, D)
        if kind == "rope":
            sys.path.insert(0, os.path.join(REF_COPY, "fused-rope"))
            import fused_rope_attn as ref_kernels   # the reference's module: this process never imports the package
            q, k, v, do, cos, sin = _sweep_inputs(B, H, N, D, dev)
            for ws in ([int(x) for x in args.ws.split(",")]):
                res = {}
                try:
                    qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
                    fn = lambda: ref_kernels.attention(qq, kk, vv, True, 0.5, cos, sin, bool(ws))
                    o = fn()
                    torch.cuda.synchronize()
                    f_ms = timed_like_do_bench(fn, reps, flush)
                    res["fwd_ms"] = f_ms[len(f_ms) // 2]
                    res["fwd_tflops"] = F / res["fwd_ms"] / 1e9
                    b_ms = timed_like_do_bench(lambda: torch.autograd.grad(o, (qq, kk, vv), do, retain_graph=True), reps, flush)
                    res["bwd_ms"] = b_ms[len(b_ms) // 2]
                    res["bwd_tflops"] = 2.5 * F / res["bwd_ms"] / 1e9
                except Exception as e:   # e.g. a Triton feature the installed version lacks on this GPU
                    res["error"] = "%s: %s" % (type(e).__name__, str(e)[:300])
                out["ws%d" % ws] = res
        else:
            # Not run: the reference's Co-RoPE Triton forward (corope-exp/flash_attn_co_rope_gqa_triton.py) did not return on
            # B200 with triton 3.6.0 at group size 4, D = 128 -- 900 s at N = 2048 and 150 s each at N = 128, 256, 512 passed
            # without the first call finishing (the GPU stayed usable; its own comparison script's small case does run and is
            # part of the tests).  Its backward is dense PyTorch (68.7 GB of temporaries at this shape).
            out = {"unavailable": "the reference's Co-RoPE Triton forward did not finish its first call within 900 s at this shape "
                                  "(nor within 150 s at N = 128) on B200 with triton 3.6.0; not run again"}
            print("TRITON_BASELINE " + json.dumps(out), flush=True)
            return
        out.update({"dtype": "f16", "shape": [B, H, Hkv, N, D], "sm_scale": 0.5 if kind == "rope" else D ** -0.5, "reps": reps,
                    "method": "L2 flushed before every call, CUDA events per call, median"})
        import triton
        out["triton"] = triton.__version__
    except Exception as e:
        out = {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:300])}
    print("TRITON_BASELINE " + json.dumps(out), flush=True)


def triton_baseline_child(extra, timeout=900):
    if not os.path.exists(os.path.join(REF_COPY, "fused-rope", "fused_rope_attn.py")):
        return {"unavailable": "no staged copy of the reference under baseline/_ref (the build step makes it where a checkout is present)"}
    cmd = [sys.executable, os.path.abspath(__file__), "--triton-baseline"] + extra
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    try:
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=timeout, env=env)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the reference's Triton kernels did not finish within %d s on this GPU" % timeout}
    for line in r.stdout.splitlines():
        if line.startswith("TRITON_BASELINE "):
            return json.loads(line[len("TRITON_BASELINE "):])
    return {"unavailable": "child exited %d: %s" % (r.returncode, (r.stderr or r.stdout)[-300:].replace("\n", " "))}


# ------------------------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweep", action="store_true", help="time the reference's 19 benchmark shapes (forward / backward) and print a table")
    ap.add_argument("--sweep-triton", action="store_true", help="with --sweep: also time the reference's Triton kernel per shape")
    ap.add_argument("--triton-baseline", action="store_true", help="child mode: time the reference's Triton kernels at --workload / --shape")
    ap.add_argument("--shape", default="", help="B,H,N,D for --triton-baseline")
    ap.add_argument("--ws", default="0,1", help="warp_specialize settings for --triton-baseline")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama7b-4k", choices=sorted(WORKLOADS))
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: strong = the workload's units are divided among the ranks; weak = every rank runs the whole workload")
    ap.add_argument("--ref-units", type=int, default=4, help="(batch, head) units per step of the CPU reference arm")
    ap.add_argument("--autograd", action="store_true", help="time the autograd entry points instead of the direct forward / backward helpers")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from Python instead of replaying CUDA graphs of the forward and the backward")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-triton", action="store_true", help="skip the child process that times the reference's Triton kernels")
    ap.add_argument("--no-sustained", action="store_true")
    ap.add_argument("--no-variants", action="store_true", help="skip timing the variant that rotates in the kernels (no rotated copies in HBM)")
    ap.add_argument("--sustained-seconds", type=float, default=2.5)
    ap.add_argument("--e2e-chunks", type=int, default=0, help="chunks of (batch, KV head) units in the host-to-host pipeline of the e2e figure (0: the pipeline's own choice)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    wl = WORKLOADS[args.workload]
    kind, B, Hq, Hkv, N, D, dt = wl
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.triton_baseline:
        run_triton_baseline(args)
        return
    if args.impl == "reference":
        run_reference_arm(args, wl, rank, world)
        return
    if args.sweep:
        if rank == 0:
            run_sweep(args)
        return

    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU path for the product kernels)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    pkg = importlib.import_module("co-rope_b200")
    lib = pkg._ext.lib()
    import oracle

    sampler = ClockSampler(local_rank)
    sampler.start()

    dtype = DTYPES[dt]
    G = Hq // Hkv
    n_units = B * Hkv
    strong = args.scaling == "strong"
    lo, hi = pkg.unit_range(n_units, rank, world) if strong else (0, n_units)
    my_units = list(range(lo, hi))
    seed = 1000 if strong else 1000 + rank
    n_loc = len(my_units)
    if n_loc == 0:
        raise RuntimeError("rank %d has no (batch, KV head) unit: %d units over %d ranks" % (rank, n_units, world))
    hq, hk, hv, hdo = (t.pin_memory() for t in unit_inputs(my_units, G, N, D, dtype, seed))
    # a rank's units as one batch entry with n_loc KV heads (units are independent, so this is the same computation)
    shp_q, shp_k = (1, n_loc * G, N, D), (1, n_loc, N, D)
    dq_, dk_, dv_, ddo = hq.to(dev).view(shp_q), hk.to(dev).view(shp_k), hv.to(dev).view(shp_k), hdo.to(dev).view(shp_q)
    sm_scale = D ** -0.5
    cos = sin = None
    if kind == "rope":
        cos, sin = oracle.precompute_freqs_cis(D, N, THETA)
        cos, sin = cos[:, : D // 2].contiguous().to(dev), sin[:, : D // 2].contiguous().to(dev)

    rope_mod = importlib.import_module("co-rope_b200.fused_rope_attn")
    gqa_mod = importlib.import_module("co-rope_b200.flash_attn_co_rope_gqa_triton")

    def step(qq, kk, vv, dd, evs=None):
        """One forward + backward.  Default: the package's forward / backward helpers (the entry points' checks and the C-ABI
        calls, without torch.autograd -- what the host pipeline and callers with their own backward pass use); their host cost
        is 0.1 ms per step, against 0.3 ms through autograd, which matters once a rank's share of the problem takes less than
        that on the GPU.  --autograd times the autograd entry points instead."""
        if args.autograd:
            qq.requires_grad_(True), kk.requires_grad_(True), vv.requires_grad_(True)
            if evs:
                evs[0].record()
            o = (pkg.fused_rope_attention(qq, kk, vv, True, sm_scale, cos, sin) if kind == "rope"
                 else pkg.corope_gqa_attention(qq, kk, vv, True, sm_scale, THETA))
            if evs:
                evs[1].record()
            g = torch.autograd.grad(o, (qq, kk, vv), dd)
            if evs:
                evs[2].record()
            return o, g
        if evs:
            evs[0].record()
        if kind == "rope":
            saved = rope_mod._forward(qq, kk, vv, True, sm_scale, cos, sin)
        else:
            saved = gqa_mod._forward(qq, kk, vv, True, sm_scale, THETA)
        if evs:
            evs[1].record()
        if kind == "rope":
            g = rope_mod._backward(*saved, dd, True, sm_scale)
        else:
            g = gqa_mod._backward(*saved, dd, sm_scale, THETA)
        if evs:
            evs[2].record()
        return saved[3], g

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def reduce_max(vals):
        if world == 1:
            return list(vals)
        t = torch.tensor(list(vals), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    graph_note = "launched from Python every step"
    last = None
    for _ in range(args.warmup):
        last = step(dq_, dk_, dv_, ddo)   # held like in the timed loop, so that the allocator's pool has its final size before timing starts
    sync_all()
    pkg.check_status()

    # ---------------------------------------------------------------- CUDA graphs of the step (one for the forward, one for the backward)
    # The library's calls are stream-ordered and allocate nothing, so a step can be captured once and replayed: the host then
    # spends a few microseconds per step instead of 0.1 ms, which is what a rank's share of a sharded problem needs once it
    # takes less than that on the GPU.  Every replay launches every kernel of the step.
    graph = None
    if not args.no_graph and not args.autograd:
        try:
            torch.cuda.synchronize()
            gf, gb = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            n0 = lib.corope_launch_count()
            with pkg._ext.batched_status(dev):   # the status mirror is refreshed once, after the captures
                with torch.cuda.graph(gf, capture_error_mode="relaxed"):
                    g_saved = (rope_mod._forward(dq_, dk_, dv_, True, sm_scale, cos, sin) if kind == "rope"
                               else gqa_mod._forward(dq_, dk_, dv_, True, sm_scale, THETA))
                with torch.cuda.graph(gb, pool=gf.pool(), capture_error_mode="relaxed"):
                    g_grads = (rope_mod._backward(*g_saved, ddo, True, sm_scale) if kind == "rope"
                               else gqa_mod._backward(*g_saved, ddo, sm_scale, THETA))
            per_step = lib.corope_launch_count() - n0
            gf.replay(), gb.replay()
            torch.cuda.synchronize()
            pkg.check_status()
            graph = {"fwd": gf, "bwd": gb, "launches_per_step": int(per_step)}
        except Exception as e:   # stay on the plain loop and say so in the line
            graph = None
            graph_note = "no graph (%s: %s)" % (type(e).__name__, str(e)[:120])
            torch.cuda.synchronize()

    # ---------------------------------------------------------------- the timed region: exactly `steps` steps
    launches0 = lib.corope_launch_count()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    t_timed0 = time.time()
    e0.record()
    if graph:
        for i in range(args.steps):
            evs[i][0].record()
            graph["fwd"].replay()
            evs[i][1].record()
            graph["bwd"].replay()
            evs[i][2].record()
        last = (g_saved[3], g_grads)
    else:
        for i in range(args.steps):
            last = step(dq_, dk_, dv_, ddo, evs[i])
    e1.record()
    torch.cuda.synchronize()
    t_timed1 = time.time()
    launches = graph["launches_per_step"] * args.steps if graph else lib.corope_launch_count() - launches0
    total_ms = e0.elapsed_time(e1)
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps
    total_ms, fwd_ms, bwd_ms = reduce_max([total_ms, fwd_ms, bwd_ms])
    if world > 1:
        dist.barrier()
    pkg.check_status()
    o_last, (gq_last, gk_last, gv_last) = last
    finite = all(bool(torch.isfinite(t).all()) for t in (o_last, gq_last, gk_last, gv_last))
    if not finite:
        raise RuntimeError("bench: a result of the timed steps is not finite")

    units_total = n_units if strong else n_units * world
    F_total = flops_fwd(1, units_total * G, N, D)          # whole job, forward
    ms_per_step = total_ms / args.steps
    value = 3.5 * F_total / (ms_per_step * 1e-3) / 1e12
    F_rank = flops_fwd(1, n_loc * G, N, D)                  # this rank's launch
    fwd_tf = F_total / (fwd_ms * 1e-3) / 1e12
    bwd_tf = 2.5 * F_total / (bwd_ms * 1e-3) / 1e12

    # ---------------------------------------------------------------- parity spot check of the timed step's results (one unit, CPU oracle)
    spot = None
    if rank == 0:
        u = 0
        sq, sk, sv, sdo = (t.cpu() for t in (dq_.detach()[:, u * G:(u + 1) * G], dk_.detach()[:, u:u + 1], dv_.detach()[:, u:u + 1], ddo[:, u * G:(u + 1) * G]))
        if kind == "rope":
            if N <= 8192:
                ro, _, rdq, rdk, rdv = oracle.rope_attn_fwd_bwd_chunked(sq, sk, sv, sdo, True, sm_scale, cos.cpu(), sin.cpu(), rows=1024)
                errs = {"o": (o_last[:, :G].float().cpu() - ro).abs().max().item(), "dq": (gq_last[:, :G].float().cpu() - rdq).abs().max().item(),
                        "dk": (gk_last[:, :1].float().cpu() - rdk).abs().max().item(), "dv": (gv_last[:, :1].float().cpu() - rdv).abs().max().item()}
            else:   # long context: the last block of 1024 query rows of the unit (O and dQ)
                blk = N // 1024 - 1
                ro, _, rdq, _, _ = oracle.rope_attn_fwd_bwd_chunked(sq, sk, sv, sdo, True, sm_scale, cos.cpu(), sin.cpu(), rows=1024, row_blocks=[blk])
                sl = slice(blk * 1024, (blk + 1) * 1024)
                errs = {"o": (o_last[:, :G, sl].float().cpu() - ro[:, :, sl]).abs().max().item(),
                        "dq": (gq_last[:, :G, sl].float().cpu() - rdq[:, :, sl]).abs().max().item()}
        else:
            blocks = [0, N // 64, N // 32 - 1]
            ro, _, _, rdq, _, _ = oracle.corope_gqa_fwd_bwd_chunked(sq, sk, sv, sdo, sm_scale, THETA, rows=32, row_blocks=blocks)
            errs = {"o": 0.0, "dq": 0.0}
            for b_ in blocks:
                sl = slice(b_ * 32, (b_ + 1) * 32)
                errs["o"] = max(errs["o"], (o_last[:, :G, sl].float().cpu() - ro[:, :, sl]).abs().max().item())
                errs["dq"] = max(errs["dq"], (gq_last[:, :G, sl].float().cpu() - rdq[:, :, sl]).abs().max().item())
        tol_f, tol_b = (1e-4, 2e-4) if dt == "f32" else (1e-2, 2e-2)
        spot = {"unit": u, "max_abs_err": errs, "ok": errs["o"] <= tol_f and all(v_ <= max(tol_b, 0.0) or k_ == "o" for k_, v_ in errs.items()),
                "note": "against the CPU oracle; gradients may exceed the absolute tolerance by one output ulp where |value| > 4 (see tests)"}

    # ---------------------------------------------------------------- strong scaling: gather the shards, compare with one GPU running everything
    shard_check = None
    if world > 1 and strong:
        per = (n_units + world - 1) // world

        def gather(t, heads_per_unit):   # [1, n_loc * g, N, D] -> [n_units * g, N, D] on every rank (NCCL; equal-size shards, padded if ragged)
            rows = per * heads_per_unit
            src = torch.zeros((rows, N, D), dtype=t.dtype, device=dev)
            src[: t.shape[1]] = t[0]
            dst = torch.empty((world * rows, N, D), dtype=t.dtype, device=dev)
            dist.all_gather_into_tensor(dst, src)
            if n_units % world == 0:
                return dst
            parts = []
            for r in range(world):
                l_, h_ = pkg.unit_range(n_units, r, world)
                parts.append(dst[r * rows: r * rows + (h_ - l_) * heads_per_unit])
            return torch.cat(parts, dim=0)

        g_o, g_dq = gather(o_last.detach(), G), gather(gq_last, G)
        g_dk, g_dv = gather(gk_last, 1), gather(gv_last, 1)
        torch.cuda.synchronize()
        if rank == 0:
            fq, fk, fv, fdo = (t.to(dev) for t in unit_inputs(list(range(n_units)), G, N, D, dtype, seed))
            fo, (fgq, fgk, fgv) = step(fq.view(1, n_units * G, N, D), fk.view(1, n_units, N, D), fv.view(1, n_units, N, D), fdo.view(1, n_units * G, N, D))
            torch.cuda.synchronize()
            pkg.check_status()
            shard_check = {
                "o_bit_identical": bool(torch.equal(fo[0], g_o)), "dk_bit_identical": bool(torch.equal(fgk[0], g_dk)),
                "dv_bit_identical": bool(torch.equal(fgv[0], g_dv)),
                "dq_max_abs_diff": (fgq[0].float() - g_dq.float()).abs().max().item(),
                "o_max_abs_diff": (fo[0].float() - g_o.float()).abs().max().item(),
                "dk_max_abs_diff": (fgk[0].float() - g_dk.float()).abs().max().item(),
                "dv_max_abs_diff": (fgv[0].float() - g_dv.float()).abs().max().item(),
                "collective": "all_gather_into_tensor (NCCL), outside the timed region",
                "against": "the same %d units run in one launch on rank 0" % n_units,
            }
            tol = 2e-2 if dt != "f32" else 2e-4
            shard_check["ok"] = all(shard_check[k_] <= tol for k_ in ("dq_max_abs_diff", "o_max_abs_diff", "dk_max_abs_diff", "dv_max_abs_diff"))
            del fq, fk, fv, fdo, fo, fgq, fgk, fgv
        del g_o, g_dq, g_dk, g_dv
        dist.barrier()

    # ---------------------------------------------------------------- seconds-long leg: sustained clocks, like-for-like with the sustained peak
    sustained = None
    if not args.no_sustained:
        n_sus = max(args.steps, int(args.sustained_seconds * 1e3 / max(ms_per_step, 1e-3)) + 1)
        sync_all()
        t_s0 = time.time()
        e0.record()
        for _ in range(n_sus):
            step(dq_, dk_, dv_, ddo)
        e1.record()
        torch.cuda.synchronize()
        t_s1 = time.time()
        (sus_ms,) = reduce_max([e0.elapsed_time(e1) / n_sus])
        pkg.check_status()
        sustained = {"steps": n_sus, "seconds": t_s1 - t_s0, "ms_per_step": sus_ms, "value": 3.5 * F_total / (sus_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                     "window": (t_s0, t_s1)}

    # ---------------------------------------------------------------- variant that keeps RoPE out of HBM (rotation inside the tensor-core kernels)
    variants = None
    if kind == "rope" and dt != "f32" and not args.no_variants:
        prev = lib.corope_set_kernel_policy(2)
        try:
            for _ in range(3):
                step(dq_, dk_, dv_, ddo)
            ev2 = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(max(3, min(args.steps, 10)))]
            sync_all()
            for e in ev2:
                step(dq_, dk_, dv_, ddo, e)
            torch.cuda.synchronize()
        finally:
            lib.corope_set_kernel_policy(prev)
        pkg.check_status()
        vf, vb = reduce_max([sum(e[0].elapsed_time(e[1]) for e in ev2) / len(ev2), sum(e[1].elapsed_time(e[2]) for e in ev2) / len(ev2)])
        variants = {"default": {"fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "what": "pre-pass writes rotated fp16 copies of K (forward) / Q (backward) to the workspace"},
                    "rotation_in_kernel": {"fwd_ms": vf, "bwd_ms": vb, "what": "K / Q tiles rotated in shared memory by the main kernels; nothing rotated reaches HBM"}}

    # ---------------------------------------------------------------- end to end: pinned host buffers -> device, forward + backward, results back
    e2e = None
    if not args.no_e2e:
        ho, hdq, hdk, hdv = (torch.empty_like(t).pin_memory() for t in (hq, hq, hk, hv))   # empty_like alone is pageable
        nb_in = int(sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo)))
        v4 = lambda t, g: t.view(1, n_loc * g, N, D)
        chunks = max(1, min(args.e2e_chunks, n_loc)) if args.e2e_chunks > 0 else pkg.host_pipeline.auto_chunks(2 * nb_in, n_loc)

        def e2e_step():   # the package's call for host tensors: chunks of (batch, KV head) units through copy-in / kernel / copy-out streams
            kw = dict(freqs_cos=cos, freqs_sin=sin) if kind == "rope" else dict(theta=THETA)
            pkg.attention_fwd_bwd_host(v4(hq, G), v4(hk, 1), v4(hv, 1), v4(hdo, G), sm_scale, out=(v4(ho, G), v4(hdq, G), v4(hdk, 1), v4(hdv, 1)), chunks=chunks, **kw)
        for _ in range(max(3, args.warmup)):
            e2e_step()
        sync_all()
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        (e2e_ms,) = reduce_max([e0.elapsed_time(e1) / args.steps])
        nb = lambda *ts: int(sum(t.numel() * t.element_size() for t in ts))
        e2e = {"value": 3.5 * F_total / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": nb(hq, hk, hv, hdo), "d2h_bytes_per_step": nb(ho, hdq, hdk, hdv),
               "bytes": "per rank" if world > 1 else "whole job",
               "copy_gbs_per_direction_per_rank": nb(hq, hk, hv, hdo) / (e2e_ms * 1e-3) / 1e9,
               "api": "attention_fwd_bwd_host", "chunks": chunks}
        pkg.check_status()

    sampler.stop()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    clocks = sampler.window(t_timed0, t_timed1)
    clocks["window"] = "timed region (%.0f ms)" % (1e3 * (t_timed1 - t_timed0))
    if sustained is not None:
        w0, w1 = sustained.pop("window")
        sc = sampler.window(w0 + 0.3, w1)     # skip the ramp of the first 0.3 s
        sustained["clocks"] = sc
        if clocks["samples"] < 3:             # the timed region is shorter than nvidia-smi's sampling period: report the run's load window as well
            clocks.update({"sm_mhz": sc["sm_mhz"] if clocks["sm_mhz"] is None else clocks["sm_mhz"], "sm_max_mhz": sc["sm_max_mhz"],
                           "reasons": sorted(set(clocks["reasons"]) | set(sc["reasons"])), "samples_sustained_leg": sc["samples"],
                           "sm_mhz_sustained_leg": sc["sm_mhz"]})

    peaks = load_peaks()
    if sustained is not None:
        sustained["value_per_gpu"] = sustained["value"] / world
        sustained["frac_of_sustained_peak"] = sustained["value"] / world / peaks["tflops_sustained"] if kind == "rope" else None
        sustained["peak_sustained"] = peaks["tflops_sustained"]
    dom_is_bwd = bwd_ms >= fwd_ms
    fam = lib.corope_last_kernel_family((1 if dom_is_bwd else 0) + (0 if kind == "rope" else 2))
    # per-launch figures of this rank's dominant kernel: algorithmic FLOPs of one launch over its average duration
    dom_ms = bwd_ms if dom_is_bwd else fwd_ms
    F_launch = (2.5 if dom_is_bwd else 1.0) * F_rank
    ach = F_launch / (dom_ms * 1e-3) / 1e12
    if kind == "rope":
        roofline = {
            "bound": "tensor", "kernel": "fused_rope_bwd" if dom_is_bwd else "fused_rope_fwd",
            "kernel_family": "tcgen05" if fam == 1 else "cuda-core fp32",
            "achieved": ach, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": ach / peaks["tflops"],
            "peak_source": peaks["source"] + " cuBLAS bf16 burst", "frac_of_sustained": ach / peaks["tflops_sustained"],
            "frac_of_nominal_2250": ach / 2250.0,
            "traffic": (NCU_DRAM_PER_TENSOR_BYTE["fused_rope_bwd" if dom_is_bwd else "fused_rope_fwd"] * dq_.numel() * dq_.element_size()
                        if fam == 1 else None),
            "traffic_unit": "bytes per launch (ncu capture of one launch at the Llama-7B-4K shape, scaled by tensor bytes for other sizes)",
            "algorithmic_flops": F_launch,
            "fwd": {"ms": fwd_ms, "tflops": F_rank / (fwd_ms * 1e-3) / 1e12, "frac": F_rank / (fwd_ms * 1e-3) / 1e12 / peaks["tflops"]},
            "bwd": {"ms": bwd_ms, "tflops": 2.5 * F_rank / (bwd_ms * 1e-3) / 1e12, "frac": 2.5 * F_rank / (bwd_ms * 1e-3) / 1e12 / peaks["tflops"]},
        }
    else:
        # Co-RoPE is bound by the special-function (XU) pipe: one sine and one cosine per (query, key <= query, frequency pair)
        # of a KV group, in the forward and again in the backward; 16 such operations per clock per SM.
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        clk = (clocks.get("sm_mhz") or peaks.get("sm_max_mhz") or 1965.0) * 1e6
        triples = n_loc * (N * (N + 1) / 2.0) * (D / 2)
        xu_peak = 16.0 * sms * 1965.0e6
        roofline = {
            "bound": "xu", "kernel": "corope_bwd" if dom_is_bwd else "corope_fwd",
            "kernel_family": "mma.sync contractions + cuda-core rotation" if fam == 1 else "cuda-core fp32",
            "achieved": 2.0 * triples / (dom_ms * 1e-3) / 1e12, "peak": xu_peak / 1e12, "unit": "T sin-or-cos/s",
            "frac": 2.0 * triples / (dom_ms * 1e-3) / xu_peak,
            "peak_source": "16 special-function results per clock per SM x %d SMs x 1965 MHz (nominal maximum clock)" % sms,
            "algorithmic_ops": 2.0 * triples, "traffic": None,
            "causal_tflops": ach, "causal_tflops_frac_of_tensor_peak": ach / peaks["tflops"],
            "fwd": {"ms": fwd_ms, "xu_frac": 2.0 * triples / (fwd_ms * 1e-3) / xu_peak, "tflops": F_rank / (fwd_ms * 1e-3) / 1e12},
            "bwd": {"ms": bwd_ms, "xu_frac": 2.0 * triples / (bwd_ms * 1e-3) / xu_peak, "tflops": 2.5 * F_rank / (bwd_ms * 1e-3) / 1e12},
        }
        del clk

    cpu_baseline = None
    if not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)   # torchrun pins OMP_NUM_THREADS to 1; the other ranks are done by now
        t1, f1, how = cpu_reference_sample(kind, Hq, Hkv, N, D, 1)
        n_cpu = int(max(1, min(B * Hkv, 12.0 / max(t1, 1e-3))))
        t, f, how = cpu_reference_sample(kind, Hq, Hkv, N, D, n_cpu)
        cpu_baseline = {"value": f / t / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": how,
                        "sample": "%d of %d (batch, KV-head) units, fwd+bwd, fp32, %.1f s, %s" % (
                            n_cpu, B * Hkv, t, "the reference's own attention_pytorch" if how == "reference" else "row-blocked CPU restatement")}

    triton_baseline = None
    if world == 1 and not args.no_triton:
        triton_baseline = triton_baseline_child(["--workload", args.workload, "--steps", str(max(5, min(args.steps, 20)))])
        if kind == "rope" and isinstance(triton_baseline, dict) and "ws0" in triton_baseline:
            triton_baseline["note"] = "reference fused_rope_attn.attention, fp16, sm_scale 0.5, same shape; ours in the main line is bf16, sm_scale 1/sqrt(D)"

    line = {
        "metric": metric_name(kind),
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": dt, "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "Hq": Hq, "Hkv": Hkv, "N": N, "D": D, "causal": True, "sm_scale": sm_scale,
                   "theta": THETA, "units_total": units_total, "units_per_gpu": n_loc,
                   "api": "autograd entry points" if args.autograd else
                          ("forward / backward helpers of the drop-in modules (C-ABI calls without torch.autograd)" +
                           (", captured once as two CUDA graphs and replayed every step" if graph else ", " + graph_note)),
                   "partition": ("(batch, KV head) units %d..%d of %d on rank 0; no data-path collective" % (lo, hi - 1, n_units)) if strong else "every rank runs all units",
                   "l2": "inputs+outputs per step (%.0f MB per GPU) %s the 126 MB L2" %
                   (8 * dq_.numel() * dq_.element_size() / 1e6, "exceed" if 8 * dq_.numel() * dq_.element_size() > 126e6 else "do NOT exceed")},
        "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "fwd_tflops": fwd_tf, "bwd_tflops": bwd_tf,
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu_baseline,
        "sustained": sustained, "variants": variants, "triton_baseline": triton_baseline, "parity_spot": spot, "shard_check": shard_check,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
