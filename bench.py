"""Benchmark of the fused-RoPE attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one forward + backward pass of fused-RoPE causal attention over one synthetic batch of the
workload (default: the Llama-7B-4K shape, B=2 H=32 N=4096 D=128 bf16).  The metric is causal-adjusted
TFLOP/s with the FLOP convention of the reference's benchmark driver (fused-rope/bench_compare.py:61-86):
F_fwd = 4*B*H*N^2*D*0.5, F_bwd = 2.5*F_fwd.  With N > 1 GPUs (torchrun, one rank per GPU) every rank
runs the full workload on its own seeded batch (weak scaling; the (batch, head) units are independent, so
there is no data-path collective) and `value` is the sum over ranks divided by the slowest rank's time.

One JSON line is printed by rank 0.  `--impl reference` times the CPU oracle (the restatement of the
reference's PyTorch path) on the host cores instead.
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

# DRAM bytes per launch of the two tensor-core kernels, from one ncu capture each (dram__bytes_read.sum +
# dram__bytes_write.sum) at B=2 H=64 N=1024 D=128 bf16 -- 112.2 MB forward, 288.4 MB backward -- expressed per byte of
# one [B,H,N,D] bf16 tensor (33.55 MB there).  Traffic of these kernels is proportional to the tensor bytes as long as a
# head's K/V (and, backward, its fp32 dQ rows) fit in L2, which holds for every workload here.
NCU_DRAM_PER_TENSOR_BYTE = {"fused_rope_fwd": 112.2 / 33.55, "fused_rope_bwd": 288.4 / 33.55}


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
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.rows = []
        self.proc = None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            ident = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            ident = str(device_index)
        self.cmd = ["nvidia-smi", "-i", ident, "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "100"]

    def start(self):
        try:
            self.proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            parts = [x.strip() for x in r.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_inputs(kind, B, Hq, Hkv, N, D, dtype, seed, device):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    def draw(shape):
        return torch.randn(shape, generator=gen, dtype=torch.float32).to(dtype)
    q = draw((B, Hq, N, D))
    k = draw((B, Hkv, N, D))
    v = draw((B, Hkv, N, D))
    do = draw((B, Hq, N, D))
    return q, k, v, do


def cpu_oracle_sample(kind, B, Hq, Hkv, N, D, n_units, threads=None):
    """Times the CPU oracle (fwd + bwd) on `n_units` (batch, KV head) units of the workload.  Returns seconds and FLOPs."""
    import oracle

    if threads:
        torch.set_num_threads(threads)
    G = Hq // Hkv
    gen = torch.Generator().manual_seed(1234)
    t0 = time.perf_counter()
    if kind == "rope":
        cos, sin = oracle.precompute_freqs_cis(D, N, THETA)
        for _ in range(n_units):
            q, k, v, do = (torch.randn((1, 1, N, D), generator=gen) for _ in range(4))
            rows = 1024 if N > 4096 else N
            oracle.rope_attn_fwd_bwd_chunked(q, k, v, do, True, D ** -0.5, cos, sin, rows=rows)
        fl = 3.5 * flops_fwd(1, 1, N, D) * n_units
    else:
        for _ in range(n_units):
            q = torch.randn((1, G, N, D), generator=gen)
            k, v = (torch.randn((1, 1, N, D), generator=gen) for _ in range(2))
            do = torch.randn((1, G, N, D), generator=gen)
            oracle.corope_gqa_fwd_bwd_chunked(q, k, v, do, D ** -0.5, THETA, rows=32)
        fl = 3.5 * flops_fwd(1, G, N, D) * n_units
    return time.perf_counter() - t0, fl


def run_reference_arm(args, wl, rank, world):
    kind, B, Hq, Hkv, N, D, dt = wl
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    units_per_step = args.ref_units
    for _ in range(args.warmup):
        cpu_oracle_sample(kind, B, Hq, Hkv, N, D, 1)
    t_total, f_total = 0.0, 0.0
    for _ in range(args.steps):
        t, f = cpu_oracle_sample(kind, B, Hq, Hkv, N, D, units_per_step)
        t_total += t
        f_total += f
    tf = f_total / t_total / 1e12
    sample = "%d of %d (batch, KV-head) units per step, fwd+bwd, fp32, %d torch threads" % (units_per_step, B * Hkv, torch.get_num_threads())
    line = {
        "impl": "reference", "metric": "fused_rope_attn_fwd_bwd_causal_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "Hq": Hq, "Hkv": Hkv, "N": N, "D": D, "causal": True, "sample": sample},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


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


def run_sweep(args):
    """Forward / backward time and causal-adjusted TFLOP/s for the reference's shape list, one markdown row per shape
    (same FLOP convention as its report: 4 B H N^2 D / 2 forward, 2.5x that backward).  fp16 like the reference's run."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    pkg = importlib.import_module("co-rope_b200")
    import oracle
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # larger than the 126 MB L2
    print("| configuration (B, H, N, D) | forward | backward | kernels |")
    print("|---|---|---|---|")
    for B, H, N, D, name in SWEEP_SHAPES:
        q, k, v, do = (t.to(dev) for t in make_inputs("rope", B, H, H, N, D, torch.float16, 7, dev))
        cos, sin = oracle.precompute_freqs_cis(D, N, THETA)
        cos, sin = cos[:, : D // 2].contiguous().to(dev), sin[:, : D // 2].contiguous().to(dev)
        reps = max(3, min(args.steps, 50))
        qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
        o = pkg.fused_rope_attention(qq, kk, vv, True, 0.5, cos, sin)

        def timed(fn):
            # the reference's method (triton.testing.do_bench, fused-rope/bench_compare.py:28-58): per repetition the L2 is
            # flushed, then one call sits between two events; nothing synchronises until all repetitions are queued, so
            # the host's launch work hides behind the flushes and the events see device time with a cold L2
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

        f_ms = timed(lambda: pkg.fused_rope_attention(qq, kk, vv, True, 0.5, cos, sin))
        b_ms = timed(lambda: torch.autograd.grad(o, (qq, kk, vv), do, retain_graph=True))
        del o
        pkg.check_status()
        F = flops_fwd(B, H, N, D)
        f, b = sorted(f_ms)[len(f_ms) // 2], sorted(b_ms)[len(b_ms) // 2]
        fam = "tcgen05" if pkg._ext.lib().corope_last_kernel_family(0) == 1 else "cuda-core fp32"
        print("| %s (%d, %d, %d, %d) | %.3f ms (%.1f TFLOP/s) | %.3f ms (%.1f TFLOP/s) | %s |"
              % (name, B, H, N, D, f, F / f / 1e9, b, 2.5 * F / b / 1e9, fam), flush=True)
        del q, k, v, do


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweep", action="store_true", help="time the reference's 19 benchmark shapes (forward / backward) and print a table")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama7b-4k", choices=sorted(WORKLOADS))
    ap.add_argument("--ref-units", type=int, default=4, help="(batch, head) units per step of the CPU reference arm")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-chunks", type=int, default=16, help="chunks of (batch, KV head) units in the host-to-host pipeline of the e2e figure")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    wl = WORKLOADS[args.workload]
    kind, B, Hq, Hkv, N, D, dt = wl
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

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

    dtype = DTYPES[dt]
    q, k, v, do = make_inputs(kind, B, Hq, Hkv, N, D, dtype, 1000 + rank, dev)
    hq, hk, hv, hdo = (t.pin_memory() for t in (q, k, v, do))
    dq_, dk_, dv_, ddo = (t.to(dev) for t in (q, k, v, do))
    sm_scale = D ** -0.5
    if kind == "rope":
        cos, sin = oracle.precompute_freqs_cis(D, N, THETA)
        cos, sin = cos[:, : D // 2].contiguous().to(dev), sin[:, : D // 2].contiguous().to(dev)

    def fwd(qq, kk, vv):
        if kind == "rope":
            return pkg.fused_rope_attention(qq, kk, vv, True, sm_scale, cos, sin)
        return pkg.corope_gqa_attention(qq, kk, vv, True, sm_scale, THETA)

    def step(qq, kk, vv, dd, evs=None):
        qq.requires_grad_(True), kk.requires_grad_(True), vv.requires_grad_(True)
        if evs:
            evs[0].record()
        o = fwd(qq, kk, vv)
        if evs:
            evs[1].record()
        g = torch.autograd.grad(o, (qq, kk, vv), dd)
        if evs:
            evs[2].record()
        return o, g

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(dq_, dk_, dv_, ddo)
    sync_all()
    pkg.check_status()

    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = lib.corope_launch_count()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for i in range(args.steps):
        step(dq_, dk_, dv_, ddo, evs[i])
    e1.record()
    torch.cuda.synchronize()
    launches = lib.corope_launch_count() - launches0
    total_ms = e0.elapsed_time(e1)
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps
    if world > 1:
        t = torch.tensor([total_ms, fwd_ms, bwd_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, fwd_ms, bwd_ms = t.tolist()
        dist.barrier()
    clocks = sampler.stop()
    pkg.check_status()

    F = flops_fwd(B, Hq, N, D)
    ms_per_step = total_ms / args.steps
    value = world * 3.5 * F / (ms_per_step * 1e-3) / 1e12
    fwd_tf = F / (fwd_ms * 1e-3) / 1e12
    bwd_tf = 2.5 * F / (bwd_ms * 1e-3) / 1e12

    # end to end: pinned host buffers -> device, forward + backward, results back to pinned host buffers
    e2e = None
    if not args.no_e2e:
        ho, hdq, hdk, hdv = (torch.empty_like(t).pin_memory() for t in (hq, hq, hk, hv))   # empty_like alone is pageable
        def e2e_step():   # the package's call for host tensors: chunks of (batch, KV head) units through copy-in / kernel / copy-out streams
            if kind == "rope":
                pkg.attention_fwd_bwd_host(hq, hk, hv, hdo, sm_scale, freqs_cos=cos, freqs_sin=sin, out=(ho, hdq, hdk, hdv), chunks=args.e2e_chunks)
            else:
                pkg.attention_fwd_bwd_host(hq, hk, hv, hdo, sm_scale, theta=THETA, out=(ho, hdq, hdk, hdv), chunks=args.e2e_chunks)
        for _ in range(max(3, args.warmup)):
            e2e_step()
        sync_all()
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = e0.elapsed_time(e1) / args.steps
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = t.item()
        nb = lambda *ts: int(sum(t.numel() * t.element_size() for t in ts))
        e2e = {"value": world * 3.5 * F / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": nb(hq, hk, hv, hdo), "d2h_bytes_per_step": nb(ho, hdq, hdk, hdv),
               "api": "attention_fwd_bwd_host", "chunks": args.e2e_chunks}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    dom_is_bwd = bwd_ms >= fwd_ms
    fam = lib.corope_last_kernel_family((1 if dom_is_bwd else 0) + (0 if kind == "rope" else 2))
    roofline = {
        "bound": "tensor", "kernel": ("fused_rope_bwd" if dom_is_bwd else "fused_rope_fwd") if kind == "rope" else ("corope_bwd" if dom_is_bwd else "corope_fwd"),
        "kernel_family": ("tcgen05" if kind == "rope" else "mma.sync contractions + cuda-core rotation") if fam == 1 else "cuda-core fp32",
        "achieved": bwd_tf if dom_is_bwd else fwd_tf, "peak": peaks["tflops"], "unit": "TFLOP/s",
        "frac": (bwd_tf if dom_is_bwd else fwd_tf) / peaks["tflops"], "peak_source": peaks["source"] + " cuBLAS bf16 burst",
        "frac_of_sustained": (bwd_tf if dom_is_bwd else fwd_tf) / peaks["tflops_sustained"],
        "frac_of_nominal_2250": (bwd_tf if dom_is_bwd else fwd_tf) / 2250.0,
        "traffic": (NCU_DRAM_PER_TENSOR_BYTE["fused_rope_bwd" if dom_is_bwd else "fused_rope_fwd"] * q.numel() * q.element_size()
                    if (kind == "rope" and fam == 1) else None),
        "traffic_unit": "bytes per launch (ncu capture at N=1024, scaled by tensor bytes)",
        "algorithmic_flops": (2.5 * F if dom_is_bwd else F),
        "fwd": {"ms": fwd_ms, "tflops": fwd_tf, "frac": fwd_tf / peaks["tflops"]},
        "bwd": {"ms": bwd_ms, "tflops": bwd_tf, "frac": bwd_tf / peaks["tflops"]},
    }

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        t1, f1 = cpu_oracle_sample(kind, B, Hq, Hkv, N, D, 1)
        n_units = int(max(1, min(B * Hkv, 12.0 / max(t1, 1e-3))))
        t, f = cpu_oracle_sample(kind, B, Hq, Hkv, N, D, n_units)
        cpu_baseline = {"value": f / t / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                        "sample": "%d of %d (batch, KV-head) units, fwd+bwd, fp32 oracle, %.1f s" % (n_units, B * Hkv, t)}

    line = {
        "metric": "fused_rope_attn_fwd_bwd_causal_tflops" if kind == "rope" else "corope_gqa_attn_fwd_bwd_causal_tflops",
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dt, "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "Hq": Hq, "Hkv": Hkv, "N": N, "D": D, "causal": True, "sm_scale": sm_scale,
                   "theta": THETA, "units_per_gpu": B * Hkv, "l2": "inputs+outputs per step (%.0f MB) exceed the 126 MB L2" %
                   (8 * q.numel() * q.element_size() / 1e6)},
        "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "fwd_tflops": fwd_tf, "bwd_tflops": bwd_tf,
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu_baseline,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
