"""bench.py on a machine without a GPU: the reference arm's JSON line (the reference's own attention_pytorch on the host
cores, or the CPU restatement where no staged copy of the reference exists) and the FLOP conventions of the line."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench_module():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_flop_convention_and_workloads():
    b = _bench_module()
    # causal-adjusted forward FLOPs as in the reference's report (fused-rope/bench_compare.py:280-292): 4 B H N^2 D / 2
    assert b.flops_fwd(2, 32, 4096, 128) == 4.0 * 2 * 32 * 4096 * 4096 * 128 * 0.5
    kind, B, Hq, Hkv, N, D, _ = b.WORKLOADS["llama7b-4k"]
    assert (kind, B, Hq, Hkv, N, D) == ("rope", 2, 32, 32, 4096, 128)
    kind, B, Hq, Hkv, N, D, _ = b.WORKLOADS["corope-gqa-2k"]
    assert (kind, B, Hq, Hkv, N, D) == ("corope", 2, 32, 8, 2048, 128)
    assert len(b.SWEEP_SHAPES) == 19   # the reference's comparison script lists 19 shapes (bench_compare.py:323-350)


def test_reference_arm_prints_the_contract_line():
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0", "--ref-units", "1"],
                       stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "fused_rope_attn_fwd_bwd_causal_tflops" and d["unit"] == "TFLOP/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1
    assert d["value"] > 0 and d["config"]["workload"] == "llama7b-4k"
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0
