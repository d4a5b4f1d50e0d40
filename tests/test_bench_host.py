"""Host-side pieces of bench.py that need no GPU: the CPU reference arm end to end on the tiny workload, the `config`
object both arms share, and the small helpers."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load_bench():
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_the_contract_line_on_cpu():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--cfg", "1",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["metric"] == "fwd+bwd lattice-nodes/sec" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["config"]["workload"].startswith("tiny") and line["config"]["lattice_nodes"] == 1523


def test_both_arms_name_the_same_workload():
    bench = _load_bench()
    for world in (1, 2, 8):
        a = bench.workload_config(2, world, "weak", "pipeline")
        b = bench.workload_config(2, world, "weak", "pipeline")
        assert a == b and a["global_sequences"] == 32 * world and a["reduction"] == "mean"
        assert a["logits_bytes_per_gpu"] > (126 << 20) and "larger than L2" in a["l2"]
    strong = bench.workload_config(5, 4, "strong", "pipeline")
    assert strong["global_sequences"] == 256 and strong["shard_imbalance"] < 1.05
    small = bench.workload_config(5, 1, "weak", "pipeline", sequences=8)
    assert small["global_sequences"] == 8


def test_spread_and_numa_helpers():
    bench = _load_bench()
    sp = bench.spread([10.0, 12.0, 11.0], 10)
    assert sp == {"median": 1.1, "min": 1.0, "max": 1.2, "blocks": 3, "steps_per_block": 10}
    import numpy as np
    buf = np.ones(1 << 20, dtype=np.uint8)
    where = bench.numa_of(buf.ctypes.data)
    assert where is None or all(k.startswith("N") and v >= 0 for k, v in where.items())
