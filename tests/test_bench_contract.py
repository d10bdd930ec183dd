"""The benchmark's reference arm (the CPU restatement on the host cores) runs without a GPU and prints
one JSON line with the agreed keys; ranks other than 0 print nothing."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _run(env_extra=None):
    env = dict(os.environ, **(env_extra or {}))
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "tiny",
                          "--gpus", "2", "--steps", "2", "--warmup", "1"], capture_output=True, text=True, env=env,
                         timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    return [l for l in out.stdout.splitlines() if l.startswith("{")]


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    lines = _run()
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "kv_swap_GBps" and d["unit"] == "GB/s"
    assert d["higher_is_better"] is True and d["scaling"] == "weak" and d["vs_baseline"] is None
    assert d["dtype"] == "u8" and d["data"] == "synthetic" and d["n_gpus"] == 2 and d["steps"] >= 1
    assert d["config"]["workload"] == "tiny" and d["value"] > 0 and d["ms_per_step"] > 0
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and "sample" in cb
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_is_silent_on_other_ranks():
    assert _run({"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"}) == []


def test_geometry_byte_counts_match_the_configurations():
    sys.path.insert(0, str(ROOT))
    import bench

    assert bench.geometry("llama3_8b_swap").swap_bytes == 1_073_741_824
    assert bench.geometry("llama3_70b_tp8_swap").swap_bytes == 10_737_418_240
    g = bench.geometry("qwen2_7b_fp8_prefetch")
    assert g.block_bytes == 8192 and g.n_swap * 2 * g.block_bytes == 4_194_304
