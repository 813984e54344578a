"""The benchmark's contract on a machine without a GPU: the reference arm (the CPU restatement of the
step, timed on the host cores) prints one JSON line with the agreed keys, on the same `config` as the
GPU arm would print; ranks other than 0 stay silent; the small CPU configuration runs in full."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _run(extra_env=None):
    env = dict(os.environ, **(extra_env or {}))
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    return [ln for ln in out.stdout.splitlines() if ln.startswith("{")]


def test_reference_arm_prints_the_agreed_line():
    sys.path.insert(0, str(ROOT))
    import bench

    lines = _run()
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "decode_tokens_per_s" and line["unit"] == "tok/s"
    assert line["higher_is_better"] is True and line["scaling"] == "strong" and line["vs_baseline"] is None
    assert line["steps"] == 1 and line["warmup"] == 1 and line["n_gpus"] == 1 and line["value"] > 0
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] == os.cpu_count() and cb["value"] == line["value"] and "layer" in cb["sample"]
    # the same configuration record as the GPU arm prints for these arguments
    saved = sys.argv
    try:
        sys.argv = ["bench.py", "--steps", "1", "--warmup", "1"]
        args = bench.parse_args()
    finally:
        sys.argv = saved
    assert line["config"] == bench.config_dict(args, 1)
    assert line["config"]["workload"] == "llama3-70b-pipeline" and line["config"]["kv_step"]["workload"] == "llama3-8b-decode-kv"


def test_reference_arm_is_silent_on_other_ranks():
    assert _run({"RANK": "3", "WORLD_SIZE": "8", "LOCAL_RANK": "3"}) == []


def test_small_cpu_configuration_runs_in_full():
    sys.path.insert(0, str(ROOT))
    import bench

    r = bench.cpu_config1_full()
    assert r["steps"] == 32 and r["sequences"] == 4 and r["value"] > 0
