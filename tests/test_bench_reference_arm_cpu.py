"""The reference arm of bench.py (the CPU oracle timed on the host cores) needs no GPU:
check that it runs on the small workload and prints one JSON line with the agreed keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(extra_env=None):
    env = dict(os.environ)
    env.update(extra_env or {})
    out = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
         "--workload", "c1", "--steps", "1", "--warmup", "0"],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    return out


def test_reference_arm_prints_one_contract_line():
    out = _run()
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference"
    assert rec["metric"] == "fused_fa_oproj_ar_prefill_tflops" and rec["unit"] == "TFLOP/s"
    assert rec["higher_is_better"] is True and rec["n_gpus"] == 1
    assert rec["steps"] == 1 and rec["warmup"] == 0
    assert rec["value"] > 0 and rec["ms_per_step"] > 0
    cb = rec["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == rec["value"]
    assert "sample" in cb
    e2e = rec["e2e"]
    assert e2e["value"] == rec["value"] and e2e["unit"] == rec["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_reference_arm_other_ranks_exit_without_work():
    # under torchrun only rank 0 runs the CPU sample; the others print nothing and exit 0
    out = _run({"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert out.returncode == 0, out.stderr[-2000:]
    assert not [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
