"""The benchmark's reference arm (the CPU restatement of the reference path on the host cores) runs without a GPU
and prints one JSON line with the keys the two arms share."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_shared_json_line():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                          capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "paged GQA decode tokens/s" and line["unit"] == "tokens/s"
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["higher_is_better"] is True and line["value"] > 0
    assert line["config"]["workload"] == "paged_decode_llama3_8b_layer" and line["config"]["n_seqs"] == 64
    cb = line["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
