"""bench.py's command line on a machine without a GPU: the reference arm runs the CPU oracle and prints
the one JSON line of the contract; arms that need a GPU refuse combinations they cannot measure."""

import json
import os
import subprocess
import sys

from tests.conftest import ROOT


def _run(*args):
    env = dict(os.environ, RANK="0", WORLD_SIZE="1")
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          env=env, timeout=600)


def test_reference_arm_prints_contract_line():
    r = _run("--impl", "reference", "--workload", "c1", "--steps", "1", "--warmup", "1")
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "hc_fwd_bwd_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["value"] > 0 and line["steps"] == 1
    have_ref = os.path.exists(os.path.join(ROOT, "baseline", "_ref", "mhc", "_torch_baseline.py"))
    assert line["cpu_baseline"]["kind"] == ("reference" if have_ref else "port") and line["cpu_baseline"]["cores"] >= 1
    assert set(line["config"]) >= {"workload", "global_tokens", "sharding", "per_gpu_batch", "layers", "cuda_graph"}
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["e2e"]["value"] == line["value"]


def test_per_token_workload_is_single_gpu_and_ours_only():
    r = _run("--impl", "reference", "--workload", "per_token")
    assert r.returncode != 0 and "single-GPU" in (r.stderr + r.stdout)
    r = _run("--workload", "per_token", "--gpus", "2")
    assert r.returncode != 0 and "single-GPU" in (r.stderr + r.stdout)
