"""The example scripts run end to end on CPU (tiny models, gloo group of one)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29591")
    return subprocess.run([sys.executable, *args], cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)


def test_calibrate_mask_example():
    r = _run("examples/calibrate_mask.py")
    assert r.returncode == 0, r.stderr[-2000:]
    assert "drivers" in r.stdout and "max error" in r.stdout


def test_ddp_example_on_cpu(tmp_path):
    ck = str(tmp_path / "run.pt")
    r = _run("examples/train_ddp_gpt2.py", "--tiny", "--steps", "12", "--warmup-steps", "2", "--micro-batch", "2",
             "--checkpoint", ck, "--save-every", "6")
    assert r.returncode == 0, r.stderr[-2000:]
    assert "compressing True" in r.stdout
    assert os.path.exists(ck + ".rank0")
    # resume from the checkpoint: starts at step 12, nothing left to do, exits cleanly
    r = _run("examples/train_ddp_gpt2.py", "--tiny", "--steps", "14", "--warmup-steps", "2", "--micro-batch", "2",
             "--checkpoint", ck)
    assert r.returncode == 0, r.stderr[-2000:]


def test_spice_partitioned_example():
    r = _run("examples/spice_partitioned.py", "--stages", "40", "--partitions", "3", "--tstop", "1e-10")
    assert r.returncode == 0, r.stderr[-2000:]
    assert "partitioned_validated" in r.stdout and ".nz v2" in r.stdout


def test_manual_reducer_example_on_cpu():
    r = _run("examples/train_manual_reducer.py", "--cpu", "--steps", "16", "--warmup-steps", "4")
    assert r.returncode == 0, r.stderr[-2000:]
    assert "bytes held / bytes sent" in r.stdout
    first, last = (float(x) for x in (r.stdout.split("first loss ")[1].split()[0], r.stdout.split("last loss ")[1].split()[0]))
    assert last < first   # it learns through the packet path


def test_hook_benchmark_example_reports_ratio_and_error():
    r = _run("examples/benchmark.py", "--size", "50000", "--iterations", "8", "--warmup-steps", "2")
    assert r.returncode == 0, r.stdout + r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["compression_ratio"] > 6.0 and out["relative_rms_error"] < 5e-3 and out["compress_melem_per_s"] > 0
