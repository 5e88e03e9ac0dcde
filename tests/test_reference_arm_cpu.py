"""The reference arm of ``bench.py`` on a tiny model on the CPU: the unmodified reference library is
importable through the stand-in packages, its training loop runs, and the JSON line has the fields the
benchmark contract names. Skipped where the reference is not installed under ``baseline/_ref``."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(not (ROOT / "baseline" / "_ref" / "keys_values").is_dir(), reason="reference not installed under baseline/_ref")
def test_reference_arm_runs_tiny_model_on_cpu():
    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--ref-allow-cpu", "--model", "tiny-qwen3", "--seq-len", "384",
           "--cache-length", "128", "--chunk-size", "64", "--num-targets", "64", "--steps", "1", "--warmup", "1"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT, env={**__import__("os").environ, "CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1]
    out = json.loads(line)
    assert out["impl"] == "reference" and "unavailable" not in out, out
    assert out["steps"] == 1 and out["value"] > 0 and out["e2e"]["value"] > 0
    assert 5.0 < out["loss"] < 7.5  # ln(512) = 6.24 for random weights
    # nothing of this repository's package may be loaded on the reference path
    probe = ("import sys; sys.argv=['bench.py','--impl','reference']; sys.path.insert(0, %r); "
             "import baseline.reference_arm as ra; ra._import_reference(); "
             "print(any(m.startswith('keys_values_b200') for m in sys.modules))" % str(ROOT))
    r = subprocess.run([sys.executable, "-c", probe], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0 and r.stdout.strip().endswith("False"), r.stdout + r.stderr


def test_reference_arm_reports_unavailable_without_gpu():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT, env={**__import__("os").environ, "CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0
    out = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])
    assert out["impl"] == "reference" and "unavailable" in out


@pytest.mark.skipif(not (ROOT / "baseline" / "_ref" / "keys_values").is_dir(), reason="reference not installed under baseline/_ref")
def test_reference_arm_runs_on_two_ranks():
    """The launch the benchmark driver uses for N > 1 (``torch.distributed.run``), on two CPU ranks over gloo: the
    reference's gradient all-reduce through the stand-in Fabric, one JSON line from rank 0."""
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(ROOT / "bench.py"), "--impl", "reference", "--ref-allow-cpu", "--gpus", "2", "--model",
           "tiny-qwen3", "--seq-len", "384", "--cache-length", "128", "--chunk-size", "64", "--num-targets", "64", "--steps", "1",
           "--warmup", "1"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT, env={**__import__("os").environ, "CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, lines
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and "unavailable" not in out, out
    assert out["n_gpus"] == 2 and out["value"] > 0


@pytest.mark.skipif(not (ROOT / "baseline" / "_ref" / "keys_values").is_dir(), reason="reference not installed under baseline/_ref")
def test_reference_inference_arm_runs_tiny_model_on_cpu():
    """The inference configuration through the reference's own generation path (chunked prompt pass, eager steps)."""
    cmd = [sys.executable, str(ROOT / "bench.py"), "--config", "inference", "--impl", "reference", "--ref-allow-cpu", "--model", "tiny-qwen3",
           "--seq-len", "384", "--cache-length", "128", "--chunk-size", "64", "--batch", "2", "--decode", "6"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT, env={**__import__("os").environ, "CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    out = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])
    assert out["impl"] == "reference" and "unavailable" not in out, out
    assert out["config"]["decode_tokens"] == 6 and out["prefill_tokens_per_s"] > 0 and out["decode_tokens_per_s"] > 0
