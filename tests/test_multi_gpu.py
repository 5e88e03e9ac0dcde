"""Multi-rank tests. On a machine with >= 2 GPUs the ranks use NCCL for the plumbing
and the framework's peer-memory kernels for the data path; without GPUs the
host-side logic of the data-parallel path runs on 2 gloo ranks."""
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

WORKER = str(Path(__file__).resolve().parent / "dist_worker.py")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(case: str, world: int, timeout: int = 300):
    port = _free_port()
    procs = [subprocess.Popen([sys.executable, WORKER, case, str(r), str(world), str(port)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=timeout)
            outs.append(out)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert "OK" in outs[0], outs[0]


def test_dp_gradients_match_on_cpu_ranks():
    _run("dp_train", 2)


def test_dp_full_finetune_gradients_match_on_cpu_ranks():
    """All parameters trainable: the embedding gradient is added in place into the arena and the head's
    segments (first and last slot of the arena) are reduced without touching the layers between them."""
    _run("dp_train_full", 2)


def test_tp_sharded_model_matches_whole_model_on_cpu_ranks():
    """Sharding of heads and MLP columns, row-parallel all-reduce, per-head eviction: two gloo ranks."""
    _run("tp_gpt", 2)


def test_tp_sharded_model_gradients_on_cpu_ranks():
    _run("tp_gpt_grads", 2)


def test_tp_long_context_training_step_on_cpu_ranks():
    _run("tp_train", 2)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_long_context_training_step_on_gpus():
    _run("tp_train", 2)


def test_dp_x_tp_training_step_on_cpu_ranks():
    _run("dp_tp_train", 4)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_dp_x_tp_training_step_on_gpus():
    _run("dp_tp_train", 4)


def test_tp_vocab_parallel_loss_on_cpu_ranks():
    _run("tp_vocab_ce", 3)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_vocab_parallel_loss_and_fused_norm_on_gpus():
    _run("tp_vocab_ce", 2)


def test_tp_lora_gradients_on_cpu_ranks():
    _run("tp_lora_grads", 2)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_lora_gradients_on_gpus():
    _run("tp_lora_grads", 2)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_sharded_model_with_captured_decode_steps_on_gpus():
    _run("tp_gpt", 2)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_sharded_model_gradients_on_gpus():
    _run("tp_gpt_grads", 2)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_allreduce_matches_nccl():
    _run("allreduce", 2)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_dp_gradients_match_on_gpus():
    _run("dp_train", 2)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_dp_full_finetune_gradients_match_on_gpus():
    _run("dp_train_full", 2)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tp_gemm_collectives_match_nccl():
    _run("tp_ops", 2)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tp_gemm_collectives_on_wide_pair_tiles(monkeypatch):
    """The same collectives with the CTA-pair GEMM forced onto its 256 x 512 tiles (all-gather gating and the
    reduce-scatter epilogue of eight epilogue warps)."""
    monkeypatch.setenv("KVB200_GEMM2_TILE", "wide")
    _run("tp_ops", 2)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_model_matches_single_gpu():
    _run("tp_model", 2)


def _all_gpus() -> int:
    n = min(torch.cuda.device_count(), 8)
    return 1 << (n.bit_length() - 1) if n >= 1 else 0  # largest power of two


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 or more GPUs")
@pytest.mark.parametrize("case", ["allreduce", "tp_ops", "dp_train"])
def test_collectives_on_all_gpus(case):
    """The fused collectives and the data-parallel step at the full width of the box."""
    _run(case, _all_gpus(), timeout=600)
