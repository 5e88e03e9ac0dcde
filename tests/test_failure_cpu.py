"""Failure detection and recovery, exercised on the host only (no GPU fault is ever provoked)."""
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

WORKER = str(Path(__file__).resolve().parent / "health_worker.py")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("case,expect", [("exit", "heartbeat at step 0, expected 1"), ("raise", "injected host failure")])
def test_surviving_ranks_detect_a_lost_rank_between_steps(case, expect):
    def attempt():
        world, port = 3, _free_port()
        procs = [subprocess.Popen([sys.executable, WORKER, case, str(r), str(world), str(port)], stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True) for r in range(world)]
        outs = [p.communicate(timeout=180)[0] for p in procs]
        ok = all("DETECTED [1]" in outs[r] and expect in outs[r] for r in (0, 2)) and "DETECTED" not in outs[1]
        return ok, outs

    # three processes and wall-clock grace times: on a heavily loaded host one more attempt is allowed
    ok, outs = attempt()
    if not ok:
        ok, outs = attempt()
    assert ok, "\n---\n".join(outs)


def test_oom_retry_ladder_lowers_the_limits_and_retries():
    from keys_values_b200.utils.recovery import OOMRetry

    calls = []

    def step(limit_gb, save_attention):
        calls.append((limit_gb, save_attention))
        if sum(isinstance(c, tuple) for c in calls) < 3:
            raise torch.OutOfMemoryError("injected")
        return "done"

    retry = OOMRetry(limits_gb=(8.0, 4.0, 2.0), free_fn=lambda: calls.append("freed"))
    assert retry.run(step) == "done"
    # first attempt with everything on, then attention outputs off, then the next smaller limit
    assert calls == [(8.0, True), "freed", (8.0, False), "freed", (4.0, False)]
    with pytest.raises(torch.OutOfMemoryError):
        OOMRetry(limits_gb=(1.0,), free_fn=lambda: None).run(lambda a, b: (_ for _ in ()).throw(torch.OutOfMemoryError("x")))


def test_training_step_recovers_from_an_injected_oom():
    """The first attempt of a step runs out of memory (raised on the host by a hook); the engine
    frees the step state, gives up the saved attention outputs and the retry succeeds."""
    from keys_values_b200.finetune.engine import build_lora_training_setup, training_step

    dev = torch.device("cpu")
    setup = build_lora_training_setup("tiny-gpt", dev, torch.float32, cache_name="h2o-torch-quantized8", cache_length=64,
                                      chunk_size=16, lora_r=4, lora_alpha=8, micro_batch_size=1, yarn_rope=False, seed=3)
    ids = torch.randint(0, setup.config.vocab_size, (1, 160))
    tg = torch.randint(0, setup.config.vocab_size, (1, 32))
    ref_loss = float(training_step(setup, ids, tg))
    state = {"n": 0}
    orig_forward = setup.model.forward

    def flaky_forward(*a, **kw):
        state["n"] += 1
        if state["n"] == 1:
            raise torch.OutOfMemoryError("injected on the host")
        return orig_forward(*a, **kw)

    setup.model.forward = flaky_forward
    loss = float(training_step(setup, ids, tg))
    assert state["n"] == 2 and setup.model.save_attention_outputs is False
    assert loss == loss and abs(loss - ref_loss) < 1.0  # finite, same ballpark after one optimizer step
