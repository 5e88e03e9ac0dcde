"""Checkpoint I/O, LR schedule, loggers (``keys_values/finetune/utils.py:91-547``).

Checkpoint format (LitGPT compatible): ``lit_model.pth`` = ``torch.save({"model": state_dict})``
(a bare state dict is accepted when loading); LoRA runs write ``lit_model.lora.pth`` with the
LoRA tensors only; heads with weights write ``head_model.pth``. A checkpoint directory also
holds ``model_config.yaml``, tokenizer files, ``hyperparameters.yaml`` and the prompt style.
"""
from __future__ import annotations

import csv
import math
import shutil
import time
from pathlib import Path
from typing import List, Any, Dict, Optional

import torch
import yaml

LIT_MODEL_FNAME = "lit_model.pth"
LORA_WEIGHTS_FNAME = "lit_model.lora.pth"
LORA_WEIGHTS_FNAME_OLD = "lit_model.pth.lora"
HEAD_MODEL_FNAME = "head_model.pth"
CONFIG_FILES = ("config.json", "generation_config.json", "model_config.yaml", "tokenizer.json", "tokenizer.model",
                "tokenizer_config.json", "prompt_style.yaml")


def get_lr_scheduler(optimizer, warmup_steps: int, max_steps: int, min_lr: float = 0.0):
    """Linear warm-up for ``warmup_steps`` then cosine decay to ``min_lr`` at ``max_steps``."""
    base_lrs = [g["lr"] for g in optimizer.param_groups]

    def factor(step: int, base_lr: float) -> float:
        if warmup_steps > 0 and step < warmup_steps:
            return (step + 1) / warmup_steps
        if max_steps <= warmup_steps:
            return 1.0
        progress = min(1.0, (step - warmup_steps) / (max_steps - warmup_steps))
        cos = 0.5 * (1.0 + math.cos(math.pi * progress))
        return (min_lr + (base_lr - min_lr) * cos) / base_lr

    return torch.optim.lr_scheduler.LambdaLR(optimizer, [lambda s, b=b: factor(s, b) for b in base_lrs])


def lora_state_dict(model: torch.nn.Module) -> Dict[str, torch.Tensor]:
    from keys_values_b200.models.lora import lora_filter

    return {k: v for k, v in model.state_dict().items() if lora_filter(k, v)}


def save_model_checkpoint(gpt_model, head_model, out_dir: Path, lora: bool = False, rank: int = 0) -> None:
    """Rank 0 writes ``lit_model.lora.pth`` (LoRA tensors only) or ``lit_model.pth``, and
    ``head_model.pth`` if the head has weights. A tensor-parallel shard (``gpt_model.tp_comm``) makes this a
    collective of its group: the whole model's tensors are put together first, so the file is the same as a
    run on one GPU writes, and every rank must call."""
    whole = None
    if getattr(gpt_model, "tp_comm", None) is not None and gpt_model.tp_comm.world > 1:
        from keys_values_b200.parallel.tp import gather_whole_state_dict

        from keys_values_b200.models.lora import lora_filter

        whole = gather_whole_state_dict(gpt_model, only_trainable=lora)  # LoRA runs move only the adapter tensors
        if whole is not None and lora:
            whole = {k: v for k, v in whole.items() if lora_filter(k, v)}
    if rank != 0:
        return
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    if lora:
        torch.save({"model": whole if whole is not None else lora_state_dict(gpt_model)}, out_dir / LORA_WEIGHTS_FNAME)
    else:
        torch.save({"model": whole if whole is not None else gpt_model.state_dict()}, out_dir / LIT_MODEL_FNAME)
    if head_model is not None and any(True for _ in head_model.parameters()):
        torch.save({"model": head_model.state_dict()}, out_dir / HEAD_MODEL_FNAME)


def _load_sd(path: Path) -> Dict[str, torch.Tensor]:
    sd = torch.load(str(path), map_location="cpu", weights_only=True, mmap=True)
    return sd.get("model", sd) if isinstance(sd, dict) else sd


def load_model_checkpoint(gpt_model, checkpoint_dir: Path, resume_dir: Optional[Path] = None, head_model=None, strict: Optional[bool] = None) -> None:
    """Base weights from ``checkpoint_dir/lit_model.pth`` (strict unless the model has LoRA
    parameters), then LoRA / head weights from ``resume_dir`` (or ``checkpoint_dir``). A full
    fine-tune saves all weights as ``lit_model.pth`` in its step folders: when resuming one,
    that file in ``resume_dir`` replaces the base weights."""
    checkpoint_dir = Path(checkpoint_dir)
    comm = getattr(gpt_model, "tp_comm", None)
    if comm is not None and comm.world > 1:
        # a tensor-parallel shard keeps its slices of every tensor of the (memory-mapped) files of the whole model
        from keys_values_b200.parallel.tp import shard_state_dict

        def load(path):
            return shard_state_dict(_load_sd(path), gpt_model.full_config, comm.world, comm.rank)
    else:
        load = _load_sd
    has_lora = any("lora_" in n for n, _ in gpt_model.named_parameters())
    base = checkpoint_dir / LIT_MODEL_FNAME
    if resume_dir is not None and not has_lora:
        resumed = Path(resume_dir) / LIT_MODEL_FNAME
        if not resumed.is_file():
            raise FileNotFoundError(f"cannot resume a full fine-tune: {resumed} does not exist")
        base = resumed
    if base.is_file() and base.stat().st_size > 0:
        gpt_model.load_state_dict(load(base), strict=(not has_lora) if strict is None else strict)
    for d in ([Path(resume_dir)] if resume_dir is not None else []) + [checkpoint_dir]:
        for fname in (LORA_WEIGHTS_FNAME, LORA_WEIGHTS_FNAME_OLD):
            if has_lora and (d / fname).is_file():
                gpt_model.load_state_dict(load(d / fname), strict=False)
                break
        if head_model is not None and (d / HEAD_MODEL_FNAME).is_file():
            head_model.load_state_dict(_load_sd(d / HEAD_MODEL_FNAME))
        if resume_dir is not None:
            break


def copy_config_files(source_dir: Path, out_dir: Path) -> None:
    out_dir.mkdir(parents=True, exist_ok=True)
    for name in CONFIG_FILES:
        if (Path(source_dir) / name).is_file():
            shutil.copy(Path(source_dir) / name, out_dir / name)


def save_hyperparameters(hparams: Dict[str, Any], out_dir: Path) -> None:
    def clean(o):
        if isinstance(o, dict):
            return {k: clean(v) for k, v in o.items()}
        if isinstance(o, (list, tuple)):
            return [clean(v) for v in o]
        if isinstance(o, (str, int, float, bool)) or o is None:
            return o
        if hasattr(o, "__dataclass_fields__"):
            from dataclasses import asdict

            return clean(asdict(o))
        return str(o)

    Path(out_dir).mkdir(parents=True, exist_ok=True)
    with open(Path(out_dir) / "hyperparameters.yaml", "w") as fp:
        yaml.safe_dump(clean(hparams), fp)


def load_generation_config(checkpoint_dir: Path) -> Dict[str, Any]:
    import json

    p = Path(checkpoint_dir) / "generation_config.json"
    return json.loads(p.read_text()) if p.is_file() else {}


def adapt_requires_grad(model: torch.nn.Module, trainable_prefixes=None) -> None:
    for n, p in model.named_parameters():
        p.requires_grad = trainable_prefixes is None or any(n.startswith(pre) for pre in trainable_prefixes)


class CSVLogger:
    """Minimal metrics logger: one CSV row per ``log_dict`` call (default logger)."""

    def __init__(self, out_dir: Path, name: str = "metrics.csv", flush_every: int = 1):
        self.path = Path(out_dir) / "logs" / name
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.rows, self.keys = [], []

    def log_dict(self, metrics: Dict[str, Any], step: Optional[int] = None) -> None:
        row = dict(metrics, step=step, time=time.time())
        self.rows.append(row)
        new_keys = [k for k in row if k not in self.keys]
        self.keys += new_keys
        with self.path.open("w", newline="") as fp:
            w = csv.DictWriter(fp, fieldnames=self.keys)
            w.writeheader()
            w.writerows(self.rows)


def choose_logger(logger_name: str, out_dir: Path, name: str = "metrics", **kwargs):
    """``csv`` (default), ``tensorboard``, ``wandb`` or ``mlflow`` (the last three need their packages);
    every logger has ``log_dict(metrics, step)`` (``keys_values/finetune/utils.py:265-325``)."""
    if logger_name == "csv":
        return CSVLogger(out_dir, name + ".csv")
    if logger_name == "tensorboard":
        from torch.utils.tensorboard import SummaryWriter

        class _TB:
            def __init__(self):
                self.w = SummaryWriter(str(Path(out_dir) / "logs" / "tensorboard"))

            def log_dict(self, metrics, step=None):
                for k, v in metrics.items():
                    if isinstance(v, (int, float)):
                        self.w.add_scalar(k, v, step)

        return _TB()
    if logger_name == "wandb":
        import wandb  # optional dependency

        class _WandB:
            def __init__(self):
                self.run = wandb.init(project=kwargs.get("project", name), dir=str(out_dir), resume=kwargs.get("resume", "allow"))

            def log_dict(self, metrics, step=None):
                self.run.log({k: v for k, v in metrics.items() if isinstance(v, (int, float))}, step=step)

        return _WandB()
    if logger_name == "mlflow":
        import mlflow  # optional dependency

        class _MLflow:
            def __init__(self):
                mlflow.set_tracking_uri(kwargs.get("tracking_uri", (Path(out_dir) / "logs" / "mlruns").resolve().as_uri()))
                mlflow.set_experiment(kwargs.get("experiment", name))
                self.run = mlflow.start_run()

            def log_dict(self, metrics, step=None):
                mlflow.log_metrics({k: float(v) for k, v in metrics.items() if isinstance(v, (int, float))}, step=step)

        return _MLflow()
    raise ValueError(f"`--logger_name={logger_name}` is not a valid option. Choose from 'csv', 'tensorboard', 'wandb', 'mlflow'.")


class ThroughputMonitor:
    """Running rates over the last ``window`` optimizer steps (role of Lightning's ``ThroughputMonitor`` in
    ``keys_values/finetune/longcontext_full.py:1387``, ``:1663-1669``): ``update`` takes the cumulative
    training time and the cumulative numbers of batches, samples and tokens; ``compute`` returns
    ``throughput/{batches,samples,items}_per_sec`` for the whole job and ``throughput/device/...`` per GPU."""

    def __init__(self, world_size: int = 1, window: int = 20):
        self.world_size, self.window = max(1, world_size), max(2, window)
        self._hist: List[Dict[str, float]] = []

    def update(self, *, time: float, batches: int, samples: int, lengths: int) -> None:
        self._hist.append(dict(time=float(time), batches=float(batches), samples=float(samples), lengths=float(lengths)))
        if len(self._hist) > self.window:
            self._hist.pop(0)

    def compute(self) -> Dict[str, float]:
        if len(self._hist) < 2:
            return {}
        first, last = self._hist[0], self._hist[-1]
        dt = last["time"] - first["time"]
        if dt <= 0:
            return {}
        out = {}
        for key, name in (("batches", "batches"), ("samples", "samples"), ("lengths", "items")):
            rate = (last[key] - first[key]) / dt
            out[f"throughput/device/{name}_per_sec"] = rate
            out[f"throughput/{name}_per_sec"] = rate * self.world_size
        return out


def finetuning_performance_report(train_time: float, total_tokens: int, steps: int, device, out_dir: Optional[Path] = None) -> Dict[str, Any]:
    """Summary printed (and written to ``performance_report.json``) when training ends: time, throughput
    and peak device memory (``keys_values/finetune/longcontext_full.py:909-914``)."""
    report: Dict[str, Any] = {
        "training_time_s": train_time, "optimizer_steps": steps, "tokens": total_tokens,
        "tokens_per_sec": total_tokens / train_time if train_time > 0 else float("nan"),
        "sec_per_step": train_time / steps if steps else float("nan"),
    }
    device = torch.device(device)
    if device.type == "cuda":
        report["peak_memory_gb"] = torch.cuda.max_memory_allocated(device) / 2**30
        report["device"] = torch.cuda.get_device_name(device)
    if out_dir is not None:
        import json

        (Path(out_dir) / "performance_report.json").write_text(json.dumps(report, indent=1))
    return report


def generate_example(gpt_model, tokenizer, prompt_ids: torch.Tensor, max_new_tokens: int, chunk_size: int, device) -> str:
    """Greedy continuation of one validation prompt through the model's caches (printed with every validation,
    ``keys_values/finetune/longcontext_full.py:1918-1962``). Leaves the caches reset and the context width
    as it found them."""
    from keys_values_b200.generate.base import generate

    width = gpt_model.max_seq_length
    was_training = gpt_model.training
    gpt_model.eval()
    try:
        with torch.no_grad():
            prompt = prompt_ids.to(device).view(-1)
            out = generate(gpt_model, prompt, max_returned_tokens=prompt.numel() + max_new_tokens, prompt_chunksize=chunk_size,
                           temperature=0.0, eos_id=getattr(tokenizer, "eos_id", None), include_prompt=False)
        return tokenizer.decode(out) if tokenizer is not None else " ".join(str(int(t)) for t in out)
    finally:
        gpt_model.reset()
        gpt_model.max_seq_length = width
        gpt_model.train(was_training)
