"""``eval_long_ext``: evaluate checkpoints of fine-tuning runs on long-context data
(``keys_values/evaluation/longcontext_eval_ext.py:120-1020``).

For every (setup, checkpoint) task and every batch that this worker can claim: load the
checkpoint if the task changed, compute the loss with the chunked forward, optionally
generate answers and score them, and write one CSV per batch. Results are reduced offline
with :mod:`keys_values_b200.tools.collect_eval_results`."""
from __future__ import annotations

import csv
import time
from pathlib import Path
from typing import Any, Dict, List, Optional, Union

import torch
import yaml

from keys_values_b200.evaluation.tasks import EvaluationTasks, EvaluationWithTasksHelper
from keys_values_b200.finetune.args import EvalArgs, KVCacheArgs, LoRAArgs
from keys_values_b200.finetune.batch_transform import BatchTransformFactory
from keys_values_b200.models.head_model import CrossEntropyOnLogits, HeadModelFactory


def load_configuration(out_dir: Path) -> Dict[str, Any]:
    """``hyperparameters.yaml`` written by the fine-tuning run (searched in ``out_dir``, then ``final``)."""
    for d in (Path(out_dir), Path(out_dir) / "final"):
        p = d / "hyperparameters.yaml"
        if p.is_file():
            return yaml.safe_load(p.read_text()) or {}
    return {}


def store_eval_metrics(path: Path, rows: List[Dict[str, Any]]) -> None:
    with open(path, "w", newline="") as fp:
        w = csv.DictWriter(fp, fieldnames=list(rows[0].keys()))
        w.writeheader()
        w.writerows(rows)


GENERATED_SAMPLES_FILENAME = "generated_samples_{}.yaml"


def store_generated_samples(path: Path, references: List[str], generated: List[str], scores: Optional[List[float]] = None) -> None:
    """One YAML document per sample: reference answer, generated text and (if given) its score."""
    with open(path, "w") as fp:
        for i, (r, g) in enumerate(zip(references, generated)):
            doc = {"reference": r, "generated": g}
            if scores is not None:
                doc["score"] = float(scores[i])
            fp.write(yaml.safe_dump(doc) + "---\n")


def setup(out_dir: Union[str, Path], checkpoints: Optional[List[str]] = None, data=None, kv_cache: Optional[KVCacheArgs] = None,
          eval: EvalArgs = EvalArgs(), devices: int = 1, precision: Optional[str] = None, eval_dir: str = "eval", setups: Optional[List[str]] = None,
          batch_size: int = 1, model_name: Optional[str] = None) -> None:
    """``out_dir``: output directory of a fine-tuning run; ``checkpoints``: names of its
    sub-directories to evaluate (default ``final``). The KV-cache setup defaults to the one the
    run was trained with."""
    from keys_values_b200.parallel.launch import launch

    out_dir = Path(out_dir)
    hp = load_configuration(out_dir)
    if kv_cache is None:
        kv_cache = KVCacheArgs(**{k: v for k, v in (hp.get("kv_cache") or {}).items() if k in KVCacheArgs.__dataclass_fields__})
    launch(main, devices, out_dir=out_dir, checkpoints=checkpoints or ["final"], data=data, kv_cache=kv_cache, eval=eval, precision=precision,
           eval_dir=eval_dir, setups=setups or [kv_cache.name], batch_size=batch_size, hp=hp, model_name=model_name or hp.get("model_name"))


def main(rank: int, local_rank: int, world_size: int, *, out_dir, checkpoints, data, kv_cache, eval, precision, eval_dir, setups, batch_size, hp,
         model_name) -> None:
    from keys_values_b200.finetune.longcontext_full import create_gpt_model, wrap_gpt_model
    from keys_values_b200.finetune.args import GradientArgs
    from keys_values_b200.finetune.utils import load_model_checkpoint
    from keys_values_b200.utils import get_default_supported_precision, str_to_torch_dtype

    device = torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
    dtype = str_to_torch_dtype(precision or hp.get("precision") or get_default_supported_precision(False))
    lora_cfg = hp.get("lora")
    lora = LoRAArgs(**lora_cfg) if isinstance(lora_cfg, dict) else None
    base_dir = Path(hp.get("checkpoint_dir", out_dir))
    helper = EvaluationWithTasksHelper(out_dir, eval_dir)
    tasks = EvaluationTasks(setups, [str(Path(out_dir) / c) for c in checkpoints])
    head_name = hp.get("head_model", CrossEntropyOnLogits.NAME)
    transform = BatchTransformFactory.from_head_model(head_name)
    if data is None:
        raise ValueError("eval_long_ext needs a data module (--data …)")
    tokenizer = None
    if (base_dir / "tokenizer.json").is_file() or (base_dir / "tokenizer.model").is_file():
        from keys_values_b200.tokenizer import Tokenizer

        tokenizer = Tokenizer(base_dir)
    data.connect(tokenizer=tokenizer, batch_size=batch_size, num_devices=1, rank=0)
    data.setup()
    loader = data.val_dataloader()
    current, model = None, None
    for task in tasks:
        for b_idx, batch in enumerate(loader):
            if eval.max_iters is not None and b_idx >= eval.max_iters:
                break
            lock = helper.get_lock(task, b_idx)
            if lock is None:
                continue
            done = False
            try:
                if current != task:
                    config, gpt = create_gpt_model(base_dir, model_name, lora, device, dtype, hp.get("yarn_rope", True))
                    head = HeadModelFactory.create(head_name, config).to(device)
                    load_model_checkpoint(gpt, base_dir, Path(task.checkpoint), head)
                    kv = KVCacheArgs(**{**kv_cache.__dict__, "name": task.setup_name})
                    model = wrap_gpt_model(gpt, head, kv, GradientArgs(), batch_size, device, dtype)
                    model.eval()
                    current = task
                t0 = time.perf_counter()
                tb = transform(batch)
                with torch.no_grad():
                    loss = model(tb["input_ids"].to(device), tb["targets"].to(device))
                rows = [{"task": task.key, "batch": b_idx, "row": i, "loss": float(l), "num_tokens": int(tb["input_ids"].shape[1]),
                         "time": time.perf_counter() - t0} for i, l in enumerate(loss.float().view(-1))]
                if eval.sample_metric is not None and tokenizer is not None:
                    # generated answers of this batch, scored (keys_values/evaluation/longcontext_eval_ext.py:671-841)
                    from keys_values_b200.evaluation.evaluator import SampleBasedMetricsEvaluator, split_prompts_and_references

                    prompts, refs = split_prompts_and_references(batch, tokenizer, getattr(tokenizer, "pad_id", None) or 0)
                    gpt.reset()
                    gpt.max_seq_length = prompts.shape[1] + (eval.max_new_tokens or 64)
                    res = SampleBasedMetricsEvaluator(gpt, tokenizer, eval.sample_metric, eval.max_new_tokens or 64, kv.chunk_size)(
                        prompts.to(device), refs)
                    for row, sc in zip(rows, res["scores"]):
                        row[eval.sample_metric] = sc
                    store_generated_samples(helper.task_dir(task) / GENERATED_SAMPLES_FILENAME.format(b_idx), [r[0] for r in refs],
                                            res["generated"], res["scores"])
                store_eval_metrics(helper.result_path(task, b_idx), rows)
                done = True
            finally:
                helper.release(lock, done)
