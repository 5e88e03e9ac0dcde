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


MODEL_TYPES = ("lora", "full")


def load_configuration(task_path: Path, model_type: Optional[str] = None) -> Dict[str, Any]:
    """``hyperparameters.yaml`` written by the fine-tuning run (searched in ``task_path``, then its ``final``
    sub-directory, then its parent). With ``model_type`` the result is checked against it: a ``lora`` run must
    have recorded its LoRA arguments, a ``full`` run must not have any."""
    task_path = Path(task_path)
    hp: Dict[str, Any] = {}
    for d in (task_path, task_path / "final", task_path.parent):
        p = d / "hyperparameters.yaml"
        if p.is_file():
            hp = yaml.safe_load(p.read_text()) or {}
            break
    if model_type is not None:
        if model_type not in MODEL_TYPES:
            raise ValueError(f"model_type = {model_type} not supported; must be in {MODEL_TYPES}")
        has_lora = isinstance(hp.get("lora"), dict)
        if model_type == "lora" and not has_lora:
            raise ValueError(f"{task_path}: model_type is 'lora', but the run recorded no LoRA arguments")
        if model_type == "full" and has_lora:
            raise ValueError(f"{task_path}: model_type is 'full', but the run recorded LoRA arguments")
    return hp


def detect_checkpoints(out_dir: Path) -> List[str]:
    """Names of the sub-directories of ``out_dir`` that hold a complete checkpoint (weights and
    hyper-parameters), ``final`` first, the rest sorted by step number."""
    names = []
    for child in Path(out_dir).iterdir():
        if child.is_dir() and (child / "hyperparameters.yaml").is_file() and any(
                (child / f).is_file() for f in ("lit_model.pth", "lit_model.lora.pth", "head_model.pth")):
            names.append(child.name)

    def order(name):
        digits = "".join(ch for ch in name if ch.isdigit())
        return (name != "final", int(digits) if digits else 0, name)

    return sorted(names, key=order)


def load_setups(setups_filename: Union[str, Path]) -> List[Dict[str, Any]]:
    """The setups file: a YAML list of records ``{out_dir, model_type, [eval_tasks], [checkpoint_dir], [kv_cache],
    [setups]}``. ``eval_tasks`` names the checkpoints (sub-directories of ``out_dir``) to evaluate; without it they
    are detected. ``kv_cache`` overrides fields of the KV-cache arguments the run was trained with, ``setups`` lists
    cache names to evaluate every checkpoint with."""
    records = yaml.safe_load(Path(setups_filename).read_text())
    if isinstance(records, dict):
        records = [records]
    if not isinstance(records, list) or not records:
        raise ValueError(f"{setups_filename} must contain a non-empty list of setups")
    for k, rec in enumerate(records):
        for key in ("out_dir", "model_type"):
            if key not in rec:
                raise ValueError(f"{setups_filename}: setup {k} has no '{key}'")
        if rec["model_type"] not in MODEL_TYPES:
            raise ValueError(f"{setups_filename}: setup {k}: model_type = {rec['model_type']} not in {MODEL_TYPES}")
        if not Path(rec["out_dir"]).is_dir():
            raise ValueError(f"{setups_filename}: setup {k}: out_dir = {rec['out_dir']} is not a directory")
    return records


def setup_from_file(setups_filename: Union[str, Path], data=None, devices: int = 1, seed: int = 1337, batch_size: int = 1,
                    precision: Optional[str] = None, eval_dir: str = "eval", use_sample_metric: Optional[str] = None,
                    sample_metric_max_generated_tokens: int = 64, sample_metric_temperature: float = 0.0,
                    sample_metric_top_k: Optional[int] = None, sample_metric_top_p: float = 1.0,
                    num_store_generated_samples: Optional[int] = None, skip_eval: bool = False, max_iters: Optional[int] = None,
                    attention_forward_temp_size_gb: Optional[float] = None, tp: int = 1) -> None:
    """Evaluate every checkpoint of every setup listed in ``setups_filename`` (see :func:`load_setups`)
    (``keys_values/evaluation/longcontext_eval_ext.py:120-262``).

    ``use_sample_metric``: also generate answers and score them with this metric (sampling controlled by the
    ``sample_metric_*`` arguments); ``num_store_generated_samples``: keep the generated text of at most this many
    samples per task; ``skip_eval``: do not compute losses, only the sample metric (which must then be given)."""
    if skip_eval and use_sample_metric is None:
        raise ValueError("skip_eval needs use_sample_metric: there would be nothing to compute")
    if batch_size < 1 or sample_metric_max_generated_tokens < 1:
        raise ValueError("batch_size and sample_metric_max_generated_tokens must be positive")
    if not 0.0 < sample_metric_top_p <= 1.0 or sample_metric_temperature < 0.0:
        raise ValueError("sample_metric_top_p must be in (0, 1], sample_metric_temperature non-negative")
    from keys_values_b200.parallel.launch import launch

    for rec in load_setups(setups_filename):
        out_dir = Path(rec["out_dir"])
        names = rec.get("eval_tasks") or ([] if rec.get("checkpoint_dir") else detect_checkpoints(out_dir))
        if rec.get("checkpoint_dir"):
            names = list(names) + [str(rec["checkpoint_dir"])]
        if not names:
            raise ValueError(f"{out_dir}: no checkpoints to evaluate")
        first = Path(names[0]) if Path(names[0]).is_absolute() else out_dir / names[0]
        hp = load_configuration(first, rec["model_type"])
        kv_fields = {k: v for k, v in (hp.get("kv_cache") or {}).items() if k in KVCacheArgs.__dataclass_fields__}
        kv_fields.update(rec.get("kv_cache") or {})
        if attention_forward_temp_size_gb is not None:
            kv_fields["attention_forward_temp_size_gb"] = attention_forward_temp_size_gb
        kv_cache = KVCacheArgs(**kv_fields)
        eval_args = EvalArgs(max_new_tokens=sample_metric_max_generated_tokens, max_iters=max_iters, sample_metric=use_sample_metric)
        sample_args = dict(temperature=sample_metric_temperature, top_k=sample_metric_top_k, top_p=sample_metric_top_p)
        launch(main, devices if tp == 1 else tp, tp=tp, out_dir=out_dir, checkpoints=names, data=data, kv_cache=kv_cache, eval=eval_args, precision=precision,
               eval_dir=eval_dir, setups=rec.get("setups") or [kv_cache.name], batch_size=batch_size, hp=hp, model_name=hp.get("model_name"),
               seed=seed, sample_args=sample_args, num_store_generated_samples=num_store_generated_samples, skip_eval=skip_eval)


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
          batch_size: int = 1, model_name: Optional[str] = None, seed: int = 1337, use_sample_metric: Optional[str] = None,
          sample_metric_max_generated_tokens: int = 64, sample_metric_temperature: float = 0.0, sample_metric_top_k: Optional[int] = None,
          sample_metric_top_p: float = 1.0, num_store_generated_samples: Optional[int] = None, skip_eval: bool = False,
          attention_forward_temp_size_gb: Optional[float] = None, tp: int = 1) -> None:
    """``out_dir``: output directory of a fine-tuning run, or a setups file (see :func:`setup_from_file`);
    ``checkpoints``: names of its sub-directories to evaluate (default ``final``). The KV-cache setup defaults to
    the one the run was trained with."""
    from keys_values_b200.parallel.launch import launch

    out_dir = Path(out_dir)
    if out_dir.is_file():
        return setup_from_file(out_dir, data=data, devices=devices, seed=seed, batch_size=batch_size, precision=precision, eval_dir=eval_dir,
                               use_sample_metric=use_sample_metric or eval.sample_metric,
                               sample_metric_max_generated_tokens=sample_metric_max_generated_tokens,
                               sample_metric_temperature=sample_metric_temperature, sample_metric_top_k=sample_metric_top_k,
                               sample_metric_top_p=sample_metric_top_p, num_store_generated_samples=num_store_generated_samples,
                               skip_eval=skip_eval, max_iters=eval.max_iters, attention_forward_temp_size_gb=attention_forward_temp_size_gb, tp=tp)
    hp = load_configuration(out_dir)
    if kv_cache is None:
        kv_cache = KVCacheArgs(**{k: v for k, v in (hp.get("kv_cache") or {}).items() if k in KVCacheArgs.__dataclass_fields__})
    if use_sample_metric is not None:
        eval = EvalArgs(**{**eval.__dict__, "sample_metric": use_sample_metric, "max_new_tokens": sample_metric_max_generated_tokens})
    launch(main, devices if tp == 1 else tp, tp=tp, out_dir=out_dir, checkpoints=checkpoints or ["final"], data=data, kv_cache=kv_cache, eval=eval, precision=precision,
           eval_dir=eval_dir, setups=setups or [kv_cache.name], batch_size=batch_size, hp=hp, model_name=model_name or hp.get("model_name"),
           seed=seed, sample_args=dict(temperature=sample_metric_temperature, top_k=sample_metric_top_k, top_p=sample_metric_top_p),
           num_store_generated_samples=num_store_generated_samples, skip_eval=skip_eval)


def main(rank: int, local_rank: int, world_size: int, *, out_dir, checkpoints, data, kv_cache, eval, precision, eval_dir, setups, batch_size, hp,
         model_name, seed: Optional[int] = None, sample_args: Optional[dict] = None, num_store_generated_samples: Optional[int] = None,
         skip_eval: bool = False, tp: int = 1) -> None:
    """One worker. ``tp == 1``: every launched rank is an independent worker that claims batches through the lock
    files. ``tp > 1``: the launched ranks form ONE worker whose model is sharded over them (heads and MLP columns);
    rank 0 claims the batches and writes the results, the others follow its decisions."""
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
    comm = None
    if tp > 1:
        import torch.distributed as dist

        from keys_values_b200.parallel.tp import TPComm, tp_model_from

        if world_size != tp:
            raise ValueError(f"tp = {tp} needs {tp} launched ranks, got {world_size}")
        comm = TPComm(tp, rank, device, dtype=dtype)
    writer = comm is None or rank == 0
    if seed is not None:
        torch.manual_seed(seed)  # the same on every worker: sampled answers do not depend on who claims a batch
    tasks = EvaluationTasks(setups, [c if Path(c).is_absolute() else str(Path(out_dir) / c) for c in checkpoints])
    stored: Dict[str, int] = {}
    head_name = hp.get("head_model", CrossEntropyOnLogits.NAME)
    transform = BatchTransformFactory.from_head_model(head_name)
    if data is None:
        # the stand-in data of the fine-tuning commands (same generator, same seed: same validation rows)
        from keys_values_b200.config import Config
        from keys_values_b200.data.module import SyntheticLongContext

        cfg_file = base_dir / "model_config.yaml"
        vocab = Config.from_file(cfg_file).vocab_size if cfg_file.is_file() else Config.from_name(model_name).vocab_size
        data = SyntheticLongContext(vocab, seq_lengths=(4 * kv_cache.cache_length,), num_targets=kv_cache.chunk_size)
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
            lock = helper.get_lock(task, b_idx) if writer else None
            if comm is not None:
                decision = [lock is not None]
                dist.broadcast_object_list(decision, src=0)
                if not decision[0]:
                    continue
            elif lock is None:
                continue
            done = False
            try:
                if current != task:
                    if seed is not None:
                        torch.manual_seed(seed)  # whatever a checkpoint leaves to the initialisation is the same for every task and worker
                    config, gpt = create_gpt_model(base_dir, model_name, lora, device if comm is None else "cpu", dtype,
                                                   hp.get("yarn_rope", True))
                    head = HeadModelFactory.create(head_name, config).to(device)
                    load_model_checkpoint(gpt, base_dir, Path(task.checkpoint), head)
                    if comm is not None:
                        if current is not None:
                            model.gpt_model.close()
                        gpt = tp_model_from(gpt, comm, device, dtype, yarn_rope=hp.get("yarn_rope", True))
                    kv = KVCacheArgs(**{**kv_cache.__dict__, "name": task.setup_name})
                    model = wrap_gpt_model(gpt, head, kv, GradientArgs(), batch_size, device, dtype)
                    model.eval()
                    current = task
                t0 = time.perf_counter()
                tb = transform(batch)
                n_rows, n_tok = tb["input_ids"].shape
                if skip_eval:
                    rows = [{"task": task.key, "batch": b_idx, "row": i, "num_tokens": int(n_tok)} for i in range(n_rows)]
                else:
                    with torch.no_grad():
                        loss = model(tb["input_ids"].to(device), tb["targets"].to(device))
                    rows = [{"task": task.key, "batch": b_idx, "row": i, "loss": float(l), "num_tokens": int(n_tok),
                             "time": time.perf_counter() - t0} for i, l in enumerate(loss.float().view(-1))]
                if eval.sample_metric is not None and tokenizer is not None:
                    # generated answers of this batch, scored (keys_values/evaluation/longcontext_eval_ext.py:671-841)
                    from keys_values_b200.evaluation.evaluator import SampleBasedMetricsEvaluator, split_prompts_and_references

                    prompts, refs = split_prompts_and_references(batch, tokenizer, getattr(tokenizer, "pad_id", None) or 0)
                    gpt.reset()
                    gpt.max_seq_length = prompts.shape[1] + (eval.max_new_tokens or 64)
                    res = SampleBasedMetricsEvaluator(gpt, tokenizer, eval.sample_metric, eval.max_new_tokens or 64, kv.chunk_size,
                                                      sample_args=sample_args)(prompts.to(device), refs)
                    for row, sc in zip(rows, res["scores"]):
                        row[eval.sample_metric] = sc
                    keep = len(refs) if num_store_generated_samples is None else max(
                        0, min(len(refs), num_store_generated_samples - stored.get(task.key, 0)))
                    if keep and writer:
                        store_generated_samples(helper.task_dir(task) / GENERATED_SAMPLES_FILENAME.format(b_idx), [r[0] for r in refs][:keep],
                                                res["generated"][:keep], res["scores"][:keep])
                        stored[task.key] = stored.get(task.key, 0) + keep
                if writer:
                    store_eval_metrics(helper.result_path(task, b_idx), rows)
                done = True
            finally:
                if lock is not None:
                    helper.release(lock, done)
    if comm is not None:
        if model is not None:
            model.gpt_model.close()
        comm.close()
