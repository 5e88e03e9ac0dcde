"""Gradients for long-context models through the KV-cache policy.

Training step = forward pass in inference mode (loss value, layer-input
checkpoints, K/V checkpoints at cell boundaries, replay logs), then a top-down
backward over *rows* of ``layers_per_cell`` layers, each row processed cell by
cell from right to left with autograd inside the cell. Parity:
``keys_values/kvcache/gradient/main.py:67-1348`` and ``accumulate.py:101-942``.

Differences that follow from the 180 GB of device memory: all checkpoints stay
on the device by default (``offload_checkpoints=True`` moves them to pinned host
memory through a side stream), and the K/V checkpoints of *all* layers are
taken during the single inference forward, so the reference's extra per-row
replay pass that recomputes them is not needed. One training step therefore
evaluates every (layer, chunk) twice forward and once backward, not three
times forward.
"""
from __future__ import annotations

import time
from typing import Any, Callable, Dict, List, Optional

import torch

from keys_values_b200.kvcache.gradient.checkpoints import KVCheckpoints, LayerInputCheckpoints
from keys_values_b200.kvcache.gradient.replay import ReplayState, TrainingReplayCache
from keys_values_b200.long_context import (
    ChunksForCell,
    LongContextInferenceModel,
    compute_loss_for_chunk,
    get_chunk_of_targets,
)
from keys_values_b200.models.head_model import HeadModel
from keys_values_b200.models.model import GPT


class LossValue:
    """Loss returned by :class:`LongContextGradientModel` in training mode: behaves
    like a scalar tensor, and ``backward()`` starts the cell-wise backward pass
    (``gradient/main.py:67-121``)."""

    def __init__(self, value: torch.Tensor, model: "LongContextGradientModel"):
        self._value = value
        self._model = model

    def backward(self) -> None:
        self._model.backward()

    def item(self) -> float:
        return self._value.item()

    def detach(self) -> torch.Tensor:
        return self._value.detach()

    @property
    def value(self) -> torch.Tensor:
        return self._value

    def __float__(self) -> float:
        return float(self._value)

    def __repr__(self) -> str:
        return f"LossValue({self._value})"


from keys_values_b200.tools.profiling import nvtx_mark  # noqa: E402

class LongContextGradientModel(LongContextInferenceModel):
    def __init__(
        self,
        gpt_model: GPT,
        head_model: HeadModel,
        layers_per_cell: int,
        chunk_size: int,
        randomize_chunk_sizes: bool = False,
        chunks_per_cell_multiplier: float = 1.0,
        single_tokens_for_targets: bool = False,
        offload_checkpoints: bool = False,
        pin_memory: bool = True,
        layercp_qname: Optional[str] = None,
        cachecp_qname: Optional[str] = None,
        profile_steps: bool = False,
        row_done_hook: Optional[Callable[[int, int], None]] = None,
        average_loss_per_batch: bool = False,
        save_attention_outputs: Optional[bool] = None,
        profile_parts: Optional[str] = None,
        profile_exit: bool = False,
        **kwargs,
    ):
        super().__init__(
            gpt_model, head_model, chunk_size, randomize_chunk_sizes, chunks_per_cell_multiplier,
            single_tokens_for_targets, **kwargs,
        )
        if layers_per_cell <= 0:
            raise ValueError("layers_per_cell must be positive")
        self.layers_per_cell = layers_per_cell
        self.offload_checkpoints = offload_checkpoints
        self.pin_memory = pin_memory
        self.layercp_qname = layercp_qname
        self.cachecp_qname = cachecp_qname
        self.row_done_hook = row_done_hook
        self.average_loss_per_batch = average_loss_per_batch
        self.profile_steps = profile_steps
        from keys_values_b200.tools.profiling import PartProfiler

        self.part_profiler = PartProfiler(profile_parts, exit_after=profile_exit)  # cProfile of "forward" / "backward" / "both"
        # Keep the attention outputs and normalisers of the forward pass (B·T·H·D values per
        # layer) so that the backward pass only recomputes the linear parts. None = decide
        # from the free device memory.
        self.save_attention_outputs = save_attention_outputs
        self._attn_saved = None
        self.profile_records: List[Dict[str, Any]] = []
        self._status = "init"
        self._layer_ckpt: Optional[LayerInputCheckpoints] = None
        self._kv_ckpt: Optional[KVCheckpoints] = None
        self._replay_logs = None
        self._inputs = None

    # -------------------------------------------------------------- forward
    def _row_boundaries(self) -> List[int]:
        n_layer = self.gpt_model.config.n_layer
        return list(range(0, n_layer, self.layers_per_cell)) + [n_layer]

    def forward(self, input_ids: torch.Tensor, targets: Optional[torch.Tensor] = None, scale_factor: float = 1.0):
        if not self.training or targets is None:
            return super().forward(input_ids, targets, scale_factor)
        t0 = time.perf_counter()
        self.part_profiler.start("forward")
        self._init_members_from_tokens(input_ids, targets)
        gpt = self.gpt_model
        B, T = input_ids.shape
        dev = input_ids.device
        dtype = gpt.transformer.wte.weight.dtype
        bounds = self._row_boundaries()
        self._layer_ckpt = LayerInputCheckpoints(
            layer_indices=bounds, batch_size=B, seq_length=T, n_embd=gpt.config.n_embd, dtype=dtype, device=dev,
            offload=self.offload_checkpoints, pin_memory=self.pin_memory, qname=self.layercp_qname,
        )
        self._kv_ckpt = KVCheckpoints(offload=self.offload_checkpoints, pin_memory=self.pin_memory)
        caches = gpt.get_kv_caches()
        n_cells = len(self.cells)

        def layer_hook(x, layer_idx, start, end):
            if layer_idx == 0:
                nvtx_mark(f"forward: cell {start}:{end}")
            if layer_idx in self._layer_ckpt.slots:
                self._layer_ckpt.write(layer_idx, start, end, x)

        def boundary_hook(layer_idx, cell_idx, end):
            if cell_idx < n_cells - 1:
                self._kv_ckpt.put(layer_idx, cell_idx + 1, caches[layer_idx].kv_snapshot())

        self._attn_saved = None
        if self._decide_save_attention(B, T, dev, dtype):
            cfg = gpt.config
            self._attn_saved = [
                (torch.empty((B, T, cfg.n_head * cfg.head_size), dtype=dtype, device=dev),
                 torch.empty((B, cfg.n_head, T), dtype=torch.float32, device=dev))
                for _ in range(cfg.n_layer)
            ]

            def recorder(block_idx, pos, attn_out, lse):
                o, l = self._attn_saved[block_idx]
                n = attn_out.shape[1]
                o[:, pos : pos + n] = attn_out
                l[:, :, pos : pos + n] = lse

        for c in caches:
            c.switch_replay_logging(True)
            c.attn_recorder = recorder if self._attn_saved is not None else None
        self.layer_input_hook, self.cell_boundary_hook = layer_hook, boundary_hook
        try:
            with torch.no_grad():
                loss_rows = self._forward_internal(input_ids, targets, scale_factor)
        finally:
            self.layer_input_hook = self.cell_boundary_hook = None
            for c in caches:
                c.attn_recorder = None
        self._replay_logs = [c.get_replay_log() for c in caches]
        for c in caches:
            c.switch_replay_logging(False)
        self._inputs = (input_ids, targets, scale_factor)
        self._status = "forward_done"
        if self.profile_steps:
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)
            self.profile_records.append(dict(forward_time=time.perf_counter() - t0))
        self.part_profiler.stop("forward", dev)
        return LossValue(loss_rows.mean(), self)

    def _decide_save_attention(self, B: int, T: int, dev, dtype) -> bool:
        if self.save_attention_outputs is not None:
            return self.save_attention_outputs
        if dev.type != "cuda":
            return False
        cfg = self.gpt_model.config
        need = cfg.n_layer * B * T * (cfg.n_head * cfg.head_size * torch.empty((), dtype=dtype).element_size() + cfg.n_head * 4)
        free, _ = torch.cuda.mem_get_info(dev)
        free += torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)
        # leave room for the other checkpoints and the per-cell activations
        other = (len(self._row_boundaries()) + 1) * B * T * cfg.n_embd * 2 + 24 * 2**30
        return need + other < free

    # ------------------------------------------------------------- backward
    def backward(self) -> None:
        if self._status != "forward_done":
            raise RuntimeError("forward (in training mode) must be called before backward")
        t0 = time.perf_counter()
        self.part_profiler.start("backward")
        input_ids, targets, scale_factor = self._inputs
        gpt, head = self.gpt_model, self.head_model
        B, T = input_ids.shape
        dev = input_ids.device
        n_layer = gpt.config.n_layer
        ckpt = self._layer_ckpt
        # 1) Head: dL/d(final hidden states), written into the gradient buffer
        head_grad = torch.zeros((B, T, gpt.config.n_embd), dtype=ckpt.dtype, device=dev)
        num = head.num_target_entries(targets)
        for cell in self.cells:
            need = not head.needs_logits() or get_chunk_of_targets(targets, cell.start, cell.end, T) is not None
            if not need:
                continue
            x = ckpt.read(n_layer, cell.start, cell.end).detach().requires_grad_(True)
            with torch.enable_grad():
                total = None
                pos = cell.start
                for c in cell.chunk_sizes:
                    t_chunk = get_chunk_of_targets(targets, pos, pos + c, T)
                    if t_chunk is not None or not head.needs_logits():
                        part = compute_loss_for_chunk(gpt, head, x[:, pos - cell.start : pos - cell.start + c], t_chunk, pos)
                        if torch.is_tensor(part):
                            total = part if total is None else total + part
                    pos += c
                if total is None or not total.requires_grad:
                    continue
                total = total.float()
                if num is not None:
                    total = total / num.clamp(min=1).to(total.dtype)
                (total.mean() * scale_factor).backward()
            head_grad[:, cell.start : cell.end] = x.grad
        if self.row_done_hook is not None:
            self.row_done_hook(n_layer, n_layer + 1)
        # 2) Rows of layers, top down; cells right to left
        bounds = self._row_boundaries()
        caches = gpt.get_kv_caches()
        blocks = gpt.transformer.h
        ws = self.weight_streamer
        for r in range(len(bounds) - 2, -1, -1):
            first, end = bounds[r], bounds[r + 1]
            nvtx_mark(f"backward: layers {first}:{end}")
            if ws is not None:
                # host-resident blocks: this row's blocks on the device with gradient buffers, the next row's on their way
                ws.acquire_many(range(first, end), need_grad=True)
                if r > 0:
                    for l in range(bounds[r - 1], bounds[r]):
                        ws.prefetch(l)
            states, tcaches = [], []
            for l in range(first, end):
                c = caches[l]
                st = ReplayState(B, c.n_query_groups, c.cache_length, c.head_size, ckpt.dtype, dev)
                states.append(st)
                saved = self._attn_saved[l] if self._attn_saved is not None else None
                tcaches.append(TrainingReplayCache(st, self._replay_logs[l], c.mha, l, c.n_head, saved=saved))
            try:
                for l, tc in zip(range(first, end), tcaches):
                    blocks[l].attn.kv_cache = tc
                for cell_idx in range(len(self.cells) - 1, -1, -1):
                    cell = self.cells[cell_idx]
                    ids = input_ids[:, cell.start : cell.end]
                    for l, st, tc in zip(range(first, end), states, tcaches):
                        st.restore(self._kv_ckpt.get(l, cell_idx) if cell_idx > 0 else None)
                        tc.start_cell(cell.first_chunk_idx)
                    x = ckpt.read(first, cell.start, cell.end).detach().requires_grad_(True)
                    with torch.enable_grad():
                        y = x
                        for l in range(first, end):
                            y = blocks[l](y, ids, gpt.mha, chunk_sizes=cell.chunk_sizes)
                        tokens = [tc.token for tc in tcaches]
                        torch.autograd.backward(
                            [y] + tokens, [head_grad[:, cell.start : cell.end]] + [torch.zeros_like(t) for t in tokens]
                        )
                    head_grad[:, cell.start : cell.end] = x.grad
                    del x, y
            finally:
                for l in range(first, end):
                    blocks[l].attn.kv_cache = caches[l]
            del states, tcaches
            if self._attn_saved is not None:
                for l in range(first, end):
                    self._attn_saved[l] = None  # release as soon as the row is done
            if ws is not None:
                ws.release_many(range(first, end), with_gradients=True)
            if self.row_done_hook is not None:
                self.row_done_hook(first, end)
        if ws is not None:
            ws.collect_gradients()
        # 3) Input embeddings
        wte = gpt.transformer.wte.weight
        if wte.requires_grad:
            g = head_grad
            if gpt.config.scale_embeddings:
                g = g * (gpt.config.n_embd**0.5)
            grad = torch.zeros_like(wte, dtype=torch.float32)
            grad.index_add_(0, input_ids.reshape(-1), g.reshape(-1, g.shape[-1]).float())
            if wte.grad is None:
                wte.grad = grad.to(wte.dtype)
            else:
                # in place: ``.grad`` may be a view into a flat gradient arena that is reduced over ranks
                wte.grad.add_(grad.to(wte.dtype))
        if self.row_done_hook is not None:
            self.row_done_hook(-1, 0)
        self.clear()
        if self.profile_steps:
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)
            self.profile_records[-1]["backward_time"] = time.perf_counter() - t0
            if dev.type == "cuda":
                self.profile_records[-1]["peak_memory_gb"] = torch.cuda.max_memory_allocated(dev) / 2**30
        self.part_profiler.stop("backward", dev)

    def clear(self) -> None:
        self._attn_saved = None
        self._layer_ckpt = None
        self._kv_ckpt = None
        self._replay_logs = None
        self._inputs = None
        self._status = "init"


class NaiveGPTAndHeadModel(torch.nn.Module):
    """Whole-sequence forward with plain autograd; the baseline that the chunked
    gradient is checked against on short sequences (``gradient/main.py:1331-1348``)."""

    def __init__(self, gpt_model: GPT, head_model: HeadModel):
        super().__init__()
        self.gpt_model = gpt_model
        self.head_model = head_model

    def forward(self, input_ids: torch.Tensor, targets: torch.Tensor, scale_factor: float = 1.0) -> torch.Tensor:
        caches = self.gpt_model.get_kv_caches()
        self.gpt_model.clear_kv_caches()
        try:
            self.gpt_model.max_seq_length = input_ids.shape[1]
            x = self.gpt_model(input_ids, skip_lm_head=True)
            loss = compute_loss_for_chunk(self.gpt_model, self.head_model, x, targets, 0).float()
            num = self.head_model.num_target_entries(targets)
            if num is not None:
                loss = loss / num.clamp(min=1).to(loss.dtype)
            return loss.mean() * scale_factor
        finally:
            if all(c is not None for c in caches):
                self.gpt_model.assign_kv_caches(caches)
