"""Chunked long-context inference through bounded KV caches.

A sequence is processed as ``[prefill chunk of C tokens, chunk, chunk, …]``. The
loop nest is *cells → layers → chunks*: a cell is a run of consecutive chunks,
and each layer processes all chunks of the cell before the next layer starts, so
that only one layer's full-precision K/V scratch is live and quantized buffers are
re-materialised once per (cell, layer). Parity:
``keys_values/long_context.py:45-1062``.

Within a (cell, layer) step the block is applied to all tokens of the cell at
once (norms, QKV/MLP GEMMs, RoPE), and only the cache update + attention runs
chunk by chunk; this keeps the GEMMs large enough for the tensor cores.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch

from keys_values_b200.models.head_model import HeadModel
from keys_values_b200.models.model import GPT

NUM_RANDOM_CHUNK_SIZE_VALUES = 5
CLOSEBY_THRESHOLD = 4
MAX_LOGITS_BYTES = 2**31


def create_chunk_sizes(gpt_model: GPT, seq_length: int, chunk_size: int, randomize_chunk_sizes: bool = False) -> List[int]:
    """Chunk sizes compatible with the caches of ``gpt_model``: the first chunk is
    the smallest ``max_prefill_length``; no cache length falls inside a chunk.
    With ``randomize_chunk_sizes`` later chunks draw from 5 values sampled in
    ``[cs − cs//2, cs + cs//2]``."""
    caches = gpt_model.get_kv_caches()
    mpl = min(c.max_prefill_length for c in caches)
    points = sorted({c.cache_length for c in caches if c.cache_length <= seq_length})
    if not points:
        return [seq_length] if mpl >= seq_length else [mpl, seq_length - mpl]
    chunk_sizes = [mpl]
    done = mpl
    step = chunk_size // 2
    lo, hi = max(chunk_size - step, 1), min(chunk_size + step, points[0])
    random_sizes = torch.randint(lo, hi + 1, (NUM_RANDOM_CHUNK_SIZE_VALUES,)) if randomize_chunk_sizes else None
    while done < seq_length:
        if randomize_chunk_sizes:
            c = int(random_sizes[int(torch.randint(0, NUM_RANDOM_CHUNK_SIZE_VALUES, (1,)))])
        else:
            c = chunk_size
        c = min(c, seq_length - done)
        if points and done + c >= points[0] - CLOSEBY_THRESHOLD:
            c = points.pop(0) - done
        if c > 0:
            chunk_sizes.append(c)
        done += c
    assert sum(chunk_sizes) == seq_length
    return chunk_sizes


@dataclass(frozen=True)
class ChunksForCell:
    """Chunks ``[first_chunk_idx, first_chunk_idx + len(chunk_sizes))`` form a cell
    that covers tokens ``[start, end)``."""

    first_chunk_idx: int
    chunk_sizes: Tuple[int, ...]
    start: int

    @property
    def end(self) -> int:
        return self.start + sum(self.chunk_sizes)

    @property
    def num_tokens(self) -> int:
        return sum(self.chunk_sizes)


def get_chunks_for_cells(chunk_sizes: List[int], max_cell_length: int) -> List[ChunksForCell]:
    """Greedy packing of consecutive chunks into cells of at most
    ``max_cell_length`` tokens; a larger single chunk forms its own cell."""
    cells, cur, cur_start, first_idx, pos = [], [], 0, 0, 0
    for i, c in enumerate(chunk_sizes):
        if cur and sum(cur) + c > max_cell_length:
            cells.append(ChunksForCell(first_idx, tuple(cur), cur_start))
            cur, cur_start, first_idx = [], pos, i
        cur.append(c)
        pos += c
    if cur:
        cells.append(ChunksForCell(first_idx, tuple(cur), cur_start))
    return cells


def default_cell_length(config, cache_length: int, chunks_per_cell_multiplier: float = 1.0) -> int:
    """Cell length for which the K/V checkpoints of a cell boundary are about as
    large as the layer-input activations of a cell (``long_context.py:756-767``)."""
    return int(2 * config.n_query_groups * config.head_size / config.n_embd * cache_length * chunks_per_cell_multiplier)


def get_chunk_of_targets(targets: Optional[torch.Tensor], start: int, end: int, num_input_tokens: int) -> Optional[torch.Tensor]:
    """Targets are right-aligned with the inputs: the chunk ``[start, end)`` sees
    ``targets[:, max(start−s, 0) : end−s]`` with ``s = num_input_tokens − targets.shape[1]``."""
    if targets is None:
        return None
    s = num_input_tokens - targets.shape[1]
    if end <= s:
        return None
    return targets[:, max(start - s, 0) : end - s]


def compute_loss_for_chunk(
    gpt_model: GPT,
    head_model: HeadModel,
    model_outputs: torch.Tensor,
    targets: Optional[torch.Tensor],
    input_pos: int,
) -> torch.Tensor:
    """Loss part (per batch row, un-normalised) for the final-layer outputs of one
    chunk. ``ln_f`` and ``lm_head`` are applied here, so checkpoints hold pre-norm
    activations; logits are materialised in pieces of at most 2 GiB."""
    if not head_model.needs_logits():
        return head_model(gpt_model.transformer.ln_f(model_outputs), targets, input_pos)
    if targets is None:
        return torch.zeros(model_outputs.shape[0], device=model_outputs.device, dtype=torch.float32)
    n_t = targets.shape[1]
    x = model_outputs[:, -n_t:, :]
    B = x.shape[0]
    vocab = gpt_model.config.padded_vocab_size
    comm = getattr(gpt_model, "tp_comm", None)
    if (comm is not None and comm.world > 1 and getattr(gpt_model, "vocab_parallel_loss", True) and type(head_model).__name__ == "CrossEntropyOnLogits"
            and isinstance(gpt_model.lm_head, torch.nn.Linear) and gpt_model.lm_head.bias is None
            and gpt_model.config.final_logit_softcapping is None):
        # tensor-parallel shard: every rank forms the logits of its slice of the vocabulary only
        from keys_values_b200.parallel.tp import vocab_parallel_cross_entropy

        bytes_per_pos = B * (vocab // comm.world + 1) * 4
        piece = max(1, MAX_LOGITS_BYTES // bytes_per_pos)
        total = None
        for s in range(0, n_t, piece):
            e = min(s + piece, n_t)
            h = gpt_model.transformer.ln_f(x[:, s:e, :])
            rows = vocab_parallel_cross_entropy(h.reshape(-1, h.shape[-1]), gpt_model.lm_head.weight, targets[:, s:e], comm)
            part = rows.view(B, e - s).sum(dim=-1)
            total = part if total is None else total + part
        return total
    bytes_per_pos = B * vocab * 4
    piece = max(1, MAX_LOGITS_BYTES // bytes_per_pos)
    total = None
    for s in range(0, n_t, piece):
        e = min(s + piece, n_t)
        logits = gpt_model.head(x[:, s:e, :])
        part = head_model(logits, targets[:, s:e], input_pos + model_outputs.shape[1] - n_t + s)
        total = part if total is None else total + part
    return total


class GPTAndHeadModel(torch.nn.Module):
    def __init__(self, gpt_model: GPT, head_model: HeadModel):
        super().__init__()
        self.gpt_model = gpt_model
        self.head_model = head_model

    @property
    def config(self):
        return self.gpt_model.config


LayerInputHook = Callable[[torch.Tensor, int, int, int], None]  # (x, layer_idx, start, end)
CellBoundaryHook = Callable[[int, int, int], None]  # (layer_idx, cell_idx, end)


class LongContextInferenceModel(GPTAndHeadModel):
    """Evaluates loss values (or last-position logits) for long sequences, in
    inference mode."""

    def __init__(
        self,
        gpt_model: GPT,
        head_model: HeadModel,
        chunk_size: int,
        randomize_chunk_sizes: bool = False,
        chunks_per_cell_multiplier: float = 1.0,
        single_tokens_for_targets: bool = False,
        verbose=None,
        tmp_array_limit_gb=None,
        debug_single_cell_per_row: bool = False,
        **_ignored,
    ):
        super().__init__(gpt_model, head_model)
        if chunk_size <= 0:
            raise ValueError("chunk_size must be positive")
        self.chunk_size = chunk_size
        self.randomize_chunk_sizes = randomize_chunk_sizes
        self.chunks_per_cell_multiplier = chunks_per_cell_multiplier
        self.single_tokens_for_targets = single_tokens_for_targets
        self.debug_single_cell_per_row = debug_single_cell_per_row
        self.chunk_sizes: Optional[List[int]] = None
        self.cells: Optional[List[ChunksForCell]] = None
        # Context width for the position encoding; None = length of the batch being processed
        # (generation sets it to prompt + new tokens before the prefill)
        self.fixed_max_seq_length: Optional[int] = None
        self.layer_input_hook: Optional[LayerInputHook] = None
        self.cell_boundary_hook: Optional[CellBoundaryHook] = None
        # keys_values_b200.optimize.weight_streaming.WeightStreamer when the blocks' weights live on the host
        self.weight_streamer = None

    # ------------------------------------------------------------ scheduling
    def _init_members_from_tokens(self, input_ids: torch.Tensor, targets: Optional[torch.Tensor]) -> None:
        gpt = self.gpt_model
        if input_ids.ndim != 2:
            raise ValueError("input_ids must be 2D (batch_size, seq_length)")
        caches = gpt.get_kv_caches()
        if any(c is None for c in caches):
            raise ValueError("KV caches must be assigned to gpt_model (see KVCacheFactory.create)")
        seq_length = input_ids.shape[1]
        if targets is not None and (targets.ndim != 2 or targets.shape[0] != input_ids.shape[0] or targets.shape[1] > seq_length):
            raise ValueError(f"targets.shape = {tuple(targets.shape)} not compatible with input_ids.shape = {tuple(input_ids.shape)}")
        # The position encoding (and for YaRN the SDPA scale) follows the batch length
        gpt.max_seq_length = seq_length if self.fixed_max_seq_length is None else max(seq_length, self.fixed_max_seq_length)
        n_single = 0
        if self.single_tokens_for_targets and targets is not None:
            n_single = min(targets.shape[1], seq_length - 1)
        sizes = create_chunk_sizes(gpt, seq_length - n_single, self.chunk_size, self.randomize_chunk_sizes)
        sizes += [1] * n_single
        self.chunk_sizes = sizes
        max_c = max(c.cache_length for c in caches)
        if self.debug_single_cell_per_row:
            cell_len = seq_length
            self.cells = [ChunksForCell(0, tuple(sizes[:1]), 0)]
            if len(sizes) > 1:
                self.cells.append(ChunksForCell(1, tuple(sizes[1:]), sizes[0]))
        else:
            # a tensor-parallel shard keeps the cell schedule of the whole model (its layer inputs are not sharded)
            cell_len = max(default_cell_length(getattr(gpt, "full_config", gpt.config), max_c, self.chunks_per_cell_multiplier), 1)
            self.cells = get_chunks_for_cells(sizes, cell_len)

    # --------------------------------------------------------------- forward
    def forward(self, input_ids: torch.Tensor, targets: Optional[torch.Tensor] = None, scale_factor: float = 1.0):
        """With ``targets``: loss per batch row ``(B,)`` (normalised by the number of
        target entries). Without: logits of the final position ``(B, 1, vocab)``. The result
        stays on the device; callers that read it on the host follow the read with
        :func:`keys_values_b200.ops.check_status` (see :meth:`loss_value`)."""
        self._init_members_from_tokens(input_ids, targets)
        with torch.no_grad():
            return self._forward_internal(input_ids, targets, scale_factor)

    def loss_value(self, input_ids: torch.Tensor, targets: torch.Tensor, scale_factor: float = 1.0) -> torch.Tensor:
        """:meth:`forward` followed by a host read of the loss and of the device status word: raises if a
        kernel of the pass reported that it gave up on a wait. Returns the per-row loss on the host."""
        from keys_values_b200 import ops as _ops

        loss = self.forward(input_ids, targets, scale_factor).detach().float().cpu()
        _ops.check_status(input_ids.device)
        return loss

    def _forward_internal(self, input_ids, targets, scale_factor: float = 1.0):
        def _dense(t):  # blocks of a tensor-parallel shard may hand on token rows sharded over the ranks
            return t.full() if hasattr(t, "full") else t

        gpt, head = self.gpt_model, self.head_model
        n_layer = gpt.config.n_layer
        seq_length = input_ids.shape[1]
        gpt.reset()
        loss_sum = None
        last_x = None
        for cell_idx, cell in enumerate(self.cells):
            ids = input_ids[:, cell.start : cell.end]
            x = gpt.embed(ids)
            for layer_idx, block in enumerate(gpt.transformer.h):
                if self.layer_input_hook is not None:
                    x = _dense(x)
                    self.layer_input_hook(x, layer_idx, cell.start, cell.end)
                ws = self.weight_streamer
                if ws is not None:  # host-resident blocks: this one on the device, the next one on its way
                    ws.acquire(layer_idx)
                    ws.prefetch(layer_idx + 1)
                x = block(x, ids, gpt.mha, chunk_sizes=cell.chunk_sizes)
                if ws is not None:
                    ws.release(layer_idx)
                if self.cell_boundary_hook is not None:
                    self.cell_boundary_hook(layer_idx, cell_idx, cell.end)
            if self.layer_input_hook is not None:
                x = _dense(x)
                self.layer_input_hook(x, n_layer, cell.start, cell.end)
            if targets is not None:
                x = _dense(x)
                pos = cell.start
                for c in cell.chunk_sizes:
                    t_chunk = get_chunk_of_targets(targets, pos, pos + c, seq_length)
                    if t_chunk is not None or not head.needs_logits():
                        part = compute_loss_for_chunk(gpt, head, x[:, pos - cell.start : pos - cell.start + c], t_chunk, pos)
                        if torch.is_tensor(part):
                            loss_sum = part if loss_sum is None else loss_sum + part
                    pos += c
            last_x = x
        if targets is None:
            return gpt.head(last_x[:, -1:, :])
        num = head.num_target_entries(targets)
        loss = loss_sum.float()
        if num is not None:
            loss = loss / num.clamp(min=1).to(loss.dtype)
        return loss * scale_factor
