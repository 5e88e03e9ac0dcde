"""Data-parallel gradient reduction.

Every rank runs the full long-context forward/backward on its own sequences;
gradients of the trainable parameters are then averaged over ranks. Role of
``keys_values/optimize/grad_accumulate.py:88-280`` (flatten per dtype →
``all_reduce(mean)`` → copy back, after the whole backward).

Here the gradients *live* in one flat arena (every ``p.grad`` is a view into it),
so nothing is flattened or copied back, and the arena is ordered by layer: as
soon as the backward pass has finished a row of layers, the slice of that row is
reduced on a separate stream while the rows below are still being computed.
With ``use_fused=True`` the arena is symmetric memory (mapped into every rank
over NVLink) and the reduction is one kernel that reads the peers' slices
directly, sums them in rank order in fp32, applies the ``1/world`` scale and the
cast, and writes the result in place (see ``csrc/comm.cu``). NCCL remains
available (``use_fused=False``) as the comparison path.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


OVERLAP_COMM_CTAS = 32


class GradientReducer:
    def __init__(self, params: Sequence[torch.nn.Parameter], world_size: int, rank: int, device, overlap: bool = True,
                 use_fused: Optional[bool] = None, group=None):
        self.params = [p for p in params if p.requires_grad]
        self.world_size, self.rank = world_size, rank
        self.device = torch.device(device)
        self.group = group
        self.overlap = overlap and self.device.type == "cuda"
        dtypes = {p.dtype for p in self.params}
        if len(dtypes) != 1:
            raise ValueError(f"all trainable parameters must share one dtype, got {dtypes}")
        self.dtype = dtypes.pop()
        if use_fused is None:
            use_fused = self.device.type == "cuda" and world_size > 1
        self.use_fused = use_fused
        # 16-byte aligned slots, in parameter order
        self.offsets: Dict[int, Tuple[int, int]] = {}
        off = 0
        align = 16 // torch.empty((), dtype=self.dtype).element_size()
        self._align = align
        for p in self.params:
            n = p.numel()
            self.offsets[id(p)] = (off, n)
            off += (n + align - 1) // align * align
        self.numel = max(off, align)
        self.symm = None
        if self.use_fused:
            from keys_values_b200.parallel.symm import SymmetricArena

            # Under overlap the all-reduce runs next to the backward kernels (one CTA per SM each): its grid
            # barrier needs all of its CTAs resident at once, so the grid stays far below the SM count.
            self.symm = SymmetricArena(self.numel, self.dtype, self.device, world_size, rank, group,
                                       n_ctas=OVERLAP_COMM_CTAS if self.overlap else 0)
            self.flat = self.symm.tensor
        else:
            self.flat = torch.zeros(self.numel, dtype=self.dtype, device=self.device)
        for p in self.params:
            o, n = self.offsets[id(p)]
            p.grad = self.flat[o : o + n].view_as(p)
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.overlap else None
        self._ranges: Optional[Dict[int, List[Tuple[int, int]]]] = None
        self._covered = set()
        self.num_reductions = 0

    # ------------------------------------------------------------------ API
    def begin_step(self) -> None:
        """Re-attach the arena views (an optimizer may have replaced ``.grad``)."""
        for p in self.params:
            o, n = self.offsets[id(p)]
            view = self.flat[o : o + n].view_as(p)
            if p.grad is None or p.grad.data_ptr() != view.data_ptr():
                if p.grad is not None:
                    view.copy_(p.grad)
                p.grad = view
        self._covered.clear()

    def _reduce_range(self, start: int, end: int) -> None:
        if end <= start:
            return
        self.num_reductions += 1
        if self.use_fused:
            self.symm.all_reduce_mean_(start, end)
        else:
            buf = self.flat[start:end]
            dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=self.group)
            buf.mul_(1.0 / self.world_size)

    def reduce_range_async(self, start: int, end: int) -> None:
        """Reduce ``flat[start:end]``; with overlap on, on the communication stream
        after everything issued so far on the current stream."""
        if self.comm_stream is None:
            self._reduce_range(start, end)
            return
        self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.comm_stream):
            self._reduce_range(start, end)

    def finish_step(self) -> None:
        """Reduce whatever has not been reduced by the row hook and join the
        communication stream."""
        if self._ranges is None:
            self.reduce_range_async(0, self.numel)
        else:
            pending = [seg for key, segs in self._ranges.items() if key not in self._covered for seg in segs]
            for lo, hi in _merge_segments(pending):
                self.reduce_range_async(lo, hi)
            self._covered.clear()
        if self.comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)

    def check(self) -> None:
        """Synchronising check that no kernel of the step gave up on a wait (a lost peer, a flag that never
        came): the gradients are then not reduced and must not reach the optimizer. Raises
        :class:`keys_values_b200.parallel.health.RankFailure` after putting the arena's flags back in order."""
        if self.device.type != "cuda":
            return
        from keys_values_b200.ops import cuda as _cu

        try:
            _cu.check_status(self.device)
        except _cu.NativeError as ex:
            if self.symm is not None:
                self.symm.reset_sync()
            from keys_values_b200.parallel.health import RankFailure

            raise RankFailure({self.rank: f"gradient all-reduce did not complete: {ex}"}) from ex

    # ------------------------------------------------- overlap with backward
    def row_done_hook(self, gpt_model) -> Callable[[int, int], None]:
        """Callback for :class:`LongContextGradientModel`: ``hook(first, end)`` is called
        when the gradients of layers ``[first, end)`` are final (``first == n_layer``
        stands for the head, ``first == -1`` for the embeddings at the very end).
        Parameters outside the GPT model (head-model weights) are reduced by
        :meth:`finish_step`.

        Each key owns a list of disjoint arena segments, never their hull: parameters that
        become final at the same time need not be neighbours in the arena (``lm_head`` comes
        first and ``ln_f`` last in ``parameters()`` order, with every layer between them), and
        a reduction must not touch slots whose gradients are still being accumulated."""
        n_layer = gpt_model.config.n_layer
        ranges: Dict[int, List[Tuple[int, int]]] = {}
        seen = set()
        for name, p in gpt_model.named_parameters():
            if id(p) not in self.offsets:
                continue
            seen.add(id(p))
            layer = n_layer
            if name.startswith("transformer.h."):
                layer = int(name.split(".")[2])
            elif name.startswith("transformer.wte"):
                layer = -1
            o, n = self.offsets[id(p)]
            ranges.setdefault(layer, []).append((o, self._slot_end(o, n)))
        rest = [self.offsets[id(p)] for p in self.params if id(p) not in seen]
        if rest:
            ranges[n_layer + 1] = [(o, self._slot_end(o, n)) for o, n in rest]
        self._ranges = {k: _merge_segments(v) for k, v in ranges.items()}
        self._covered = set()

        def hook(first: int, end: int) -> None:
            keys = [-1] if first == -1 else list(range(first, end))
            keys = [k for k in keys if k in self._ranges and k not in self._covered]
            self._covered.update(keys)
            for lo, hi in _merge_segments([seg for k in keys for seg in self._ranges[k]]):
                self.reduce_range_async(lo, hi)

        return hook

    def _slot_end(self, offset: int, numel: int) -> int:
        """End of a parameter's slot including its alignment padding (which holds zeros), so that
        neighbouring slots merge into one reduction."""
        return min(self.numel, offset + (numel + self._align - 1) // self._align * self._align)


def _merge_segments(segments: Sequence[Tuple[int, int]]) -> List[Tuple[int, int]]:
    """Sorted union of half-open segments; touching or overlapping ones become one."""
    out: List[Tuple[int, int]] = []
    for lo, hi in sorted(segments):
        if out and lo <= out[-1][1]:
            out[-1] = (out[-1][0], max(out[-1][1], hi))
        else:
            out.append((lo, hi))
    return out


def all_reduce_scalar_mean(x: torch.Tensor, world_size: int, group=None) -> torch.Tensor:
    if world_size > 1:
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
        x = x / world_size
    return x
