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
        for p in self.params:
            n = p.numel()
            self.offsets[id(p)] = (off, n)
            off += (n + align - 1) // align * align
        self.numel = max(off, align)
        self.symm = None
        if self.use_fused:
            from keys_values_b200.parallel.symm import SymmetricArena

            self.symm = SymmetricArena(self.numel, self.dtype, self.device, world_size, rank, group)
            self.flat = self.symm.tensor
        else:
            self.flat = torch.zeros(self.numel, dtype=self.dtype, device=self.device)
        for p in self.params:
            o, n = self.offsets[id(p)]
            p.grad = self.flat[o : o + n].view_as(p)
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.overlap else None
        self._ranges: Optional[Dict[int, Tuple[int, int]]] = None
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
            for key, (lo, hi) in self._ranges.items():
                if key not in self._covered:
                    self.reduce_range_async(lo, hi)
            self._covered.clear()
        if self.comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)

    # ------------------------------------------------- overlap with backward
    def row_done_hook(self, gpt_model) -> Callable[[int, int], None]:
        """Callback for :class:`LongContextGradientModel`: ``hook(first, end)`` is called
        when the gradients of layers ``[first, end)`` are final (``first == n_layer``
        stands for the head, ``first == -1`` for the embeddings at the very end).
        Parameters outside the GPT model (head-model weights) are reduced by
        :meth:`finish_step`."""
        n_layer = gpt_model.config.n_layer
        ranges: Dict[int, Tuple[int, int]] = {}
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
            lo, hi = ranges.get(layer, (o, o + n))
            ranges[layer] = (min(lo, o), max(hi, o + n))
        rest = [self.offsets[id(p)] for p in self.params if id(p) not in seen]
        if rest:
            ranges[n_layer + 1] = (min(o for o, _ in rest), max(o + n for o, n in rest))
        self._ranges = ranges
        self._covered = set()

        def hook(first: int, end: int) -> None:
            keys = [-1] if first == -1 else list(range(first, end))
            los = [ranges[k][0] for k in keys if k in ranges and k not in self._covered]
            his = [ranges[k][1] for k in keys if k in ranges and k not in self._covered]
            self._covered.update(k for k in keys if k in ranges)
            if los:
                self.reduce_range_async(min(los), max(his))

        return hook


def all_reduce_scalar_mean(x: torch.Tensor, world_size: int, group=None) -> torch.Tensor:
    if world_size > 1:
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
        x = x / world_size
    return x
