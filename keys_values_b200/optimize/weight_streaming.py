"""Host-resident transformer blocks, streamed to the device one block at a time.

For models whose weights do not fit next to the activation checkpoints of a long-context
step (or do not fit at all), the weights of the transformer blocks live in pinned host
memory, one flat buffer per block, and the device holds a small ring of block-sized slots.
A block is copied into a free slot on a side stream while the previous block computes
(``prefetch``), becomes usable once the copy has landed (``acquire``: the block's
parameters are re-pointed at views of the slot, no module is cloned), and gives the slot
back when its work is done (``release``). In the backward pass the gradients of the
trainable parameters of a row are staged back to pinned host memory on the side stream
and become the ``.grad`` of the host-resident parameters, so that a plain host optimizer
updates the master copy. The embedding, the final norm and the head stay on the device.

Role of the reference's weight offloading: ``clone_model_shard_via_flat_vectors``
(``keys_values/optimize/clone_model.py:33-141``), ``GPTShardCellBlock`` /
``ModelFromFlatVectorsFactory`` (``optimize/model_factory.py:317-491``), the orchestration in
``kvcache/gradient/main.py:1100-1301`` and the per-row all-reduce + device-to-host
accumulation of ``optimize/grad_accumulate.py:196-245``. Differences: parameters are
re-bound instead of cloning modules, copies overlap with compute (two streams, events),
and every block is copied once per (cell, layer) or per row, whichever the pass visits.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch


def _aligned(n: int, unit: int) -> int:
    return (n + unit - 1) // unit * unit


class _BlockLayout:
    """Flat layout of one block's parameters: ``(param, offset, numel)`` with 256-byte aligned offsets."""

    def __init__(self, block: torch.nn.Module):
        self.params: List[Tuple[torch.nn.Parameter, int, int]] = []
        dtypes = {p.dtype for p in block.parameters()}
        if len(dtypes) != 1:
            raise ValueError(f"all parameters of a block must share one dtype to be streamed, got {dtypes}")
        self.dtype = dtypes.pop()
        unit = 256 // torch.empty((), dtype=self.dtype).element_size()
        off = 0
        seen = set()
        for p in block.parameters():
            if id(p) in seen:
                continue
            seen.add(id(p))
            self.params.append((p, off, p.numel()))
            off += _aligned(p.numel(), unit)
        self.numel = max(off, unit)


class WeightStreamer:
    def __init__(self, gpt_model, device, n_slots: int = 2, pin_memory: Optional[bool] = None,
                 reduce_fn: Optional[Callable[[torch.Tensor], None]] = None):
        """``reduce_fn(flat_gradients)`` is called on the device gradients of a block before they leave for
        the host (data parallel: an in-place mean over ranks)."""
        self.gpt_model = gpt_model
        self.device = torch.device(device)
        self.blocks = list(gpt_model.transformer.h)
        self.n_layer = len(self.blocks)
        self.n_slots = max(2, n_slots)
        self.reduce_fn = reduce_fn
        cuda = self.device.type == "cuda"
        pin = cuda if pin_memory is None else pin_memory
        self.layouts = [_BlockLayout(b) for b in self.blocks]
        self.dtype = self.layouts[0].dtype
        # host master copies: the parameters become views of one pinned flat buffer per block
        self.host: List[torch.Tensor] = []
        self.host_grad: List[Optional[torch.Tensor]] = []
        for lay in self.layouts:
            flat = torch.empty(lay.numel, dtype=lay.dtype, pin_memory=pin)
            flat.zero_()
            for p, off, n in lay.params:
                flat[off : off + n].copy_(p.detach().reshape(-1))
                p.data = flat[off : off + n].view(p.shape)
            self.host.append(flat)
            trainable = any(p.requires_grad for p, _, _ in lay.params)
            self.host_grad.append(torch.zeros(lay.numel, dtype=lay.dtype, pin_memory=pin) if trainable else None)
        size = max(lay.numel for lay in self.layouts)
        self.slots = [torch.empty(size, dtype=self.dtype, device=self.device) for _ in range(self.n_slots)]
        self.slot_grads: List[Optional[torch.Tensor]] = [None] * self.n_slots  # allocated on first use by a trainable block
        self.slot_layer: List[Optional[int]] = [None] * self.n_slots   # which block a slot holds (or is receiving)
        self.slot_busy: List[bool] = [False] * self.n_slots            # acquired and not yet released
        self.copy_stream = torch.cuda.Stream(device=self.device) if cuda else None
        self._ready: Dict[int, Optional[torch.cuda.Event]] = {}        # slot -> copy finished
        self._free: Dict[int, Optional[torch.cuda.Event]] = {}         # slot -> last use finished
        self._grad_done: List[Optional[torch.cuda.Event]] = []
        self._next_slot = 0
        self._attached = False  # the host gradients are attached to the parameters as .grad
        self.bytes_to_device = 0
        self.bytes_to_host = 0

    # ------------------------------------------------------------------ slots
    def _slot_of(self, layer: int) -> Optional[int]:
        for s, l in enumerate(self.slot_layer):
            if l == layer:
                return s
        return None

    def _pick_slot(self) -> int:
        for k in range(self.n_slots):
            s = (self._next_slot + k) % self.n_slots
            if not self.slot_busy[s]:
                self._next_slot = (s + 1) % self.n_slots
                return s
        raise RuntimeError("every weight slot is in use: release a block before acquiring another (or raise n_slots)")

    def prefetch(self, layer: int) -> None:
        """Start the copy of block ``layer`` into a free slot (no-op if it is on the device or on its way)."""
        layer %= self.n_layer
        if self._slot_of(layer) is not None:
            return
        s = self._pick_slot()
        self.slot_layer[s] = layer
        n = self.layouts[layer].numel
        if self.copy_stream is None:
            self.slots[s][:n].copy_(self.host[layer])
            self._ready[s] = None
        else:
            with torch.cuda.stream(self.copy_stream):
                free = self._free.get(s)
                if free is not None:
                    self.copy_stream.wait_event(free)  # the previous tenant's kernels have finished with the slot
                self.slots[s][:n].copy_(self.host[layer], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_stream)
                self._ready[s] = ev
        self.bytes_to_device += n * self.host[layer].element_size()

    def acquire(self, layer: int, need_grad: bool = False) -> None:
        """Make block ``layer`` usable on the device: its parameters point into a slot once the copy has
        landed. With ``need_grad`` the trainable parameters get zeroed device gradients to accumulate into."""
        layer %= self.n_layer
        s = self._slot_of(layer)
        if s is None:
            self.prefetch(layer)
            s = self._slot_of(layer)
        if self.slot_busy[s]:
            return
        ev = self._ready.get(s)
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
        self.slot_busy[s] = True
        lay = self.layouts[layer]
        need_grad = need_grad and self.host_grad[layer] is not None
        if need_grad:
            if self.slot_grads[s] is None:
                self.slot_grads[s] = torch.zeros_like(self.slots[s])
            else:
                self.slot_grads[s][: lay.numel].zero_()
        for p, off, n in lay.params:
            p.data = self.slots[s][off : off + n].view(p.shape)
            if p.requires_grad:
                # autograd accumulates in place into the flat device buffer; without need_grad the host gradients
                # (if attached) step aside while the parameter is on the device and come back at release
                p.grad = self.slot_grads[s][off : off + n].view(p.shape) if need_grad else None

    def release(self, layer: int, with_gradients: bool = False) -> None:
        """Give the slot of block ``layer`` back; with ``with_gradients`` the gradients accumulated since
        ``acquire`` are staged to the host first (added to what the host already holds for this step)."""
        layer %= self.n_layer
        s = self._slot_of(layer)
        if s is None or not self.slot_busy[s]:
            return
        lay = self.layouts[layer]
        if with_gradients and self.host_grad[layer] is not None:
            g = self.slot_grads[s][: lay.numel]
            if self.reduce_fn is not None:
                self.reduce_fn(g)
            if self.copy_stream is None:
                self.host_grad[layer].add_(g.to(self.host_grad[layer].device))
            else:
                done = torch.cuda.Event()
                done.record(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(self.copy_stream):
                    self.copy_stream.wait_event(done)
                    from keys_values_b200.utils.host_pool import pinned_empty

                    staged = pinned_empty((lay.numel,), lay.dtype)  # from the pinned pool: no cudaHostAlloc per block
                    staged.copy_(g, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self.copy_stream)
                self._grad_done.append((layer, staged, ev))
            self.bytes_to_host += lay.numel * g.element_size()
        attach = self._attached and not with_gradients and self.host_grad[layer] is not None
        for p, off, n in lay.params:
            p.grad = None
            p.data = self.host[layer][off : off + n].view(p.shape)
            if attach and p.requires_grad:
                p.grad = self.host_grad[layer][off : off + n].view(p.shape)
        self.slot_busy[s] = False
        if self.copy_stream is not None:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._free[s] = ev

    def acquire_many(self, layers: Iterable[int], need_grad: bool = False) -> None:
        layers = list(layers)
        for l in layers:
            self.prefetch(l)
        for l in layers:
            self.acquire(l, need_grad)

    def release_many(self, layers: Iterable[int], with_gradients: bool = False) -> None:
        for l in layers:
            self.release(l, with_gradients)

    # -------------------------------------------------------------- gradients
    def zero_grad(self) -> None:
        for g in self.host_grad:
            if g is not None:
                g.zero_()
        for lay in self.layouts:
            for p, _, _ in lay.params:
                p.grad = None
        self._attached = False

    def collect_gradients(self) -> None:
        """After the backward pass: wait for the staged gradients and attach them as ``.grad`` (host tensors)
        of the host-resident parameters, ready for a host optimizer."""
        for layer, staged, ev in self._grad_done:
            ev.synchronize()
            self.host_grad[layer].add_(staged)
        self._grad_done = []
        for lay, g in zip(self.layouts, self.host_grad):
            if g is None:
                continue
            for p, off, n in lay.params:
                if p.requires_grad:
                    p.grad = g[off : off + n].view(p.shape)
        self._attached = True

    def trainable_parameters(self) -> List[torch.nn.Parameter]:
        return [p for lay in self.layouts for p, _, _ in lay.params if p.requires_grad]

    def resident_bytes(self) -> int:
        """Device memory held by the slots (weights and, once used, gradients)."""
        n = sum(s.numel() * s.element_size() for s in self.slots)
        n += sum(g.numel() * g.element_size() for g in self.slot_grads if g is not None)
        return n
