"""Optimizer state and master weights in pinned host memory.

The reference's ``finetune_offload_*`` commands keep weights, gradients and optimizer state on the
host and copy shards of the model to the GPU for each row of the backward pass
(``keys_values/kvcache/gradient/main.py:1100-1301``, ``optimize/grad_accumulate.py:196-245``,
``optimize/clone_model.py:33-141``), because a 40–80 GB GPU cannot hold all of them. With 180 GB of
HBM3e the bf16 weights and their bf16 gradients (4 bytes per parameter) stay on the device, where
every row of the backward pass needs them anyway; what moves to the host is what only the optimizer
touches: fp32 master weights, fp32 gradients and the optimizer moments (16 bytes per parameter for
AdamW). Per step: gradients device → host (pinned staging, side stream), optimizer step on the
host, updated weights host → device. A 14B-parameter full fine-tune then needs 56 GB on the device
instead of 224 GB.

:class:`HostOffloadOptimizer` has the surface the training loop uses of a ``torch.optim.Optimizer``
(``param_groups, zero_grad, step, state_dict, load_state_dict``) plus ``clip_grad_norm_``.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Sequence

import torch


class HostOffloadOptimizer:
    def __init__(self, params: Sequence[torch.nn.Parameter], create: Callable[[List[torch.nn.Parameter]], torch.optim.Optimizer],
                 master_dtype: torch.dtype = torch.float32, pin_memory: Optional[bool] = None):
        self.device_params = [p for p in params if p.requires_grad]
        if not self.device_params:
            raise ValueError("no trainable parameters")
        dev = self.device_params[0].device
        self.on_gpu = dev.type == "cuda"
        pin = self.on_gpu if pin_memory is None else pin_memory
        self.host_params: List[torch.nn.Parameter] = []
        self._staging: List[torch.Tensor] = []
        for p in self.device_params:
            master = torch.empty(p.shape, dtype=master_dtype, pin_memory=pin)
            master.copy_(p.detach())
            hp = torch.nn.Parameter(master, requires_grad=True)
            hp.grad = torch.zeros(p.shape, dtype=master_dtype, pin_memory=pin)
            self.host_params.append(hp)
            self._staging.append(torch.empty(p.shape, dtype=p.dtype, pin_memory=pin))
        self.optimizer = create(self.host_params)
        self.stream = torch.cuda.Stream(device=dev) if self.on_gpu else None
        self._grads_on_host = False

    # ------------------------------------------------------------ optimizer surface
    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.device_params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()
        self._grads_on_host = False

    def state_dict(self) -> Dict[str, Any]:
        return self.optimizer.state_dict()

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        self.optimizer.load_state_dict(state)

    # -------------------------------------------------------------------- transfers
    def fetch_gradients(self) -> None:
        """Device gradients → fp32 host gradients (a parameter without gradient gets zeros)."""
        if self._grads_on_host:
            return
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream(self.device_params[0].device))
            with torch.cuda.stream(self.stream):
                for p, st in zip(self.device_params, self._staging):
                    if p.grad is not None:
                        st.copy_(p.grad, non_blocking=True)
            self.stream.synchronize()
        for p, hp, st in zip(self.device_params, self.host_params, self._staging):
            if p.grad is None:
                hp.grad.zero_()
            elif self.stream is not None:
                hp.grad.copy_(st)
            else:
                hp.grad.copy_(p.grad)
        self._grads_on_host = True

    def push_weights(self) -> None:
        """Master weights → device parameters (cast to the device dtype)."""
        if self.stream is not None:
            with torch.cuda.stream(self.stream):
                for p, hp, st in zip(self.device_params, self.host_params, self._staging):
                    st.copy_(hp.detach())  # cast on the host into the pinned staging buffer
                    p.data.copy_(st, non_blocking=True)
            torch.cuda.current_stream(self.device_params[0].device).wait_stream(self.stream)
        else:
            for p, hp in zip(self.device_params, self.host_params):
                p.data.copy_(hp.detach())

    # ------------------------------------------------------------------------- step
    def clip_grad_norm_(self, max_norm: float) -> torch.Tensor:
        self.fetch_gradients()
        return torch.nn.utils.clip_grad_norm_(self.host_params, max_norm)

    def step(self) -> None:
        self.fetch_gradients()
        self.optimizer.step()
        self.push_weights()
        self._grads_on_host = False

    def host_bytes(self) -> int:
        state = sum(t.numel() * t.element_size() for s in self.optimizer.state.values() for t in s.values() if torch.is_tensor(t))
        own = sum(hp.numel() * hp.element_size() * 2 for hp in self.host_params) + sum(s.numel() * s.element_size() for s in self._staging)
        return own + state
