"""Differentiable replay of a KV cache: explicit reversible-cache backward.

During the training forward pass every cache records a replay log (the slots
each chunk was written to). For the backward pass the same sequence of
``write → SDPA`` steps is replayed with autograd. The K/V buffers of a layer are
mutated *in place*; each step saves only what is needed to undo it:

    saved per step:  query, the slots, the rows that were overwritten, out, lse

Backward visits the steps in reverse order. At step ``c`` the buffers are in the
state right after the write of step ``c`` (later steps have been undone), so the
SDPA backward sees the same keys/values as the forward did. Gradients w.r.t. the
buffers accumulate in persistent ``dk_buf/dv_buf``; the gradient of the rows
written at step ``c`` is read from there, those entries are zeroed (the
overwritten older rows received no gradient from steps ``>= c``), and the old
rows are restored. What remains in ``dk_buf/dv_buf`` at the left edge of a cell
is the gradient w.r.t. the K/V checkpoint and is carried into the cell on the
left.

This replaces the reference's saved-tensor hooks, which store deltas of
full-size K/V tensors found by pattern matching
(``keys_values/kvcache/gradient/autograd_hooks.py:305-1337``,
``train_attn_weights_replay.py:55-710``, ``attention/sdpa_op.py:474-978``).

A dummy "token" tensor is threaded through consecutive steps of one layer, so
that autograd cannot reorder them.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from keys_values_b200 import ops
from keys_values_b200.ops import cuda as _cu
from keys_values_b200.kvcache.base import KVCacheReplayLog


class ReplayState:
    """Mutable K/V state of one layer during the backward pass."""

    def __init__(self, batch_size: int, n_query_groups: int, cache_length: int, head_size: int, dtype, device):
        shape = (batch_size, n_query_groups, cache_length, head_size)
        self.k_buf = torch.zeros(shape, dtype=dtype, device=device)
        self.v_buf = torch.zeros(shape, dtype=dtype, device=device)
        self.token_pos = torch.zeros(shape[:3], dtype=torch.int32, device=device)
        self.dk_buf = torch.zeros(shape, dtype=torch.float32, device=device)
        self.dv_buf = torch.zeros(shape, dtype=torch.float32, device=device)
        self.current_length = 0
        self.input_pos = 0
        self.cache_length = cache_length
        self.next_grace_pos: Optional[int] = None  # oldest entry of the grace ring (caches with a grace period)

    def restore(self, snap: Optional[Dict[str, Any]]) -> None:
        """Load the state at the left edge of a cell (``None`` = empty cache)."""
        self.next_grace_pos = None if snap is None else snap.get("next_grace_pos")
        if snap is None:
            self.current_length = 0
            self.input_pos = 0
            return
        L = snap["current_length"]
        self.current_length = L
        self.input_pos = snap["input_pos"]
        self.token_pos[:, :, :L] = snap["token_pos"]
        if "quantized" in snap:
            q = snap["quantized"]
            bits = snap["num_bits"]
            if snap.get("blocks_over_heads"):
                for name, buf in (("k", self.k_buf), ("v", self.v_buf)):
                    qq = q[name + "_q"]
                    if bits == 4:
                        qq = torch.cat(((qq >> 4) & 0xF, qq & 0xF), dim=-1)
                    s, z = q[name + "_s"], q[name + "_z"]
                    buf[:, :, :L] = ((qq.float() - z.float()[:, None, :, None]) * s[:, None, :, None]).to(buf.dtype)
            else:
                ops.dequantize_rows(q["k_q"], q["k_s"], q["k_z"], bits, self.k_buf.dtype, out=self.k_buf[:, :, :L])
                ops.dequantize_rows(q["v_q"], q["v_s"], q["v_z"], bits, self.v_buf.dtype, out=self.v_buf[:, :, :L])
        else:
            self.k_buf[:, :, :L] = snap["k"]
            self.v_buf[:, :, :L] = snap["v"]


class CacheWriteSDPA(torch.autograd.Function):
    """One replay step: write ``key/value`` at ``slots``, attend with ``query``."""

    @staticmethod
    def forward(ctx, query, key, value, token, state: ReplayState, slots, new_length: int, scale: float, sliding_window, softcap, saved=None,
                move=None):
        """``move = (src (B,G,n2), dst (B,G,n2), first_pos, next_grace_pos_after)``: grace ring of a full cache.
        Before the chunk is written, the rows in the ring slots ``src`` (the oldest ring entries, token
        positions from ``first_pos``) are copied to the evicted slots ``dst``; the chunk's last ``n2``
        tokens then take the ring slots (``slots`` already says so). The copy is undone in ``backward``,
        where the gradient collected by a copy returns to the ring slot its row came from."""
        B, G, n, D = key.shape
        old_length = state.current_length
        input_pos = state.input_pos
        moved = None
        if move is not None:
            src, dst, first_pos, ngp_after = move
            src4, dst4 = src.unsqueeze(-1).expand(-1, -1, -1, D), dst.unsqueeze(-1).expand(-1, -1, -1, D)
            moved = (src, dst, state.k_buf.gather(2, dst4), state.v_buf.gather(2, dst4), state.token_pos.gather(2, dst), state.next_grace_pos)
            state.k_buf.scatter_(2, dst4, state.k_buf.gather(2, src4))
            state.v_buf.scatter_(2, dst4, state.v_buf.gather(2, src4))
            pos = torch.arange(first_pos, first_pos + src.shape[2], dtype=torch.int32, device=src.device)
            state.token_pos.scatter_(2, dst, pos.view(1, 1, -1).expand_as(dst).contiguous())
            state.next_grace_pos = ngp_after
        fused = (state.k_buf.is_cuda and state.dk_buf.is_contiguous() and state.token_pos.is_contiguous()
                 and _cu.replay_supported(state.k_buf, key) and state.k_buf.shape[0] == B)
        if fused:
            # save the old content of the slots and write the chunk: one kernel
            idx = slots if slots.dtype == torch.int32 else slots.to(torch.int32)
            old_k, old_v, old_tp = _cu.replay_write(state.k_buf, state.v_buf, state.token_pos, idx, key, value, input_pos)
        else:
            idx = slots.to(torch.int64)
            idx4 = idx.unsqueeze(-1).expand(-1, -1, -1, D)
            old_k = state.k_buf.gather(2, idx4)
            old_v = state.v_buf.gather(2, idx4)
            old_tp = state.token_pos.gather(2, idx)
            ops.cache_write(state.k_buf, state.v_buf, state.token_pos, slots, key, value, input_pos)
        state.current_length = new_length
        state.input_pos = input_pos + n
        L = new_length
        if saved is not None:
            # attention outputs and normalisers were kept by the forward pass
            out = saved[0][:, input_pos : input_pos + n]
            lse = saved[1][:, :, input_pos : input_pos + n]
        else:
            out, _, lse = ops.sdpa_fwd(
                query, state.k_buf[:, :, :L], state.v_buf[:, :, :L], scale, input_pos,
                state.token_pos[:, :, :L], False, sliding_window, softcap,
            )
        ctx.save_for_backward(query, out, lse, idx, old_k, old_v, old_tp)
        ctx.state = state
        ctx.meta = (input_pos, old_length, new_length, scale, sliding_window, softcap, key.dtype)
        ctx.fused = fused
        ctx.moved = moved
        return out, token.clone()

    @staticmethod
    def backward(ctx, grad_out, grad_token):
        query, out, lse, idx, old_k, old_v, old_tp = ctx.saved_tensors
        state: ReplayState = ctx.state
        input_pos, old_length, L, scale, sliding_window, softcap, kv_dtype = ctx.meta
        if state.current_length != L or state.input_pos != input_pos + idx.shape[2]:
            raise RuntimeError("replay steps are being differentiated out of order")
        D = old_k.shape[-1]
        dq, _, _ = ops.sdpa_bwd(
            grad_out.contiguous(), query, state.k_buf[:, :, :L], state.v_buf[:, :, :L], out, lse, scale, input_pos,
            state.token_pos[:, :, :L], sliding_window, softcap, dk_accum=state.dk_buf, dv_accum=state.dv_buf,
        )
        if ctx.fused:
            # gradients of the chunk's rows out of the accumulators, slots cleared and restored: one kernel
            dk_new, dv_new = _cu.replay_undo(state.k_buf, state.v_buf, state.token_pos, state.dk_buf, state.dv_buf, idx,
                                                  old_k, old_v, old_tp)
        else:
            idx4 = idx.unsqueeze(-1).expand(-1, -1, -1, D)
            dk_new = state.dk_buf.gather(2, idx4)
            dv_new = state.dv_buf.gather(2, idx4)
            state.dk_buf.scatter_(2, idx4, 0.0)
            state.dv_buf.scatter_(2, idx4, 0.0)
            # undo the write
            state.k_buf.scatter_(2, idx4, old_k)
            state.v_buf.scatter_(2, idx4, old_v)
            state.token_pos.scatter_(2, idx, old_tp)
        if ctx.moved is not None:
            # undo the copy ring -> evicted slots: what the copies collected belongs to the rows in the ring
            src, dst, old_k2, old_v2, old_tp2, ngp_before = ctx.moved
            src4, dst4 = src.unsqueeze(-1).expand(-1, -1, -1, D), dst.unsqueeze(-1).expand(-1, -1, -1, D)
            for buf in (state.dk_buf, state.dv_buf):
                buf.scatter_add_(2, src4, buf.gather(2, dst4))
                buf.scatter_(2, dst4, 0.0)
            state.k_buf.scatter_(2, dst4, old_k2)
            state.v_buf.scatter_(2, dst4, old_v2)
            state.token_pos.scatter_(2, dst, old_tp2)
            state.next_grace_pos = ngp_before
        state.current_length = old_length
        state.input_pos = input_pos
        return dq.to(query.dtype), dk_new.to(kv_dtype), dv_new.to(kv_dtype), grad_token, None, None, None, None, None, None, None, None


class TrainingReplayCache(torch.nn.Module):
    """Stands in for the KV cache of one layer while a cell is differentiated.
    Follows the slot decisions of ``replay_log``; no scores are computed."""

    def __init__(self, state: ReplayState, replay_log: KVCacheReplayLog, mha, block_idx: int, n_head: int, saved=None):
        super().__init__()
        self.grace_period = int(getattr(replay_log, "grace_period", 0) or 0)
        self.state = state
        self.replay_log = replay_log
        self.mha = mha
        self.block_idx = block_idx
        self.n_head = n_head
        self.n_query_groups = state.k_buf.shape[1]
        self.head_size = state.k_buf.shape[3]
        self.cache_length = state.cache_length
        self._chunk_idx = 0
        self.token: Optional[torch.Tensor] = None
        self.saved = saved  # (attn_out (B,T,H·D), lse (B,H,T)) of the whole sequence, or None

    @property
    def input_pos(self) -> int:
        return self.state.input_pos

    def start_cell(self, first_chunk_idx: int) -> None:
        self._chunk_idx = first_chunk_idx
        self.token = torch.zeros((), dtype=torch.float32, device=self.state.k_buf.device, requires_grad=True)

    def forward(self, query, key, value, token_idx):
        st = self.state
        n = key.shape[2]
        log = self.replay_log
        if log.token_chunks[self._chunk_idx] != n:
            raise ValueError(f"chunk {self._chunk_idx} has {log.token_chunks[self._chunk_idx]} tokens in the replay log, got {n}")
        slots = log.slot_positions[self._chunk_idx]
        g, C = self.grace_period, self.cache_length
        is_prefill = slots is None
        if is_prefill:
            B = key.shape[0]
            st.next_grace_pos = C - g if g > 0 else None
            slots = torch.arange(n, dtype=torch.int32, device=key.device).view(1, 1, n).expand(B, self.n_query_groups, n)
            new_length = n
        else:
            new_length = min(self.cache_length, max(st.current_length, st.current_length + n if st.current_length < self.cache_length else 0))
        self._chunk_idx += 1
        move = None
        if g > 0 and not is_prefill and st.current_length == C:
            # full cache with a grace ring (keys_values/kvcache/attn_weights.py:637-783): the logged slots are
            # those of the evicted entries; the oldest ring entries move there, the newest tokens enter the ring
            if st.next_grace_pos is None:
                raise RuntimeError("the KV checkpoint of this cell does not carry the position of the grace ring")
            prefix, n2 = C - g, min(n, g)
            ring = ((torch.arange(n2, device=key.device) + (st.next_grace_pos - prefix)) % g + prefix)
            ring = ring.view(1, 1, n2).expand(key.shape[0], self.n_query_groups, n2)
            index = slots.to(torch.int64)
            ngp_after = st.next_grace_pos if n > g else (st.next_grace_pos - prefix + n) % g + prefix
            move = (ring.contiguous(), index[:, :, :n2].contiguous(), st.input_pos - g, ngp_after)
            slots = torch.cat((index[:, :, n2:], ring), dim=-1).to(torch.int32)
        out, self.token = CacheWriteSDPA.apply(
            query, key, value, self.token, st, slots, new_length,
            self.mha.pos_encoding.sdpa_scale_factor(), self.mha.sliding_window(self.block_idx),
            self.mha.config.attention_logit_softcapping, self.saved, move,
        )
        return out
