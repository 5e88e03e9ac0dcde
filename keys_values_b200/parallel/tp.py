"""Tensor parallelism over KV heads with fused GEMM + collective kernels.

Layout (per transformer block, ``tp`` ranks on one NVSwitch node):

* ``qkv`` and the MLP up projections are column parallel: rank ``r`` holds the
  query heads / KV heads / MLP columns of its shard; the attention projection and
  the MLP down projection are row parallel.
* Between blocks the activations are sharded over *tokens* (sequence parallel).
  A block therefore is: all-gather→QKV GEMM, local cache update + attention for
  the rank's KV heads (cache policy state is per KV head, so eviction needs no
  communication), attn-out GEMM→reduce-scatter (+ residual), all-gather→MLP-up
  GEMM, MLP-down GEMM→reduce-scatter (+ residual).

Both collectives are fused into the tcgen05 GEMM kernel of ``csrc/gemm_sm100.cu``:
the reduce-scatter is the GEMM's epilogue (finished tiles are stored straight
into the owner rank's receive buffer over NVLink, remote owners first), and the
all-gather feeds the GEMM's TMA producer chunk by chunk from a local staging
buffer that copy CTAs of the same kernel fill from the peers. NCCL is used only
to exchange the IPC handles and in the reference path of the tests.

The reference library has no tensor parallelism (``README.md:273-275``); this
module is additive API.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from keys_values_b200.ops import cuda as _cu
from keys_values_b200.parallel.symm import _RawCudaBuffer


class _SymmBuffer:
    """A ``cudaMalloc`` allocation mapped into every rank (CUDA IPC)."""

    def __init__(self, nbytes: int, device, world: int, rank: int, group=None):
        lib = _cu.lib()
        self.nbytes = (nbytes + 255) // 256 * 256
        ptr = ctypes.c_void_p()
        _cu._check(lib.kvb_symm_alloc(ctypes.byref(ptr), ctypes.c_longlong(self.nbytes)), "symm_alloc")
        self.ptr = ptr.value
        self._raw = _RawCudaBuffer(self.ptr, self.nbytes)
        self.bytes = torch.as_tensor(self._raw, device=device)
        hsize = lib.kvb_ipc_handle_size()
        hbuf = (ctypes.c_ubyte * hsize)()
        _cu._check(lib.kvb_ipc_get_handle(ctypes.c_void_p(self.ptr), hbuf), "ipc_get_handle")
        handles: List[Optional[bytes]] = [None] * world
        dist.all_gather_object(handles, bytes(hbuf), group=group)
        self.peer_ptrs: List[int] = []
        self._opened: List[int] = []
        for r, h in enumerate(handles):
            if r == rank:
                self.peer_ptrs.append(self.ptr)
            else:
                out = ctypes.c_void_p()
                _cu._check(lib.kvb_ipc_open_handle((ctypes.c_ubyte * hsize).from_buffer_copy(h), ctypes.byref(out)), "ipc_open_handle")
                self.peer_ptrs.append(out.value)
                self._opened.append(out.value)

    def ptr_array(self, offset: int = 0):
        return (ctypes.c_void_p * len(self.peer_ptrs))(*[p + offset for p in self.peer_ptrs])

    def close(self):
        lib = _cu.lib()
        for p in self._opened:
            lib.kvb_ipc_close_handle(ctypes.c_void_p(p))
        self._opened = []
        if self.ptr:
            self.bytes = None
            lib.kvb_symm_free(ctypes.c_void_p(self.ptr))
            self.ptr = 0


class TPContext:
    """Symmetric buffers and flag words for the fused tensor-parallel GEMMs.

    ``max_rows``: largest number of token rows of a call (all ranks together), a
    multiple of ``128 · world``; ``max_features``: largest feature dimension that is
    gathered (K of all-gather→GEMM) or scattered (N of GEMM→reduce-scatter).
    """

    FLAG_WORDS = 256

    def __init__(self, world: int, rank: int, device, max_rows: int, max_features: int, group=None, timeout_s: float = 20.0,
                 copy_ctas: Optional[int] = None):
        if max_rows % (128 * world):
            raise ValueError(f"max_rows must be a multiple of {128 * world}")
        self.world, self.rank, self.group = world, rank, group
        self.device = torch.device(device)
        # CTAs that pull the peers' shards: the remote fraction (world − 1) / world of the activation must
        # arrive while the local fraction is being multiplied, so more ranks need more copy CTAs
        if copy_ctas is None:
            copy_ctas = min(16, 2 + 2 * world)  # each keeps 192 KB in flight through the TMA engine
        self.timeout_s, self.copy_ctas = timeout_s, copy_ctas
        self.max_rows, self.max_features = max_rows, max_features
        torch.cuda.set_device(self.device)
        esz = 2
        # all-gather staging (also the buffer the producer of the shard writes into)
        self.stage = _SymmBuffer(max_rows * max_features * esz, self.device, world, rank, group)
        # reduce-scatter receive buffers, two of them (consecutive calls alternate)
        self.recv = [_SymmBuffer(max_rows * max_features * esz, self.device, world, rank, group) for _ in range(2)]
        # flag words: [0:16) rs counters parity 0, [16:32) rs counters parity 1, [32] ag ready, [33] ag pulled
        self.flags = _SymmBuffer(self.FLAG_WORDS * 4, self.device, world, rank, group)
        self.chunk_flags = torch.zeros(16, dtype=torch.int32, device=self.device)
        self._rs_calls = [0, 0]
        self._rs_tiles = [0, 0]
        self._ag_calls = 0
        self._ag_pulled = 0
        dist.barrier(group=group)

    # ------------------------------------------------------------ all-gather → GEMM
    def stage_view(self, rows_per_rank: int, features: int) -> torch.Tensor:
        """Slot of this rank in the staging buffer, ``(rows_per_rank, features)`` bf16: the
        producer of the token-sharded activation writes its output here."""
        full = self.stage.bytes[: self.world * rows_per_rank * features * 2].view(torch.bfloat16).view(self.world * rows_per_rank, features)
        return full[self.rank * rows_per_rank : (self.rank + 1) * rows_per_rank]

    def allgather_gemm(self, rows_per_rank: int, weight: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``cat_r(shard_r) @ weight^T``: the shards are the ``stage_view`` slots of all ranks.
        ``weight (N, K)`` bf16. Returns ``(world·rows_per_rank, N)``."""
        N, K = weight.shape
        M = self.world * rows_per_rank
        if rows_per_rank % 128 or M > self.max_rows or K > self.max_features:
            raise ValueError("allgather_gemm: rows per rank must be a multiple of 128 within the context limits")
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        self._ag_calls += 1
        self._ag_pulled += (self.world - 1) * self.copy_ctas
        st = _cu.status_word(self.device)
        _cu._check(
            _cu.lib().kvb_allgather_gemm(
                ctypes.c_void_p(self.stage.ptr), self.stage.ptr_array(), _cu._p(weight), _cu._p(out), _cu._p(self.chunk_flags),
                self.flags.ptr_array(32 * 4), self.flags.ptr_array(33 * 4), self.rank, self.world, rows_per_rank, N, K,
                ctypes.c_longlong(K), ctypes.c_longlong(weight.stride(0)), ctypes.c_longlong(out.stride(0)),
                ctypes.c_uint(self._ag_calls), ctypes.c_uint(self._ag_calls * self.copy_ctas), ctypes.c_uint(self._ag_pulled),
                self.copy_ctas, _cu._p(st), ctypes.c_double(self.timeout_s), _cu._stream(weight),
            ),
            "allgather_gemm",
        )
        _cu._count()
        return out

    # ----------------------------------------------------------- GEMM → reduce-scatter
    def gemm_reduce_scatter(self, x: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor] = None,
                            out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``reduce_scatter_rows(x @ weight^T) (+ residual)``: ``x (M, K_shard)``, ``weight (N, K_shard)``
        are this rank's shards along K. Returns this rank's ``(M/world, N)`` rows."""
        M, K = x.shape
        N = weight.shape[0]
        rows = M // self.world
        if M % self.world or rows % 128 or M > self.max_rows or N > self.max_features:
            raise ValueError("gemm_reduce_scatter: M/world must be a multiple of 128 within the context limits")
        par = (self._rs_calls[0] + self._rs_calls[1]) & 1
        self._rs_calls[par] += 1
        tiles_per_dest = (rows // 128) * ((N + 255) // 256)  # the kernel works on 128 x 256 tiles
        self._rs_tiles[par] += 4 * tiles_per_dest
        if out is None:
            out = torch.empty((rows, N), dtype=torch.bfloat16, device=self.device)
        st = _cu.status_word(self.device)
        _cu._check(
            _cu.lib().kvb_gemm_reduce_scatter(
                _cu._p(x), _cu._p(weight), _cu._p(out), _cu._p(residual), self.recv[par].ptr_array(),
                self.flags.ptr_array(par * 16 * 4), self.rank, self.world, M, N, K, ctypes.c_longlong(x.stride(0)),
                ctypes.c_longlong(weight.stride(0)), ctypes.c_uint(self._rs_tiles[par]), _cu._p(st),
                ctypes.c_double(self.timeout_s), _cu._stream(x),
            ),
            "gemm_reduce_scatter",
        )
        _cu._count(2)
        return out

    def close(self):
        for b in (self.stage, self.flags, *self.recv):
            b.close()


def shard_rows(t: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    n = t.shape[0] // world
    return t[rank * n : (rank + 1) * n]


class TPBlockWeights:
    """Weights of one transformer block sharded over KV heads for rank ``rank``.

    ``qkv (H+2G)·D x E`` → rows of the rank's query heads, key heads and value heads;
    ``proj E x H·D`` → columns of the rank's query heads; ``fc_1/fc_2`` → row shards,
    ``mlp.proj`` → column shards. Norm weights are replicated.
    """

    def __init__(self, block, config, world: int, rank: int):
        H, G, D = config.n_head, config.n_query_groups, config.head_size
        if G % world:
            raise ValueError(f"n_query_groups = {G} must be divisible by the tensor-parallel size {world}")
        gs = H // G
        g0, g1 = rank * (G // world), (rank + 1) * (G // world)
        w = block.attn.qkv.weight if not hasattr(block.attn.qkv, "linear") else block.attn.qkv.linear.weight
        q_rows = w[g0 * gs * D : g1 * gs * D]
        k_rows = w[H * D + g0 * D : H * D + g1 * D]
        v_rows = w[(H + G) * D + g0 * D : (H + G) * D + g1 * D]
        self.qkv = torch.cat((q_rows, k_rows, v_rows)).contiguous()
        pw = block.attn.proj.weight if not hasattr(block.attn.proj, "linear") else block.attn.proj.linear.weight
        self.proj = pw[:, g0 * gs * D : g1 * gs * D].contiguous()
        inter = config.intermediate_size
        i0, i1 = rank * (inter // world), (rank + 1) * (inter // world)

        def _w(m):
            return m.weight if not hasattr(m, "linear") else m.linear.weight

        self.fc = torch.cat((_w(block.mlp.fc_1)[i0:i1], _w(block.mlp.fc_2)[i0:i1])).contiguous()
        self.mlp_proj = _w(block.mlp.proj)[:, i0:i1].contiguous()
        self.norm_1 = block.norm_1.weight
        self.norm_2 = block.norm_2.weight
        self.norm_q = block.attn.norm_q.weight if block.attn.norm_q is not None else None
        self.norm_k = block.attn.norm_k.weight if block.attn.norm_k is not None else None
        self.n_head_local = (g1 - g0) * gs
        self.n_groups_local = g1 - g0
        self.inter_local = i1 - i0


class TPModel:
    """Tensor-parallel inference wrapper around a (LLaMA-style) ``GPT``.

    Every rank keeps the full embedding and head (vocab-parallel heads are not needed
    for generation of one token at a time), the blocks are sharded as in
    :class:`TPBlockWeights`, and each rank owns the KV caches of its KV heads, created
    by ``make_cache(block_idx, n_query_groups_local, n_head_local)``.
    """

    def __init__(self, gpt, ctx: TPContext, make_cache):
        cfg = gpt.config
        if cfg.mlp_class_name != "LLaMAMLP" or cfg.parallel_residual or cfg.norm_class_name != "RMSNorm":
            raise NotImplementedError("tensor parallelism supports LLaMA-style blocks (RMSNorm, SwiGLU, sequential residual)")
        self.gpt, self.ctx, self.config = gpt, ctx, cfg
        self.blocks = [TPBlockWeights(b, cfg, ctx.world, ctx.rank) for b in gpt.transformer.h]
        self.caches = [make_cache(i, self.blocks[i].n_groups_local, self.blocks[i].n_head_local) for i in range(cfg.n_layer)]

    def reset(self):
        for c in self.caches:
            c.reset()

    @torch.no_grad()
    def forward_hidden(self, x_shard: torch.Tensor, token_idx: torch.Tensor, chunk_sizes=None) -> torch.Tensor:
        """``x_shard (rows_per_rank, E)``: this rank's token rows of the embedded chunk (batch
        and time flattened, B = 1). Returns the rank's rows of the final hidden states."""
        from keys_values_b200 import ops

        cfg, ctx = self.config, self.ctx
        D = cfg.head_size
        rows = x_shard.shape[0]
        T = rows * ctx.world
        mha = self.gpt.mha
        for li, (w, cache) in enumerate(zip(self.blocks, self.caches)):
            # all-gather → QKV GEMM
            ctx.stage_view(rows, cfg.n_embd).copy_(ops.rmsnorm(x_shard, w.norm_1, cfg.norm_eps))
            qkv = ctx.allgather_gemm(rows, w.qkv).view(1, T, -1)
            input_pos = cache.input_pos
            cos, sin = mha.pos_encoding.tables(input_pos, T, li, qkv.device) if cfg.rope_n_elem > 0 else (None, None)
            q, k, v = ops.qknorm_rope(qkv, w.n_head_local, w.n_groups_local, D, cos, sin, w.norm_q, w.norm_k, cfg.norm_eps, cfg.rope_n_elem)
            y = cache(query=q, key=k, value=v, token_idx=token_idx)  # (1, T, H_local·D)
            # attention projection GEMM → reduce-scatter (+ residual)
            x_shard = ctx.gemm_reduce_scatter(y.view(T, -1), w.proj, residual=x_shard)
            # all-gather → MLP-up GEMM, SwiGLU, MLP-down GEMM → reduce-scatter (+ residual)
            ctx.stage_view(rows, cfg.n_embd).copy_(ops.rmsnorm(x_shard, w.norm_2, cfg.norm_eps))
            h = ctx.allgather_gemm(rows, w.fc)
            a = ops.swiglu(h[:, : w.inter_local].contiguous(), h[:, w.inter_local :].contiguous())
            x_shard = ctx.gemm_reduce_scatter(a, w.mlp_proj, residual=x_shard)
        return x_shard
