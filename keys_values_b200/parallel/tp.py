"""Tensor parallelism over KV heads.

Two layers live here.

**Fused GEMM + collective kernels** (:class:`TPContext`, ``csrc/gemm_sm100.cu``). Between blocks the activations are
sharded over *tokens*; a block is all-gather→QKV GEMM, local cache update + attention for the rank's KV heads (cache
policy state is per KV head, so eviction needs no communication), attn-out GEMM→reduce-scatter (+ residual),
all-gather→MLP-up GEMM, MLP-down GEMM→reduce-scatter (+ residual). The reduce-scatter is the GEMM's epilogue
(finished tiles are stored straight into the owner rank's receive buffer over NVLink, remote owners first), and the
all-gather feeds the GEMM's TMA producer chunk by chunk from a local staging buffer that copy CTAs of the same kernel
fill from the peers.

**A sharded model that runs through the ordinary stack** (:class:`TPComm`, ``TPGPT`` / ``TPLoRAGPT``, ``TPBlock``).
``qkv`` and the MLP up projections are column parallel, the attention and MLP output projections row parallel and end
in this package's all-reduce (``csrc/comm.cu``: one-shot kernel for the rows of a decode step, fused with the residual
add and the next RMSNorm; two-shot kernel for prefill chunks); chunks whose rows divide by ``128 · world`` may take the
fused path above. Caches, chunked inference, generation with the captured decode step, evaluation, autograd (LoRA
included), data parallel x tensor parallel training and checkpoints of the whole model work as with a ``GPT``. The
sharding rules are in :mod:`keys_values_b200.parallel.tp_shard`.

NCCL is used to exchange the IPC handles, for per-row scalars (vocabulary-parallel loss, gradient norm), to gather
token-sharded rows at the end of a chunk, and in the reference paths of the tests. The reference library has no tensor
parallelism (``README.md:273-275``); this module is additive API.
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


# =====================================================================================================
# Tensor-parallel model that runs through the ordinary single-GPU stack
# =====================================================================================================
#
# ``TPGPT`` is a :class:`GPT` whose blocks hold this rank's shard of the attention heads and of the MLP
# columns; the two row-parallel projections of a block end in an all-reduce. Activations between blocks are
# replicated, so everything that works with a ``GPT`` (caches and their eviction policies, chunked
# inference, generation, the captured decode step, evaluation) works with a ``TPGPT`` unchanged, for any
# batch size and any number of rows. The all-reduce is this package's own: a one-shot peer-memory kernel
# for the few rows of a decode step (one NVLink round trip, graph-capturable), the two-shot in-place kernel
# of :class:`SymmetricArena` for the chunks of a prefill.


class TPComm:
    """All-reduce (sum) of the outputs of row-parallel linears over the ranks of ``group``.

    The producer GEMM writes straight into symmetric memory (:meth:`out_buffer`), :meth:`all_reduce`
    returns the sum (plus an optional residual). Small payloads (up to ``small_bytes``) are reduced by
    ``kvb_oneshot_allreduce``; they rotate over slots ("sites") so that a slot is never rewritten while a
    peer may still read it. Eager calls use the sites ``[0, EAGER_SITES)`` with epochs counted on the host;
    calls recorded into a CUDA graph use the sites above them with epochs ``k + 1 + *epoch_word`` (``k``: index
    of the call in the captured step; the graph adds the number of captured calls to the device word at its
    end, so every replay has fresh epochs). Larger payloads use two alternating arenas, grown on demand,
    and the two-shot kernel. On CPU ranks (gloo) the library all-reduce stands in, so that the host logic is
    testable without GPUs."""

    EAGER_SITES = 64
    GRAPH_SITES = 128

    def __init__(self, world: int, rank: int, device, group=None, small_bytes: int = 256 << 10, timeout_s: float = 20.0,
                 dtype: torch.dtype = torch.bfloat16):
        self.world, self.rank, self.group = world, rank, group
        self.device = torch.device(device)
        self.native = self.device.type == "cuda" and world > 1
        self.small_bytes, self.timeout_s, self.dtype = small_bytes, timeout_s, dtype
        self.eager_calls = 0           # one-shot calls issued eagerly so far
        self.captured_calls = 0        # one-shot calls recorded in the graph that is being (or was last) captured
        self._capturing = False
        self._large: List[Optional["SymmetricArena"]] = [None, None]
        self._large_numel = 0
        self._large_calls = 0
        self._pending: Optional[tuple] = None
        if self.native:
            n_sites = self.EAGER_SITES + self.GRAPH_SITES
            self._flag_bytes = 16 * 16 * 4  # [writer rank][CTA] words per site
            self.slots = _SymmBuffer(n_sites * small_bytes, self.device, world, rank, group)
            self.flags = _SymmBuffer(n_sites * self._flag_bytes, self.device, world, rank, group)
            self.epoch_word = torch.zeros(1, dtype=torch.int32, device=self.device)
            dist.barrier(group=group)

    # ----------------------------------------------------------------------- buffers
    def _next_site(self) -> int:
        if self._capturing:
            return self.EAGER_SITES + self.captured_calls % self.GRAPH_SITES
        return self.eager_calls % self.EAGER_SITES

    def out_buffer(self, rows: int, features: int, dtype: torch.dtype) -> torch.Tensor:
        """``(rows, features)`` tensor for the partial result of this rank; hand it to :meth:`all_reduce` next."""
        if not self.native:
            return torch.empty((rows, features), dtype=dtype, device=self.device)
        if dtype != self.dtype:
            raise ValueError(f"this communicator reduces {self.dtype}, got {dtype}")
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = rows * features * esz
        if nbytes <= self.small_bytes and nbytes % 16 == 0:
            site = self._next_site()
            buf = self.slots.bytes[site * self.small_bytes : site * self.small_bytes + nbytes].view(dtype).view(rows, features)
            self._pending = ("small", site, buf)
            return buf
        if self._capturing:
            raise RuntimeError(f"a payload of {nbytes} bytes cannot be reduced inside a captured step (limit {self.small_bytes})")
        numel = rows * features
        if numel > self._large_numel:
            self._grow_large(numel)
        par = self._large_calls & 1
        buf = self._large[par].tensor[:numel].view(rows, features)
        self._pending = ("large", par, buf)
        return buf

    def _grow_large(self, numel: int) -> None:
        from keys_values_b200.parallel.symm import SymmetricArena

        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # nobody still reads an arena that is about to go
        for a in self._large:
            if a is not None:
                a.close()
        numel = (numel + 4095) // 4096 * 4096
        self._large = [SymmetricArena(numel, self.dtype, self.device, self.world, self.rank, self.group, self.timeout_s) for _ in range(2)]
        self._large_numel = numel

    # --------------------------------------------------------------------- all-reduce
    def all_reduce(self, buf: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum of ``buf (rows, features)`` over the ranks (+ ``residual``). The result may live in
        symmetric memory that the call after the next one reuses: consume it before."""
        if self.world == 1:
            return buf if residual is None else buf + residual
        if not self.native:
            dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=self.group)
            return buf if residual is None else buf + residual
        kind, idx, mine = self._pending or (None, None, None)
        if mine is None or mine.data_ptr() != buf.data_ptr():
            # a tensor that was not produced into symmetric memory: copy it in
            mine = self.out_buffer(buf.shape[0], buf.shape[1], buf.dtype)
            mine.copy_(buf)
            kind, idx, _ = self._pending
        self._pending = None
        if kind == "large":
            arena = self._large[idx]
            self._large_calls += 1
            arena.all_reduce_mean_(0, buf.numel(), scale=1.0)
            return mine if residual is None else mine + residual
        site = idx
        out = torch.empty_like(mine)
        st = _cu.status_word(self.device)
        if residual is not None:
            residual = residual.contiguous()
        if self._capturing:
            base, word = self.captured_calls + 1, self.epoch_word
        else:
            base, word = self.eager_calls + 1, None
        _cu._check(
            _cu.lib().kvb_oneshot_allreduce(
                self.slots.ptr_array(site * self.small_bytes), self.flags.ptr_array(site * self._flag_bytes), self.rank, self.world,
                ctypes.c_longlong(mine.numel()), _cu._p(residual), _cu._p(out), ctypes.c_uint(base & 0xFFFFFFFF),
                _cu._p(word), _cu._code(mine.dtype), _cu._p(st), ctypes.c_double(self.timeout_s), _cu._stream(mine),
            ),
            "oneshot_allreduce",
        )
        _cu._count()
        if self._capturing:
            self.captured_calls += 1
        else:
            self.eager_calls += 1
        return out

    def all_reduce_add_norm(self, buf: torch.Tensor, residual: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                            unit_offset: bool = False):
        """``x = sum over ranks of buf + residual`` and ``rmsnorm(x) · norm_weight`` in one kernel (a decode step's
        handful of rows: one CTA per row). ``buf`` must come from :meth:`out_buffer`. Returns ``(x, normed)``."""
        rows, feat = buf.shape
        fused = (self.native and self._pending is not None and self._pending[0] == "small" and self._pending[2].data_ptr() == buf.data_ptr()
                 and rows <= 16 and feat % 8 == 0 and feat <= 8192 and buf.dtype in (torch.bfloat16, torch.float16)
                 and norm_weight.dtype == buf.dtype)
        if not fused:
            from keys_values_b200 import ops

            x = self.all_reduce(buf, residual)
            return x, ops.rmsnorm(x, norm_weight, eps, unit_offset)
        _, site, mine = self._pending
        self._pending = None
        out_x, out_n = torch.empty_like(mine), torch.empty_like(mine)
        st = _cu.status_word(self.device)
        if residual is not None:
            residual = residual.contiguous()
        if self._capturing:
            base, word = self.captured_calls + 1, self.epoch_word
        else:
            base, word = self.eager_calls + 1, None
        _cu._check(
            _cu.lib().kvb_oneshot_allreduce_norm(
                self.slots.ptr_array(site * self.small_bytes), self.flags.ptr_array(site * self._flag_bytes), self.rank, self.world,
                rows, feat, _cu._p(residual), _cu._p(norm_weight.contiguous()), ctypes.c_float(eps), int(bool(unit_offset)), _cu._p(out_x),
                _cu._p(out_n), ctypes.c_uint(base & 0xFFFFFFFF), _cu._p(word), _cu._code(mine.dtype), _cu._p(st),
                ctypes.c_double(self.timeout_s), _cu._stream(mine),
            ),
            "oneshot_allreduce_norm",
        )
        _cu._count()
        if self._capturing:
            self.captured_calls += 1
        else:
            self.eager_calls += 1
        return out_x, out_n

    # ------------------------------------------------------------------ graph capture
    def begin_capture(self) -> None:
        self._capturing, self.captured_calls = True, 0

    def end_capture(self) -> None:
        """Last operation inside the capture: every replay moves the epochs of the captured calls on."""
        self._capturing = False
        if self.native and self.captured_calls:
            if self.captured_calls % self.GRAPH_SITES == 1:
                raise RuntimeError("the last captured all-reduce would share its slot with the first one of the next replay")
            self.epoch_word.add_(self.captured_calls)

    def close(self) -> None:
        if self.native:
            for a in self._large:
                if a is not None:
                    a.close()
            self._large = [None, None]
            self.slots.close()
            self.flags.close()


class RowParallelLinear(torch.nn.Linear):
    """``all_reduce(x_shard @ W_shard^T) (+ bias)``: the weight holds this rank's columns; the bias is kept by
    rank 0 only (the sum over ranks adds it once)."""

    comm: Optional[TPComm] = None

    @classmethod
    def from_linear(cls, linear: torch.nn.Linear, comm: TPComm) -> "RowParallelLinear":
        new = cls.__new__(cls)
        torch.nn.Module.__init__(new)
        new.in_features, new.out_features = linear.in_features, linear.out_features
        new.weight = linear.weight
        new.bias = linear.bias
        new.comm = comm
        return new

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        comm = self.comm
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad):
            y = _AllReduceSum.apply(torch.nn.functional.linear(x2, self.weight, self.bias), comm)
            return y.view(*lead, self.out_features)
        buf = comm.out_buffer(x2.shape[0], self.out_features, x.dtype)
        if self.bias is not None:
            torch.addmm(self.bias, x2, self.weight.t(), out=buf)
        else:
            torch.mm(x2, self.weight.t(), out=buf)
        return comm.all_reduce(buf).view(*lead, self.out_features)


class _AllReduceSum(torch.autograd.Function):
    """Sum over ranks in the forward pass; the gradient of a sum reaches every rank unchanged."""

    @staticmethod
    def forward(ctx, x, comm):
        return comm.all_reduce(x.contiguous().clone())

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyToShards(torch.autograd.Function):
    """Identity in the forward pass (the replicated input of column-parallel linears); the gradients of the
    ranks' shards are summed in the backward pass."""

    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return x

    @staticmethod
    def backward(ctx, g):
        return ctx.comm.all_reduce(g.contiguous().clone().view(-1, g.shape[-1])).view_as(g), None


class _GatherColumns(torch.autograd.Function):
    """``(rows,)`` per rank → ``(rows, world)`` on every rank. What follows is computed identically everywhere (one
    loss, replicated), so the gradient of a rank's own column is the gradient of its input."""

    @staticmethod
    def forward(ctx, x, comm):
        ctx.rank = comm.rank
        parts = [torch.empty_like(x) for _ in range(comm.world)]
        dist.all_gather(parts, x.contiguous(), group=comm.group)
        return torch.stack(parts, dim=1)

    @staticmethod
    def backward(ctx, g):
        return g[:, ctx.rank].contiguous(), None


class _SumScalars(torch.autograd.Function):
    """Sum over ranks of a small fp32 tensor (library all-reduce: these are per-row scalars); identity backward."""

    @staticmethod
    def forward(ctx, x, comm):
        y = x.contiguous().clone()
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=comm.group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


def vocab_parallel_cross_entropy(x: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, comm: "TPComm",
                                 ignore_index: int = -100) -> torch.Tensor:
    """Token cross-entropy with the vocabulary split over the ranks: rank ``r`` multiplies ``x (rows, E)`` (the final
    hidden states after ``ln_f``, replicated) with rows ``[r·V/world, (r+1)·V/world)`` of the head's weight only, so
    the logits of a position never exist in one place. Per row the ranks exchange two numbers (the log-sum-exp of
    their slice and, from the owner, the target's logit): ``loss = logsumexp_r(lse_r) − logit_target``. Returns the
    per-row losses (0 where ``targets == ignore_index``); differentiable in ``x`` and ``weight``."""
    V = weight.shape[0]
    world, rank = comm.world, comm.rank
    per = (V + world - 1) // world
    v0, v1 = min(rank * per, V), min((rank + 1) * per, V)
    tg = targets.reshape(-1)
    if torch.is_grad_enabled() and x.requires_grad:
        x = _CopyToShards.apply(x, comm)  # every rank contributes the part of dL/dx that runs through its slice
    if torch.is_grad_enabled() and weight.requires_grad:
        weight = _CopyToShards.apply(weight, comm)  # replicated parameter: rank r produces the gradient of its rows only
    logits = torch.nn.functional.linear(x, weight[v0:v1]).float()  # (rows, V_local)
    lse_local = torch.logsumexp(logits, dim=-1) if v1 > v0 else torch.full_like(tg, float("-inf"), dtype=torch.float32)
    lse = torch.logsumexp(_GatherColumns.apply(lse_local, comm), dim=1)
    mine = (tg >= v0) & (tg < v1)
    picked = logits.gather(1, (tg - v0).clamp(0, max(v1 - v0 - 1, 0)).unsqueeze(1)).squeeze(1)
    target_logit = _SumScalars.apply(torch.where(mine, picked, torch.zeros_like(picked)), comm)
    loss = lse - target_logit
    return torch.where(tg == ignore_index, torch.zeros_like(loss), loss)


from keys_values_b200.parallel.tp_shard import (  # noqa: E402,F401  (re-exported)
    _qkv_segments, _shard_rule, local_config, shard_state_dict, unshard_state_dict,
)


def gather_whole_state_dict(model, only_trainable: bool = False, dst: int = 0):
    """The state dict of the whole model, put together from the shards of the ranks of the model's tensor-parallel
    group, on the group's rank ``dst`` (``None`` elsewhere): what a checkpoint of a run under tensor parallelism
    stores, readable by a run on any number of GPUs. ``only_trainable`` keeps the tensors that are being trained
    (LoRA factors), as a LoRA checkpoint does. The tensors travel as host copies through the process group."""
    comm = model.tp_comm
    trainable = {n for n, p in model.named_parameters() if p.requires_grad}
    mine = {k: v.detach().cpu() for k, v in model.state_dict().items() if not only_trainable or k in trainable}
    if comm.world == 1:
        return mine
    shards = [None] * comm.world if comm.rank == dst else None
    dist.gather_object(mine, shards, dst=dist.get_global_rank(comm.group, dst) if comm.group is not None else dst, group=comm.group)
    if comm.rank != dst:
        return None
    return unshard_state_dict(shards, model.full_config)


def clip_grad_norm_sharded(model, max_norm: float) -> torch.Tensor:
    """Gradient clipping for a shard: the norm is that of the whole model (squares of sharded tensors summed over
    the ranks, replicated tensors counted once), so every rank scales by the same factor and replicated
    parameters stay equal. Returns the norm."""
    comm = model.tp_comm
    cfg = model.full_config
    sq_sharded = torch.zeros((), dtype=torch.float32, device=comm.device)
    sq_rep = torch.zeros((), dtype=torch.float32, device=comm.device)
    grads = []
    for name, p in model.named_parameters():
        if p.grad is None:
            continue
        grads.append(p.grad)
        sq = p.grad.float().pow(2).sum()
        if _shard_rule(name, cfg)[0] in ("rep", "rank0"):
            sq_rep = sq_rep + sq
        else:
            sq_sharded = sq_sharded + sq
    if comm.world > 1:
        dist.all_reduce(sq_sharded, op=dist.ReduceOp.SUM, group=comm.group)  # a scalar: library plumbing
    norm = (sq_sharded + sq_rep).sqrt()
    factor = (max_norm / (norm + 1e-6)).clamp(max=1.0)
    for g in grads:
        g.mul_(factor.to(g.dtype))
    return norm


def load_sharded_checkpoint(model, checkpoint_dir) -> None:
    """Fill a :class:`TPGPT` with its shard of ``checkpoint_dir/lit_model.pth`` (the file of the whole model,
    memory-mapped: a rank reads only the slices it keeps)."""
    from pathlib import Path

    path = Path(checkpoint_dir) / "lit_model.pth"
    if not path.is_file() or path.stat().st_size == 0:
        return  # a directory with only the configuration: the random initialisation stays (tests, benchmarks)
    sd = torch.load(path, map_location="cpu", mmap=True, weights_only=True)
    sd = sd.get("model", sd)
    comm = model.tp_comm
    model.load_state_dict(shard_state_dict(sd, model.full_config, comm.world, comm.rank))


def plain_state_dict(gpt_model) -> dict:
    """State dict of a model in the key layout of the plain :class:`GPT`; LoRA adapters are merged into the
    linears they decorate first (the model is changed in place)."""
    from keys_values_b200.models import lora as lora_mod

    if any(isinstance(m, lora_mod.LoRALinear) for m in gpt_model.modules()):
        lora_mod.merge_lora_weights(gpt_model)
    out = {}
    for k, v in gpt_model.state_dict().items():
        if "lora_" in k:
            continue
        out[k.replace(".linear.", ".")] = v
    return out


def tp_model_from(gpt_model, comm: "TPComm", device, dtype, yarn_rope: bool = True):
    """Shard a whole model (on the host; LoRA adapters are merged) over the ranks of ``comm``: returns this rank's
    :class:`TPGPT` on ``device``."""
    import dataclasses

    from keys_values_b200.config import Config
    from keys_values_b200.models.pos_encoding import position_encoding_factory

    src = gpt_model.config
    cfg = Config(**{f.name: getattr(src, f.name) for f in dataclasses.fields(Config) if f.init})
    sd = shard_state_dict(plain_state_dict(gpt_model), cfg, comm.world, comm.rank)
    local = local_config(cfg, comm.world)
    cls = globals().get("TPGPT") or __getattr__("TPGPT")
    with torch.device(device):
        model = cls(cfg, comm, pos_encoding=position_encoding_factory(local, do_yarn=yarn_rope, device=device))
    model = model.to(dtype)
    model.load_state_dict(sd)
    return model


class RowShard:
    """Token rows of an activation ``(B, T, E)`` sharded over the ranks (flattened batch-major; rank ``r`` holds
    rows ``[r·n, (r+1)·n)``). Blocks of a :class:`TPGPT` pass it from one to the next on the fused path; whoever
    needs the whole tensor calls :meth:`full` (one all-gather, cached) or indexes it."""

    def __init__(self, rows: torch.Tensor, shape, comm: "TPComm"):
        self.rows, self.shape, self.comm = rows, tuple(shape), comm
        self._full: Optional[torch.Tensor] = None

    def full(self) -> torch.Tensor:
        if self._full is None:
            out = torch.empty((self.rows.shape[0] * self.comm.world, self.rows.shape[1]), dtype=self.rows.dtype, device=self.rows.device)
            dist.all_gather_into_tensor(out, self.rows.contiguous(), group=self.comm.group)
            self._full = out.view(self.shape)
        return self._full

    def __getitem__(self, idx):
        return self.full()[idx]

    @property
    def dtype(self):
        return self.rows.dtype

    @property
    def device(self):
        return self.rows.device


def dense(x):
    """The whole tensor behind ``x`` (a tensor, or a :class:`RowShard`)."""
    return x.full() if isinstance(x, RowShard) else x


def _tp_classes(lora: bool):
    from keys_values_b200 import ops
    from keys_values_b200.models.model import LLaMAMLP, RMSNorm

    if lora:
        from keys_values_b200.models.lora import GPT, Block
    else:
        from keys_values_b200.models.model import GPT, Block

    class TPBlock(Block):
        """A block of the shard. Inference chunks whose rows divide by ``128 · world`` take the fused path:
        all-gather→QKV GEMM, attention over this rank's heads, projection GEMM→reduce-scatter (+ residual),
        all-gather→MLP-up GEMM, SwiGLU, MLP-down GEMM→reduce-scatter (+ residual), with the activations
        between blocks sharded over token rows. Everything else (decode steps, ragged chunks, training) runs
        the ordinary block with the all-reduce inside the row-parallel projections."""

        owner = None  # the TPGPT, set after construction (not a sub-module: no reference cycle in the module tree)

        def _fusable(self, rows: int) -> bool:
            gpt = self.owner()
            c = self.config
            return (
                gpt is not None and gpt.fused_prefill and gpt.tp_comm.native and not torch.is_grad_enabled()
                and rows % (128 * gpt.tp_comm.world) == 0 and rows // gpt.tp_comm.world >= 128
                and type(self.mlp) is LLaMAMLP and isinstance(self.norm_1, RMSNorm) and isinstance(self.norm_2, RMSNorm)
                and not c.parallel_residual and not c.post_attention_norm and not c.post_mlp_norm and not c.bias and not c.attn_bias
                and self.attn.kv_cache is not None and type(self.attn.qkv) is torch.nn.Linear
                and self.attn.qkv.weight.dtype == torch.bfloat16
            )

        def _few_rows(self, rows: int) -> bool:
            """Single-token steps: the residual add and the RMSNorm after each all-reduce run inside its kernel."""
            gpt = self.owner()
            c = self.config
            return (
                gpt is not None and gpt.tp_comm.native and not torch.is_grad_enabled() and rows <= 16
                and c.n_embd % 8 == 0 and c.n_embd <= 8192 and rows * c.n_embd * 2 <= gpt.tp_comm.small_bytes
                and isinstance(self.norm_1, RMSNorm) and isinstance(self.norm_2, RMSNorm) and not c.parallel_residual
                and not c.post_attention_norm and not c.post_mlp_norm and type(self.attn.proj) is RowParallelLinear
                and type(self.mlp.proj) is RowParallelLinear and self.attn.proj.bias is None and self.mlp.proj.bias is None
                and self.attn.proj.weight.dtype == gpt.tp_comm.dtype
            )

        def _forward_few_rows(self, x, token_idx, mha, chunk_sizes):
            comm = self.owner().tp_comm
            B, T, E = x.shape
            rows = B * T
            x2 = x.reshape(rows, E)
            y = self.attn.attend(self.attn.qkv(self.norm_1(x)), token_idx, mha, chunk_sizes)
            buf = comm.out_buffer(rows, E, x.dtype)
            torch.mm(y.reshape(rows, -1), self.attn.proj.weight.t(), out=buf)
            x2, normed = comm.all_reduce_add_norm(buf, x2, self.norm_2.weight, self.norm_2.eps, self.norm_2.add_unit_offset)
            a = ops.swiglu(self.mlp.fc_1(normed), self.mlp.fc_2(normed))  # the caller checked that this is a SwiGLU MLP
            buf = comm.out_buffer(rows, E, x.dtype)
            torch.mm(a, self.mlp.proj.weight.t(), out=buf)
            return comm.all_reduce(buf, residual=x2).view(B, T, E)

        def forward(self, x, token_idx, mha, chunk_sizes=None):
            B, T = token_idx.shape
            if not self._fusable(B * T):
                if type(self.mlp) is LLaMAMLP and self._few_rows(B * T):
                    return self._forward_few_rows(dense(x), token_idx, mha, chunk_sizes)
                return super().forward(dense(x), token_idx, mha, chunk_sizes=chunk_sizes)
            gpt = self.owner()
            comm, c = gpt.tp_comm, self.config
            world, rank = comm.world, comm.rank
            E = c.n_embd
            rows = B * T // world
            ctx = gpt.fused_context(B * T)
            if isinstance(x, RowShard):
                xs = x.rows
            else:
                xs = x.reshape(B * T, E)[rank * rows : (rank + 1) * rows]
            ctx.stage_view(rows, E).copy_(self.norm_1(xs))
            qkv = ctx.allgather_gemm(rows, self.attn.qkv.weight).view(B, T, -1)
            y = self.attn.attend(qkv, token_idx, mha, chunk_sizes)
            xs = ctx.gemm_reduce_scatter(y.reshape(B * T, -1), self.attn.proj.weight, residual=xs)
            ctx.stage_view(rows, E).copy_(self.norm_2(xs))
            h = ctx.allgather_gemm(rows, gpt.fc_weight(self))
            inter = c.intermediate_size
            a = ops.swiglu(h[:, :inter], h[:, inter:])
            xs = ctx.gemm_reduce_scatter(a, self.mlp.proj.weight, residual=xs)
            return RowShard(xs, (B, T, E), comm)

    class TPGPT(GPT):
        """This rank's shard of a model (``full_config`` describes the whole). Built empty; fill it with
        ``load_state_dict(shard_state_dict(full_state_dict, full_config, world, rank))`` or initialise it
        at random. ``tp_comm`` is read by the captured decode step. ``fused_prefill``: whether inference chunks take
        the fused all-gather→GEMM / GEMM→reduce-scatter path (``False``: every chunk on the all-reduce path); the
        default picks what was measured faster, the fused path from 8 ranks on (+4 % there, −6.5 % at 4, −19 % at 2)."""

        def __init__(self, full_config, comm: TPComm, fused_prefill: Optional[bool] = None, **mha_kwargs):
            super().__init__(local_config(full_config, comm.world), **mha_kwargs)
            import weakref

            self.full_config = full_config
            self.tp_comm = comm
            self.fused_prefill = comm.world >= 8 if fused_prefill is None else fused_prefill
            self._fused_ctx: Optional[TPContext] = None
            self._fc_cat = {}
            if lora and getattr(full_config, "lora_kind", "default") != "default":
                raise NotImplementedError("tensor parallelism supports plain LoRA adapters (lora_kind = 'default')")
            for block in self.transformer.h:
                block.owner = weakref.ref(self)
                for holder, name in ((block.attn, "proj"), (block.mlp, "proj")):
                    mod = getattr(holder, name)
                    if type(mod) is torch.nn.Linear:
                        setattr(holder, name, RowParallelLinear.from_linear(mod, comm))
                    else:  # a LoRA linear: W holds this rank's columns, A its columns too, B is replicated
                        mod.register_forward_hook(self._sum_output_hook)
                    bias = getattr(getattr(holder, name), "bias", None)
                    if bias is not None and comm.rank != 0:
                        # the sum over ranks must add the bias once: rank 0 owns it, the others hold a frozen zero
                        bias.data.zero_()
                        bias.requires_grad_(False)
                # the inputs of the column-parallel linears (after the norms; the residual path is replicated)
                block.attn.register_forward_pre_hook(self._shard_input_hook)
                block.mlp.register_forward_pre_hook(self._shard_input_hook)
                # Replicated parameters of which every rank sees a part of the gradient: the per-head QK norms (one
                # weight serves all heads), LoRA A of column-parallel linears and LoRA B of row-parallel linears
                shared = [p for norm in (block.attn.norm_q, block.attn.norm_k) if norm is not None for p in norm.parameters()]
                for mod, which in ((block.attn.qkv, "lora_A"), (getattr(block.mlp, "fc_1", None), "lora_A"),
                                   (getattr(block.mlp, "fc_2", None), "lora_A"), (getattr(block.mlp, "fc", None), "lora_A"),
                                   (block.attn.proj, "lora_B"), (block.mlp.proj, "lora_B")):
                    p = getattr(mod, which, None) if mod is not None else None
                    if isinstance(p, torch.nn.Parameter):
                        shared.append(p)
                for p in shared:
                    p.register_hook(self._sum_over_ranks)

        def _sum_output_hook(self, module, args, output):
            return _AllReduceSum.apply(output.reshape(-1, output.shape[-1]), self.tp_comm).view_as(output)

        def _make_block(self, config, block_idx):
            return TPBlock(config, block_idx)

        def _sum_over_ranks(self, g):
            return self.tp_comm.all_reduce(g.reshape(1, -1).clone()).view_as(g)

        def _shard_input_hook(self, module, args):
            # training: the gradient of the input of column-parallel linears is the sum over the ranks' shards
            x = args[0]
            if torch.is_grad_enabled() and x.requires_grad:
                return (_CopyToShards.apply(x, self.tp_comm),) + tuple(args[1:])
            return None

        # ------------------------------------------------------------------ fused path
        def fused_context(self, total_rows: int) -> TPContext:
            ctx = self._fused_ctx
            if ctx is None or total_rows > ctx.max_rows:
                if ctx is not None:
                    torch.cuda.synchronize(self.tp_comm.device)
                    dist.barrier(group=self.tp_comm.group)
                    ctx.close()
                comm = self.tp_comm
                ctx = TPContext(comm.world, comm.rank, comm.device, total_rows, self.config.n_embd, comm.group, comm.timeout_s)
                self._fused_ctx = ctx
            return ctx

        def fc_weight(self, block) -> torch.Tensor:
            """``fc_1 | fc_2`` of a block as one matrix (one all-gather→GEMM for both); the two parameters become
            views of it the first time it is asked for, so the weights are not held twice."""
            key = id(block)
            w = self._fc_cat.get(key)
            f1, f2 = block.mlp.fc_1.weight, block.mlp.fc_2.weight
            if w is None or f1.data_ptr() != w.data_ptr():
                w = torch.cat((f1.data, f2.data)).contiguous()
                n = f1.shape[0]
                f1.data, f2.data = w[:n], w[n:]
                self._fc_cat[key] = w
            return w

        def forward(self, idx, skip_lm_head: bool = False, chunk_sizes=None):
            if idx.ndim == 1:
                idx = idx.unsqueeze(0)
            T = idx.size(1)
            caches = self.get_kv_caches()
            input_pos = caches[0].input_pos if caches[0] is not None else 0
            if input_pos + T > self.max_seq_length:
                raise ValueError(f"Cannot forward sequence: input_pos {input_pos} + {T} > max_seq_length {self.max_seq_length}")
            x = self.embed(idx)
            hook = self._start_of_layer_hook
            for block_idx, block in enumerate(self.transformer.h):
                if hook is not None:
                    x = dense(x)
                    hook(x, block_idx)
                x = block(x, idx, self.mha, chunk_sizes=chunk_sizes)
            x = dense(x)
            if hook is not None:
                hook(x, self.config.n_layer)
            return x if skip_lm_head else self.head(x)

        def close(self) -> None:
            if self._fused_ctx is not None:
                self._fused_ctx.close()
                self._fused_ctx = None

    TPGPT.__name__ = TPGPT.__qualname__ = "TPLoRAGPT" if lora else "TPGPT"
    return TPGPT, TPBlock


def __getattr__(name):
    if name in ("TPGPT", "TPBlock"):
        globals()["TPGPT"], globals()["TPBlock"] = _tp_classes(False)
        return globals()[name]
    if name == "TPLoRAGPT":
        globals()["TPLoRAGPT"] = _tp_classes(True)[0]
        return globals()[name]
    raise AttributeError(name)
