"""The 27B-class decode layer stack: the callers of the packed-quant matmul path.

One layer is the matmul sequence of ``Qwen35::forward_cached`` (crates/ferric-llama/src/qwen35.rs:953-1014,
ffn :834-840): rmsnorm -> fused q|k|v projection -> [mixer] -> o projection -> add_rmsnorm ->
fused gate|up + SwiGLU -> down projection -> add.  Attention / GDN and the KV cache are outside this
backend's scope, so the mixer is a pass-through: the q slice of the qkv output feeds the o
projection.  Everything else (shapes, formats, fusion of q|k|v and gate|up into one matrix as
``qm_cat`` does, :380-402) is as the model runs it.

Tensor parallelism (one process per GPU): q|k|v and gate|up are split by output rows, o and down by
input columns on 256-weight super-block boundaries, and the f32 [B, hidden] partial sums of o and
down are all-reduced (2 per layer).  K = 5120 is 20 super-blocks and n_ff = 17408 is 68, which do
not divide by 8, so shards are uneven but aligned (3,3,3,3,2,2,2,2 and 9,9,9,9,8,8,8,8 blocks).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

import torch

from . import synth
from .ops import Context, QMatrix, TPGroup, GGML_Q4_K, GGML_Q6_K


def split_blocks(total_blocks: int, world: int) -> List[int]:
    """Blocks per rank: as even as block granularity allows, larger shards first."""
    base, extra = divmod(total_blocks, world)
    return [base + (1 if r < extra else 0) for r in range(world)]


@dataclass(frozen=True)
class TPPlan:
    """Which slice of each layer matrix one rank owns."""
    world: int
    rank: int
    hidden: int
    n_ff: int
    q_out: int
    kv_out: int
    q_row0: int
    q_rows: int      # rows of Q this rank computes == its K slice of O
    kv_row0: int
    kv_rows: int     # rows of K (and of V)
    ff_row0: int
    ff_rows: int     # rows of gate (and of up) == its K slice of down

    @staticmethod
    def make(world: int, rank: int, hidden: int = 5120, n_ff: int = 17408, q_out: int = 5120,
             kv_out: int = 1024) -> "TPPlan":
        assert 0 <= rank < world
        assert q_out % 256 == 0 and n_ff % 256 == 0 and kv_out % world == 0
        qb = split_blocks(q_out // 256, world)
        fb = split_blocks(n_ff // 256, world)
        assert min(qb) > 0 and min(fb) > 0, "more ranks than 256-column blocks"
        return TPPlan(world, rank, hidden, n_ff, q_out, kv_out,
                      256 * sum(qb[:rank]), 256 * qb[rank],
                      (kv_out // world) * rank, kv_out // world,
                      256 * sum(fb[:rank]), 256 * fb[rank])

    def weight_bytes_per_layer(self) -> int:
        """Algorithmic (on-disk format) weight bytes this rank streams per layer."""
        q4 = lambda r, c: r * c // 256 * 144
        q6 = lambda r, c: r * c // 256 * 210
        return (q4(self.q_rows + 2 * self.kv_rows, self.hidden) + q4(self.hidden, self.q_rows)
                + q4(2 * self.ff_rows, self.hidden) + q6(self.hidden, self.ff_rows))


AllReduce = Callable[[torch.Tensor], None]


class Layer:
    def __init__(self, wqkv: QMatrix, wo: QMatrix, wgu: QMatrix, wdown: QMatrix):
        self.wqkv, self.wo, self.wgu, self.wdown = wqkv, wo, wgu, wdown

    def close(self):
        for w in (self.wqkv, self.wo, self.wgu, self.wdown):
            w.close()


class DecodeStack:
    """``n_layers`` decoder layers' worth of packed-quant matmuls for ``batch`` tokens per step."""

    def __init__(self, ctx: Context, plan: TPPlan, n_layers: int = 64, batch: int = 1, eps: float = 1e-6,
                 all_reduce: Optional[AllReduce] = None, group: Optional[TPGroup] = None, push: bool = True,
                 chain: Optional[bool] = None):
        """`all_reduce`: a callable summing a tensor over ranks in place (e.g. NCCL through torch.distributed).
        `group`: a connected TPGroup -- then the exchange is done by this library's own kernels instead; with
        `push` the o / down products store their partial sums straight into every rank's memory, otherwise each
        rank signals its buffer and the consumers read the peers' buffers.
        `chain`: one launch per matrix, the norms, residual adds and activation preparation riding in the products' own
        launches.  It applies up to 4 tokens (one pass of the GEMV) with one rank or the pushed exchange; by default it is used on one rank up
        to 2 tokens (one activation tile), where it measured faster (4.06 against 4.29 ms per step).  With more tiles
        the one warp that prepares a block becomes the tail of every launch (13.2 against 11.1 ms at 8 tokens), and
        across ranks the exchange's own consumer kernel, spread over a cluster, polls faster than one warp per block
        (3.77 against 3.46 ms per step on 2 GPUs)."""
        self.ctx, self.plan, self.n_layers, self.batch, self.eps = ctx, plan, n_layers, batch, eps
        can_chain = batch <= 4 and (plan.world == 1 or (group is not None and push))
        self.chain = (can_chain and batch <= 2 and plan.world == 1) if chain is None else (chain and can_chain)
        self.all_reduce = all_reduce if (plan.world > 1 and group is None) else None
        self.group = group if plan.world > 1 else None
        self.push = push
        if plan.world > 1 and all_reduce is None and group is None:
            raise ValueError("a tensor-parallel stack needs an all-reduce or an exchange group")
        self.layers: List[Layer] = []
        dev = torch.device("cuda", ctx.device)
        p, B = plan, batch
        f32 = dict(dtype=torch.float32, device=dev)
        self.h = torch.zeros((B, p.hidden), **f32)
        self.xn = torch.empty((B, p.hidden), **f32)
        self.qkv = torch.empty((B, p.q_rows + 2 * p.kv_rows), **f32)
        self.f = torch.empty((B, p.ff_rows), **f32)
        if self.group is not None:      # the row-parallel products write straight into the exchange buffers
            self.o, self.d = self.group.partial(0), self.group.partial(1)
        else:
            self.o = torch.empty((B, p.hidden), **f32)
            self.d = torch.empty((B, p.hidden), **f32)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches_per_step = 0

    # -- weights ---------------------------------------------------------------------------
    def add_layer(self, wqkv: QMatrix, wo: QMatrix, wgu: QMatrix, wdown: QMatrix) -> None:
        p = self.plan
        assert (wqkv.rows(), wqkv.cols()) == (p.q_rows + 2 * p.kv_rows, p.hidden)
        assert (wo.rows(), wo.cols()) == (p.hidden, p.q_rows)
        assert (wgu.rows(), wgu.cols()) == (2 * p.ff_rows, p.hidden)
        assert (wdown.rows(), wdown.cols()) == (p.hidden, p.ff_rows)
        self.layers.append(Layer(wqkv, wo, wgu, wdown))

    def build_synthetic(self, seed: int = 4) -> None:
        """Random-init weights of the named shapes and block distributions, generated on the device.

        Layer l, matrix k, rank r draw from an independent stream; a rank's matrices have its shard's
        shape (the values are synthetic, so nothing is gained by generating the whole tensor first)."""
        p, dev = self.plan, torch.device("cuda", self.ctx.device)
        for l in range(self.n_layers):
            s = (seed * 1_000_003 + l) * 64 + p.rank * 4

            def mk(ty, rows, cols, k):
                raw = synth.matrix_on_device(ty, rows, cols, s + k, dev)
                return QMatrix.from_device_bytes(self.ctx, raw, ty, rows, cols)

            self.add_layer(mk(GGML_Q4_K, p.q_rows + 2 * p.kv_rows, p.hidden, 0), mk(GGML_Q4_K, p.hidden, p.q_rows, 1),
                           mk(GGML_Q4_K, 2 * p.ff_rows, p.hidden, 2), mk(GGML_Q6_K, p.hidden, p.ff_rows, 3))
        self.reserve()

    def reserve(self) -> None:
        need = 0
        for L in self.layers[:1]:
            need = max(w.scratch_bytes(self.batch) for w in (L.wqkv, L.wo, L.wgu, L.wdown))
        if self.chain:
            self.ctx.chain_reserve(need)
        else:
            self.ctx.reserve_scratch(need)

    def weight_bytes_per_step(self) -> int:
        return sum(w.nbytes() for L in self.layers for w in (L.wqkv, L.wo, L.wgu, L.wdown))

    # -- one token step --------------------------------------------------------------------
    def step(self) -> torch.Tensor:
        """h <- stack(h) on the device, in place; returns h.

        Per layer: [norm + prepare] -> q|k|v -> o (+ all-reduce) -> [add + norm + prepare] ->
        gate|up+SwiGLU -> down (+ all-reduce); the residual add after down is fused into the next
        layer's first kernel."""
        c, p = self.ctx, self.plan
        before = c.launches()
        n = len(self.layers)
        if self.batch > 8:
            return self._step_wide(before)
        if self.chain:
            return self._step_chain(before)
        m = self.layers[0].wqkv.add_rmsnorm_prepare(self.h, None, None, self.eps)
        G = self.group
        for i, L in enumerate(self.layers):
            L.wqkv.matmul_prepared(m, out=self.qkv)
            if G is not None and self.push:
                G.matmul_push(0, L.wo, self.qkv[:, :p.q_rows])
                G.add_rmsnorm_prepare(0, L.wgu, self.h, None, self.eps, sum_out=self.h, pushed=True)
            elif G is not None:
                L.wo.matmul(self.qkv[:, :p.q_rows], out=self.o)      # mixer pass-through: q feeds o
                G.signal(0)
                G.add_rmsnorm_prepare(0, L.wgu, self.h, None, self.eps, sum_out=self.h)
            else:
                L.wo.matmul(self.qkv[:, :p.q_rows], out=self.o)
                if self.all_reduce:
                    self.all_reduce(self.o)
                L.wgu.add_rmsnorm_prepare(self.h, self.o, None, self.eps, sum_out=self.h)
            L.wgu.matmul_prepared(m, out=self.f, swiglu=True)
            nxt = self.layers[i + 1].wqkv if i + 1 < n else self.layers[0].wqkv
            last_norm = self.xn if i + 1 == n else None      # after the last layer the norm itself is the result
            if G is not None and self.push:
                G.matmul_push(1, L.wdown, self.f)
                G.add_rmsnorm_prepare(1, nxt, self.h, None, self.eps, sum_out=self.h, norm_out=last_norm, pushed=True)
            elif G is not None:
                L.wdown.matmul(self.f, out=self.d)
                G.signal(1)
                G.add_rmsnorm_prepare(1, nxt, self.h, None, self.eps, sum_out=self.h, norm_out=last_norm)
            else:
                L.wdown.matmul(self.f, out=self.d)
                if self.all_reduce:
                    self.all_reduce(self.d)
                nxt.add_rmsnorm_prepare(self.h, self.d, None, self.eps, sum_out=self.h, norm_out=last_norm)
        self.launches_per_step = c.launches() - before
        return self.h

    def _step_chain(self, before: int) -> torch.Tensor:
        """The same step as four launches per layer: q|k|v prepares o's input, o adds to the residual stream and prepares
        gate|up's (whose result takes the 1/rms factor), gate|up+SwiGLU prepares down's, down adds to the residual
        stream and prepares the next layer's q|k|v.  Slots alternate 0 -> 1 -> 0 -> 1 -> 0 through a layer."""
        c, p, G = self.ctx, self.plan, self.group
        n = len(self.layers)
        m = self.layers[0].wqkv.add_rmsnorm_prepare(self.h, None, None, self.eps)       # slot 0, already normalised
        for i, L in enumerate(self.layers):
            nxt = self.layers[i + 1].wqkv if i + 1 < n else self.layers[0].wqkv
            L.wqkv.chain_matmul(m, self.qkv, in_slot=0, in_rms=i > 0, eps=self.eps, next=1, next_qm=L.wo)
            if G is not None:
                G.chain_matmul(0, L.wo, m, 1, L.wgu, self.h)
            else:
                L.wo.chain_matmul(m, self.o, in_slot=1, next=2, next_qm=L.wgu, h=self.h)
            L.wgu.chain_matmul(m, self.f, swiglu=True, in_slot=0, in_rms=True, eps=self.eps, next=1, next_qm=L.wdown)
            if G is not None:
                G.chain_matmul(1, L.wdown, m, 1, nxt, self.h)
            else:
                L.wdown.chain_matmul(m, self.d, in_slot=1, next=2, next_qm=nxt, h=self.h)
        c.add_rmsnorm(self.h, None, None, self.eps, norm_out=self.xn)      # after the last layer the norm itself is the result
        self.launches_per_step = c.launches() - before
        return self.h

    def _step_wide(self, before: int) -> torch.Tensor:
        """The same step for more than 8 tokens: the products go through ``matmul`` / ``try_matmul_swiglu`` so that the
        Q4_K ones can take the tensor-core kernel, which prepares its own activation form; add + rmsnorm runs unfused."""
        c, p = self.ctx, self.plan
        n = len(self.layers)
        c.add_rmsnorm(self.h, None, None, self.eps, norm_out=self.xn)
        for i, L in enumerate(self.layers):
            L.wqkv.matmul(self.xn, out=self.qkv)
            if self.group is not None:      # the library's two-step pushed all-reduce, fused into add + rmsnorm; the
                # product scatters its own result (step 1) where its K range is cut across CTAs
                self.group.matmul_scatter(0, L.wo, self.qkv[:, :p.q_rows])
                self.group.allreduce_add_rmsnorm(0, self.o, self.h, None, self.eps, sum_out=self.h, norm_out=self.xn, steps=6)
            else:
                L.wo.matmul(self.qkv[:, :p.q_rows], out=self.o)
                if self.all_reduce:
                    self.all_reduce(self.o)
                c.add_rmsnorm(self.h, self.o, None, self.eps, sum_out=self.h, norm_out=self.xn)
            if L.wgu.try_matmul_swiglu(self.xn, out=self.f) is None:
                raise RuntimeError("gate|up matrix is not fusable")
            if self.group is not None:
                self.group.matmul_scatter(1, L.wdown, self.f)
                self.group.allreduce_add_rmsnorm(1, self.d, self.h, None, self.eps, sum_out=self.h, norm_out=self.xn, steps=6)
            else:
                L.wdown.matmul(self.f, out=self.d)
                if self.all_reduce:
                    self.all_reduce(self.d)
                c.add_rmsnorm(self.h, self.d, None, self.eps, sum_out=self.h, norm_out=self.xn)
        self.launches_per_step = c.launches() - before
        return self.h

    def capture(self, warmup: int = 2) -> None:
        """Record one step into a CUDA graph (launch-bound loop: ~10 kernels per layer)."""
        side = torch.cuda.Stream(device=self.ctx.device)
        side.wait_stream(torch.cuda.current_stream(self.ctx.device))
        with torch.cuda.stream(side):
            self.ctx.use_torch_stream()
            for _ in range(warmup):
                self.step()
        torch.cuda.current_stream(self.ctx.device).wait_stream(side)
        torch.cuda.synchronize(self.ctx.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.ctx.use_torch_stream()
            self.step()
        self.ctx.use_torch_stream()
        self.graph = g

    def run(self) -> torch.Tensor:
        if self.graph is not None:
            self.graph.replay()
            return self.h
        return self.step()

    def step_host(self, x_host: torch.Tensor, y_host: torch.Tensor) -> None:
        """One step with HOST (pinned) input and result buffers: copy in, run, copy out, wait."""
        self.h.copy_(x_host, non_blocking=True)
        self.run()
        y_host.copy_(self.h, non_blocking=True)
        torch.cuda.current_stream(self.ctx.device).synchronize()

    def close(self) -> None:
        for L in self.layers:
            L.close()
        self.layers = []


def shard_bytes(raw, ggml_type: int, rows: int, cols: int, row0: int, nrows: int, col0: int, ncols: int):
    """Host-side twin of ``QMatrix.from_bytes_view``: the raw GGUF block bytes of a row range x K range.

    Row ranges are contiguous byte ranges; K ranges gather each row's blocks (256-column aligned)."""
    import numpy as np

    vals, bb = synth.BLOCK[ggml_type]
    assert cols % vals == 0 and col0 % vals == 0 and ncols % vals == 0
    a = np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, np.ndarray) else raw
    blocks = a.reshape(rows, cols // vals, bb)
    return np.ascontiguousarray(blocks[row0:row0 + nrows, col0 // vals:(col0 + ncols) // vals, :]).reshape(-1)


def layer_shards(plan: TPPlan, full: dict) -> dict:
    """Slice one layer's full matrices {"q","k","v","o","gate","up","down"} (raw bytes, GGUF [out, in]) into this
    rank's fused shards {"qkv","o","gate_up","down"}: q|k|v and gate|up stacked along rows as ``qm_cat`` does
    (crates/ferric-llama/src/qwen35.rs:380-402), o and down cut along K."""
    import numpy as np

    p = plan
    q = shard_bytes(full["q"], GGML_Q4_K, p.q_out, p.hidden, p.q_row0, p.q_rows, 0, p.hidden)
    k = shard_bytes(full["k"], GGML_Q4_K, p.kv_out, p.hidden, p.kv_row0, p.kv_rows, 0, p.hidden)
    v = shard_bytes(full["v"], GGML_Q4_K, p.kv_out, p.hidden, p.kv_row0, p.kv_rows, 0, p.hidden)
    g = shard_bytes(full["gate"], GGML_Q4_K, p.n_ff, p.hidden, p.ff_row0, p.ff_rows, 0, p.hidden)
    u = shard_bytes(full["up"], GGML_Q4_K, p.n_ff, p.hidden, p.ff_row0, p.ff_rows, 0, p.hidden)
    return {
        "qkv": np.concatenate([q, k, v]),
        "o": shard_bytes(full["o"], GGML_Q4_K, p.hidden, p.q_out, 0, p.hidden, p.q_row0, p.q_rows),
        "gate_up": np.concatenate([g, u]),
        "down": shard_bytes(full["down"], GGML_Q6_K, p.hidden, p.n_ff, 0, p.hidden, p.ff_row0, p.ff_rows),
    }
