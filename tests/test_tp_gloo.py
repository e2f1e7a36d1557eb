"""Tensor-parallel host logic on CPU: shard plan, byte slicing, and the all-reduce exchange over gloo.

Two ranks (world_size 2, gloo, 127.0.0.1) each take their shard of one small layer, compute their
partial products with the CPU oracle, all-reduce the f32 partial sums of the row-parallel matrices, and
must reproduce the unsharded layer.  The CUDA kernels are not involved (no GPU here); what is covered is
everything around them on the N > 1 path."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ferric_b200 import synth
from ferric_b200.stack import TPPlan, layer_shards, shard_bytes, split_blocks
from oracle import oracle as O

HID, NFF, QOUT, KV = 1024, 1536, 1024, 512


def full_layer(seed):
    shapes = {"q": (12, QOUT, HID), "k": (12, KV, HID), "v": (12, KV, HID), "o": (12, HID, QOUT),
              "gate": (12, NFF, HID), "up": (12, NFF, HID), "down": (14, HID, NFF)}
    return {n: synth.matrix(ty, r, c, seed + i) for i, (n, (ty, r, c)) in enumerate(shapes.items())}


def layer_forward(plan, sh, h, reduce):
    """One layer on one rank with oracle products; `reduce` sums partials across ranks in place."""
    xn = O.add_rmsnorm(h, None, None, 1e-6)[1]
    qkv = O.matmul_q(sh["qkv"], 12, plan.q_rows + 2 * plan.kv_rows, plan.hidden, xn)
    o = O.matmul_q(sh["o"], 12, plan.hidden, plan.q_rows, np.ascontiguousarray(qkv[:, :plan.q_rows]))
    reduce(o)
    h, xn = O.add_rmsnorm(h, o, None, 1e-6)
    gu = O.matmul_q(sh["gate_up"], 12, 2 * plan.ff_rows, plan.hidden, xn)
    f = O.swiglu(gu, plan.ff_rows)
    d = O.matmul_q(sh["down"], 14, plan.hidden, plan.ff_rows, f)
    reduce(d)
    return O.add_rmsnorm(h, d, None, 1e-6)[0]


def layer_forward_f64(plan, sh, h):
    """The same layer (unsharded) with the oracle-dequantised weights and float64 arithmetic throughout: what the f32
    oracle itself deviates from, so that a parity bar can leave the oracle's own rounding out."""
    def w64(raw, ty, rows, cols):
        return O.deq_raw(raw, rows * cols, ty).reshape(rows, cols).astype(np.float64)

    def norm(v):
        return v / np.sqrt((v * v).mean(axis=-1, keepdims=True) + 1e-6)

    xn = norm(h)
    qkv = xn @ w64(sh["qkv"], 12, plan.q_rows + 2 * plan.kv_rows, plan.hidden).T
    h = h + qkv[:, :plan.q_rows] @ w64(sh["o"], 12, plan.hidden, plan.q_rows).T
    gu = norm(h) @ w64(sh["gate_up"], 12, 2 * plan.ff_rows, plan.hidden).T
    g, u = gu[:, :plan.ff_rows], gu[:, plan.ff_rows:]
    f = g / (1.0 + np.exp(-g)) * u
    return h + f @ w64(sh["down"], 14, plan.hidden, plan.ff_rows).T


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    plan = TPPlan.make(world, rank, HID, NFF, QOUT, KV)
    sh = layer_shards(plan, full_layer(7))
    h = synth.activations(3, HID, seed=5)

    def reduce(a):
        t = torch.from_numpy(a)
        dist.all_reduce(t)          # f32 sum of the [B, hidden] partials, as the NCCL path does

    res = layer_forward(plan, sh, h, reduce)
    if rank == 0:
        np.save(out, res)
    dist.destroy_process_group()


def test_two_rank_layer_equals_unsharded(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    out = str(tmp_path / "tp2.npy")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    got = np.load(out)
    plan1 = TPPlan.make(1, 0, HID, NFF, QOUT, KV)
    ref = layer_forward(plan1, layer_shards(plan1, full_layer(7)), synth.activations(3, HID, seed=5), lambda a: None)
    assert np.abs(got - ref).max() <= 1e-4 + 1e-3 * np.abs(ref).max()


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_plan_partitions_the_27b_layer(world):
    plans = [TPPlan.make(world, r) for r in range(world)]
    assert sum(p.q_rows for p in plans) == 5120 and sum(p.kv_rows for p in plans) == 1024
    assert sum(p.ff_rows for p in plans) == 17408
    for a, b in zip(plans, plans[1:]):
        assert a.q_row0 + a.q_rows == b.q_row0 and a.ff_row0 + a.ff_rows == b.ff_row0 and a.kv_row0 + a.kv_rows == b.kv_row0
    assert all(p.q_rows % 256 == 0 and p.ff_rows % 256 == 0 for p in plans)       # K shards on super-block boundaries
    assert sum(p.weight_bytes_per_layer() for p in plans) == 208_773_120          # the config's bytes per layer
    if world == 8:
        assert [p.q_rows // 256 for p in plans] == [3, 3, 3, 3, 2, 2, 2, 2]
        assert [p.ff_rows // 256 for p in plans] == [9, 9, 9, 9, 8, 8, 8, 8]


def test_split_blocks_and_shard_bytes():
    assert split_blocks(20, 8) == [3, 3, 3, 3, 2, 2, 2, 2] and split_blocks(68, 4) == [17] * 4
    raw = synth.matrix(14, 6, 768, seed=2)
    full = O.deq_raw(raw, 6 * 768, 14).reshape(6, 768)
    part = shard_bytes(raw, 14, 6, 768, 2, 3, 256, 512)
    assert (O.deq_raw(part, 3 * 512, 14).reshape(3, 512) == full[2:5, 256:768]).all()
