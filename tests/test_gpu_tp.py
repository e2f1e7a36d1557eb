"""Tensor-parallel decode stack on two GPUs: NCCL all-reduce and the library's own peer-memory
exchanges (signalled buffers read by the peers; values pushed by the product's epilogue) against the
unsharded CPU oracle.  Needs 2 GPUs (skipped otherwise); ranks are separate processes, one per GPU,
NVLS off.  The pushed exchange also runs with a group of one rank, which needs one GPU only."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_stack_matches_unsharded_oracle(tmp_path):
    import test_tp_gloo as T
    import tp_worker as W
    from ferric_b200 import synth
    from ferric_b200.stack import TPPlan, layer_shards

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    out = str(tmp_path / "tp2.npz")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), str(r), "2", str(port), out])
             for r in range(2)]
    for p in procs:
        assert p.wait(timeout=300) == 0
    got = np.load(out)
    T.HID, T.NFF, T.QOUT, T.KV = W.HID, W.NFF, W.QOUT, W.KV
    plan1 = TPPlan.make(1, 0, W.HID, W.NFF, W.QOUT, W.KV)
    h = synth.activations(W.B, W.HID, seed=5)
    for l in range(W.LAYERS):
        h = T.layer_forward(plan1, layer_shards(plan1, T.full_layer(100 + 10 * l)), h, lambda a: None)
    tol = 1e-4 + 1e-3 * np.abs(h).max()
    assert np.abs(got["nccl"] - h).max() <= tol
    assert np.abs(got["fused"] - h).max() <= tol
    assert np.array_equal(got["fused"], got["fused_replay"])       # graph replay == eager
    assert np.array_equal(got["nccl"], got["nccl_replay"])
    wide = np.load(out + ".wide.npz")
    hw = synth.activations(W.WIDE_B, W.HID, seed=6)
    for l in range(W.LAYERS):
        hw = T.layer_forward(plan1, layer_shards(plan1, T.full_layer(100 + 10 * l)), hw, lambda a: None)
    tolw = 1e-4 + 1e-3 * np.abs(hw).max()
    assert np.abs(wide["nccl"] - hw).max() <= tolw and np.abs(wide["wide"] - hw).max() <= tolw
    assert np.array_equal(wide["wide"], wide["wide_replay"])
    assert np.abs(got["push"] - h).max() <= tol
    assert np.array_equal(got["push"], got["push_replay"])
    assert np.array_equal(got["push"], got["fused"])               # same partials, same rank-order sum


@pytest.mark.parametrize("cluster", [0, 2, 4, 8])
@pytest.mark.parametrize("m", [1, 2, 5, 8])
def test_pushed_exchange_with_one_rank(m, cluster, monkeypatch):
    """A group of one rank pushes to itself: matmul_push + the pushed add+norm+prepare must equal the plain matmul
    followed by add+norm+prepare bit for bit, for both kinds, with one kind used several times running (the parity
    double-buffer) and with both formats of the row-parallel products.  `cluster`: CTAs sharing one consumer tile
    (0 = the library's choice, which is one CTA for a single rank)."""
    import ferric_b200 as F
    from ferric_b200 import synth

    if cluster:
        monkeypatch.setenv("FERRIC_CUDA_PUSH_CLUSTER", str(cluster))
    ctx = F.Context(0)
    hid, kshard = 1536, 768
    grp = F.TPGroup(ctx, 0, 1, m, hid)
    grp.connect([grp.export()])
    nxt = F.QMatrix.from_bytes(ctx, synth.matrix(12, 64, hid, seed=1), 12, 64, hid)
    rng = np.random.default_rng(m)
    for ty, kinds in ((12, (0, 0, 0, 1)), (14, (1, 0, 1, 1, 1))):
        w = F.QMatrix.from_bytes(ctx, synth.matrix(ty, hid, kshard, seed=ty), ty, hid, kshard)
        for i, kind in enumerate(kinds):
            x = torch.from_numpy(synth.activations(m, kshard, seed=10 * ty + i)).cuda()
            a = torch.from_numpy(rng.standard_normal((m, hid)).astype(np.float32)).cuda()
            wn = torch.from_numpy(rng.uniform(0.5, 1.5, hid).astype(np.float32)).cuda()
            s1, n1 = torch.empty_like(a), torch.empty_like(a)
            mm = nxt.add_rmsnorm_prepare(a, w.matmul(x), wn, 1e-6, sum_out=s1, norm_out=n1)
            y1 = nxt.matmul_prepared(mm).clone()
            s2, n2 = torch.empty_like(a), torch.empty_like(a)
            grp.matmul_push(kind, w, x)
            grp.add_rmsnorm_prepare(kind, nxt, a, wn, 1e-6, sum_out=s2, norm_out=n2, pushed=True)
            y2 = nxt.matmul_prepared(mm)
            grp.check()
            # the cluster adds the per-super-block sums of squares in the order one CTA does: the same bits
            assert torch.equal(s1, s2) and torch.equal(n1, n2) and torch.equal(y1, y2)
        w.close()
    with pytest.raises(F.FerricError):
        grp.add_rmsnorm_prepare(0, nxt, a, None, 1e-6, pushed=True)       # the pushed form needs sum_out
    nxt.close()
    grp.close()
    ctx.close()


@pytest.mark.parametrize("world,m", [(2, 1), (3, 2), (4, 1), (8, 1), (8, 4)])
def test_pushed_exchange_many_ranks_in_one_process(world, m):
    """`world` ranks as groups of this process on one GPU (connected by address, not by IPC handle).  All ranks push,
    the device is synchronised, then all ranks consume: no kernel ever waits for one that has not run.  Every rank
    must form the same sum -- the partial products added in rank order -- and the same norm, bit for bit, twice over
    (both parities of the receive regions)."""
    import ferric_b200 as F
    from ferric_b200 import synth

    hid, kshard = 2048, 256
    ctxs = [F.Context(0) for _ in range(world)]
    grps = [F.TPGroup(ctxs[r], r, world, m, hid) for r in range(world)]
    F.TPGroup.connect_local(grps)
    ws = [F.QMatrix.from_bytes(ctxs[r], synth.matrix(12 if r % 2 == 0 else 14, hid, kshard, seed=r), 12 if r % 2 == 0 else 14, hid, kshard)
          for r in range(world)]
    nxt = [F.QMatrix.from_bytes(ctxs[r], synth.matrix(12, 64, hid, seed=99), 12, 64, hid) for r in range(world)]
    rng = np.random.default_rng(world * 10 + m)
    wn = torch.from_numpy(rng.uniform(0.5, 1.5, hid).astype(np.float32)).cuda()
    for it in range(3):
        kind = it & 1 if it < 2 else 1
        xs = [torch.from_numpy(synth.activations(m, kshard, seed=100 * it + r)).cuda() for r in range(world)]
        a = torch.from_numpy(rng.standard_normal((m, hid)).astype(np.float32)).cuda()
        total = ws[0].matmul(xs[0]).clone()
        for r in range(1, world):
            total += ws[r].matmul(xs[r])
        s_ref, n_ref = torch.empty_like(a), torch.empty_like(a)
        mm = nxt[0].add_rmsnorm_prepare(a, total, wn, 1e-6, sum_out=s_ref, norm_out=n_ref)
        y_ref = nxt[0].matmul_prepared(mm).clone()
        torch.cuda.synchronize()
        for r in range(world):
            grps[r].matmul_push(kind, ws[r], xs[r])
        torch.cuda.synchronize()
        for r in range(world):
            s, n = torch.empty_like(a), torch.empty_like(a)
            grps[r].add_rmsnorm_prepare(kind, nxt[r], a, wn, 1e-6, sum_out=s, norm_out=n, pushed=True)
            y = nxt[r].matmul_prepared(mm)
            grps[r].check()
            assert torch.equal(s, s_ref) and torch.equal(n, n_ref) and torch.equal(y, y_ref), (it, r)
    for o in ws + nxt + grps + ctxs:
        o.close()


@pytest.mark.parametrize("world,cap_rows,rows,d", [(1, 9, 9, 1024), (2, 16, 16, 1024), (3, 16, 10, 512), (8, 64, 64, 1536), (8, 8, 5, 260),
                                                   (4, 64, 3, 5120)])
def test_two_step_allreduce_many_ranks_in_one_process(world, cap_rows, rows, d):
    """The all-reduce for many activation rows (scatter to slice owners, reduce, store to all, add + RMSNorm) with
    `world` ranks as groups of this process on one GPU.  The three steps run as phases with a device synchronise
    between them, so no kernel waits for one that has not been launched.  Every rank must end with a + (the partials
    added in rank order), bit for bit, three exchanges running (both kinds, both parities); rows below the group's
    capacity leave some ranks without a slice."""
    import ferric_b200 as F

    ctxs = [F.Context(0) for _ in range(world)]
    grps = [F.TPGroup(ctxs[r], r, world, cap_rows, d) for r in range(world)]
    F.TPGroup.connect_local(grps)
    gen = torch.Generator(device="cuda").manual_seed(world * 100 + rows)
    wn = torch.rand(d, device="cuda", generator=gen) + 0.5
    for it, kind in enumerate((0, 1, 1)):
        parts = [torch.randn(rows, d, device="cuda", generator=gen) * (r + 1) for r in range(world)]
        a = torch.randn(rows, d, device="cuda", generator=gen)
        total = parts[0].clone()
        for r in range(1, world):
            total += parts[r]
        s_ref, n_ref = torch.empty_like(a), torch.empty_like(a)
        ctxs[0].add_rmsnorm(a, total, wn, 1e-6, sum_out=s_ref, norm_out=n_ref)
        outs = [(torch.empty_like(a), torch.empty_like(a)) for _ in range(world)]
        for step in (1, 2, 4):
            torch.cuda.synchronize()
            for r in range(world):
                grps[r].allreduce_add_rmsnorm(kind, parts[r], a, wn, 1e-6, sum_out=outs[r][0], norm_out=outs[r][1], steps=step)
        for r in range(world):
            grps[r].check()
            assert torch.equal(outs[r][0], s_ref), (it, r)
            assert torch.allclose(outs[r][1], n_ref, rtol=2e-6, atol=1e-7), (it, r)
            assert torch.equal(outs[r][1], outs[0][1])         # the same bits on every rank
    for o in grps + ctxs:
        o.close()
