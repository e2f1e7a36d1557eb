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


def elementwise_ok(got, ref, exact):
    """The path's bar, element by element, on the stack's result -- the RMS-normalised residual stream, whose values
    are of order one like the activations the bar is stated for: |got - ref| <= 1e-4 + 1e-3 |ref|, where the oracle's own
    f32 rounding (its distance from the same layers evaluated in float64) is not charged to the kernels.  Returns the
    worst ratio of error to bar."""
    def norm(h):
        h = h.astype(np.float64)
        return h / np.sqrt((h * h).mean(axis=-1, keepdims=True) + 1e-6)

    g, r, e = norm(got), norm(ref), norm(exact)
    tol = 1e-4 + 1e-3 * np.abs(r) + np.abs(r - e)
    return float((np.abs(g - r) / tol).max())


@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_gpu_stack_matches_unsharded_oracle(tmp_path, world):
    """`world` GPUs, one process each: every exchange form against the unsharded layers on the CPU oracle."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import test_tp_gloo as T
    import tp_worker as W
    from ferric_b200 import synth
    from ferric_b200.stack import TPPlan, layer_shards

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    out = str(tmp_path / f"tp{world}.npz")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), str(r), str(world), str(port), out])
             for r in range(world)]
    for p in procs:
        assert p.wait(timeout=600) == 0
    got = np.load(out)
    HID, NFF, QOUT, KV = W.dims(world)
    T.HID, T.NFF, T.QOUT, T.KV = HID, NFF, QOUT, KV
    plan1 = TPPlan.make(1, 0, HID, NFF, QOUT, KV)

    def reference(h):
        h64 = h.astype(np.float64)
        for l in range(W.LAYERS):
            sh = layer_shards(plan1, T.full_layer(100 + 10 * l))
            h = T.layer_forward(plan1, sh, h, lambda a: None)
            h64 = T.layer_forward_f64(plan1, sh, h64)
        return h, h64

    h, h64 = reference(synth.activations(W.B, HID, seed=5))
    for mode in ("nccl", "fused", "push", "chain"):
        assert np.isfinite(got[mode]).all(), mode
        assert elementwise_ok(got[mode], h, h64) <= 1.0, (mode, elementwise_ok(got[mode], h, h64))
        assert np.array_equal(got[mode], got[mode + "_replay"]), mode      # graph replay == eager
    assert np.array_equal(got["push"], got["fused"])               # same partials, same rank-order sum
    wide = np.load(out + ".wide.npz")
    hw, hw64 = reference(synth.activations(W.WIDE_B, HID, seed=6))
    assert elementwise_ok(wide["nccl"], hw, hw64) <= 1.0 and elementwise_ok(wide["wide"], hw, hw64) <= 1.0
    assert np.array_equal(wide["wide"], wide["wide_replay"])


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


@pytest.mark.parametrize("world,ty,rows,cols_per_rank,m", [(2, 12, 512, 1024, 24), (4, 14, 640, 1024, 64), (3, 12, 19200, 256, 16),
                                                          (2, 12, 512, 1024, 4)])
def test_product_scatters_its_own_result_into_the_two_step_allreduce(world, ty, rows, cols_per_rank, m):
    """`matmul_scatter`: each rank's row-parallel product goes straight into step 1 of the all-reduce -- by the product's own
    finish kernel where its K range is cut across CTAs (few row tiles), by the scatter kernel after it otherwise (one K
    piece: 19200 rows; or the GEMV path: 4 activation rows).  Ranks are groups of this process on one GPU, the steps run as
    phases.  The result must equal add_rmsnorm(a, sum over ranks of the plain products), the sum bit for bit."""
    import ferric_b200 as F
    from ferric_b200 import synth

    ctxs = [F.Context(0) for _ in range(world)]
    grps = [F.TPGroup(ctxs[r], r, world, m, rows) for r in range(world)]
    F.TPGroup.connect_local(grps)
    gen = torch.Generator(device="cuda").manual_seed(world * 7 + m)
    qms = [F.QMatrix.from_bytes(ctxs[r], synth.matrix(ty, rows, cols_per_rank, seed=50 + r), ty, rows, cols_per_rank) for r in range(world)]
    for it, kind in enumerate((0, 1, 1)):
        xs = [torch.randn(m, cols_per_rank, device="cuda", generator=gen) for _ in range(world)]
        a = torch.randn(m, rows, device="cuda", generator=gen)
        total = qms[0].matmul(xs[0]).clone()
        for r in range(1, world):
            total += qms[r].matmul(xs[r])
        s_ref, n_ref = torch.empty_like(a), torch.empty_like(a)
        ctxs[0].add_rmsnorm(a, total, None, 1e-6, sum_out=s_ref, norm_out=n_ref)
        outs = [(torch.empty_like(a), torch.empty_like(a)) for _ in range(world)]
        torch.cuda.synchronize()
        fused = [grps[r].matmul_scatter(kind, qms[r], xs[r]) for r in range(world)]
        assert all(f == (m >= 9 and rows < 19200) for f in fused), fused
        for step in (2, 4):
            torch.cuda.synchronize()
            for r in range(world):
                grps[r].allreduce_add_rmsnorm(kind, a, a, None, 1e-6, sum_out=outs[r][0], norm_out=outs[r][1], steps=step)
        for r in range(world):
            grps[r].check()
            assert torch.equal(outs[r][0], s_ref), (it, r)
            assert torch.allclose(outs[r][1], n_ref, rtol=2e-6, atol=1e-7), (it, r)
    for o in qms + grps + ctxs:
        o.close()


# ---------------------------------------------------------------------------------- a peer that never arrives
def _two_local_ranks(F, m, hid):
    ctxs = [F.Context(0) for _ in range(2)]
    grps = [F.TPGroup(ctxs[r], r, 2, m, hid) for r in range(2)]
    F.TPGroup.connect_local(grps)
    return ctxs, grps


def test_a_missing_peer_runs_out_the_pushed_wait_and_the_group_recovers(monkeypatch):
    """Rank 1 never pushes.  Rank 0's consumer polls its own memory a bounded number of rounds (set small here through
    FERRIC_CUDA_PEER_WAIT_SPINS), gives up, and says so through ferric_cuda_tp_status; nothing hangs or faults.  A later
    consumer of the group does not wait again.  After both ranks reset, a full exchange is correct."""
    import ferric_b200 as F
    from ferric_b200 import synth

    monkeypatch.setenv("FERRIC_CUDA_PEER_WAIT_SPINS", "2000")
    m, hid, k = 2, 1024, 256
    ctxs, grps = _two_local_ranks(F, m, hid)
    ws = [F.QMatrix.from_bytes(ctxs[r], synth.matrix(12, hid, k, seed=r), 12, hid, k) for r in range(2)]
    nxt = [F.QMatrix.from_bytes(ctxs[r], synth.matrix(12, 64, hid, seed=9), 12, 64, hid) for r in range(2)]
    xs = [torch.from_numpy(synth.activations(m, k, seed=20 + r)).cuda() for r in range(2)]
    a = torch.randn((m, hid), device="cuda")
    s = torch.empty_like(a)
    grps[0].matmul_push(0, ws[0], xs[0])                          # only rank 0 pushes
    grps[0].add_rmsnorm_prepare(0, nxt[0], a, None, 1e-6, sum_out=s, pushed=True)
    with pytest.raises(F.FerricError) as e:
        grps[0].check()                                           # returns: the wait ran out
    assert e.value.status == 7
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    grps[0].matmul_push(1, ws[0], xs[0])
    t0.record()
    grps[0].add_rmsnorm_prepare(1, nxt[0], a, None, 1e-6, sum_out=s, pushed=True)      # status is set: no second wait
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 50.0
    # the chained form of the same exchange: product, poll and job in one launch
    ctxs[0].chain_reserve(max(ws[0].scratch_bytes(m), nxt[0].scratch_bytes(m)))
    for g in grps:
        g.reset()
    ws[0].prepare(xs[0])
    h = a.clone()
    grps[0].chain_matmul(0, ws[0], m, 0, nxt[0], h)
    with pytest.raises(F.FerricError) as e:
        grps[0].check()
    assert e.value.status == 7
    for g in grps:
        g.reset()
    # both ranks push, the device is synchronised, both consume: correct again
    total = ws[0].matmul(xs[0]) + ws[1].matmul(xs[1])
    s_ref = torch.empty_like(a)
    nxt[0].add_rmsnorm_prepare(a, total, None, 1e-6, sum_out=s_ref)
    for r in range(2):
        grps[r].matmul_push(0, ws[r], xs[r])
    torch.cuda.synchronize()
    for r in range(2):
        s_r = torch.empty_like(a)
        grps[r].add_rmsnorm_prepare(0, nxt[r], a, None, 1e-6, sum_out=s_r, pushed=True)
        grps[r].check()
        assert torch.equal(s_r, s_ref)
    for o in ws + nxt + grps + ctxs:
        o.close()


def test_a_missing_peer_runs_out_the_two_step_allreduce_wait(monkeypatch):
    """The same for the all-reduce of many rows: rank 1's scatter is left out, so rank 0's reduce step finds only its
    own copy of its slice, gives up after the bound and reports it; after a reset the exchange works."""
    import ferric_b200 as F

    monkeypatch.setenv("FERRIC_CUDA_PEER_WAIT_SPINS", "2000")
    rows, d = 12, 1024
    ctxs, grps = _two_local_ranks(F, rows, d)
    gen = torch.Generator(device="cuda").manual_seed(3)
    parts = [torch.randn(rows, d, device="cuda", generator=gen) for _ in range(2)]
    a = torch.randn(rows, d, device="cuda", generator=gen)
    outs = [(torch.empty_like(a), torch.empty_like(a)) for _ in range(2)]
    grps[0].allreduce_add_rmsnorm(0, parts[0], a, None, 1e-6, sum_out=outs[0][0], norm_out=outs[0][1], steps=1)
    torch.cuda.synchronize()
    grps[0].allreduce_add_rmsnorm(0, parts[0], a, None, 1e-6, sum_out=outs[0][0], norm_out=outs[0][1], steps=2)
    with pytest.raises(F.FerricError) as e:
        grps[0].check()
    assert e.value.status == 7
    for g in grps:
        g.reset()
    s_ref, n_ref = ctxs[0].add_rmsnorm(a, parts[0] + parts[1], None, 1e-6)
    for step in (1, 2, 4):
        torch.cuda.synchronize()
        for r in range(2):
            grps[r].allreduce_add_rmsnorm(0, parts[r], a, None, 1e-6, sum_out=outs[r][0], norm_out=outs[r][1], steps=step)
    for r in range(2):
        grps[r].check()
        assert torch.equal(outs[r][0], s_ref)
    for o in grps + ctxs:
        o.close()


def test_signalled_exchange_refuses_the_same_kind_twice():
    """The signalled (pull) form has one buffer per kind and is safe only while kinds alternate."""
    import ferric_b200 as F

    ctxs, grps = _two_local_ranks(F, 1, 256)
    grps[0].signal(0)
    with pytest.raises(F.FerricError) as e:
        grps[0].signal(0)
    assert e.value.status == 1 and "alternate" in str(e.value)
    grps[0].signal(1)
    grps[0].signal(0)
    for o in grps + ctxs:
        o.close()
