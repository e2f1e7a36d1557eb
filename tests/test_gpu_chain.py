"""Chained decoder-layer products (``ferric_cuda_chain_matmul``): one launch per matrix, with the activation
preparation, the residual add and the RMSNorm statistics done by the products' own launches.

What must hold:
* a PREPARE link's fragments are the ones ``prepare_x`` would have written, so the next product is bit-identical
  to the unchained pair;
* a RESIDUAL link updates the residual stream with the same single f32 add as ``add_rmsnorm`` (bit-exact) and the next
  product, which applies 1/rms to its result instead of to its input, stays within f32 rounding of the unchained
  sequence and within the path's tolerance (1e-3 relative + 1e-4 absolute) of the CPU oracle;
* the whole stack, chained, equals the stack run kernel by kernel.
All calls go through the C ABI.
"""
import numpy as np
import pytest
import torch

from ferric_b200 import synth
from oracle import oracle as O
from test_gpu_parity import assert_close, exact_product

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F():
    import ferric_b200
    return ferric_b200


@pytest.fixture()
def ctx(F):
    c = F.Context(0)
    yield c
    c.close()


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("m", [1, 2, 3, 4])
@pytest.mark.parametrize("ty,ty_next", [(12, 12), (12, 14), (14, 12), (13, 14)])
def test_prepare_link_is_the_unchained_pair_bit_for_bit(F, ctx, ty, ty_next, m):
    rows, cols, cols_next, rows_next = 800, 512, 768, 96       # the next product reads the first 768 of 800 columns
    w = F.QMatrix.from_bytes(ctx, synth.matrix(ty, rows, cols, seed=1), ty, rows, cols)
    nx = F.QMatrix.from_bytes(ctx, synth.matrix(ty_next, rows_next, cols_next, seed=2), ty_next, rows_next, cols_next)
    x = cuda(synth.activations(m, cols, seed=3 + m))
    y_ref = w.matmul(x)
    z_ref = nx.matmul(y_ref[:, :cols_next])
    ctx.chain_reserve(max(w.scratch_bytes(m), nx.scratch_bytes(m)))
    for _ in range(2):                                          # twice: the block tickets must be back at zero
        mm = w.prepare(x)                                       # slot 0
        y = torch.full((m, rows), float("nan"), device="cuda")
        z = torch.full((m, rows_next), float("nan"), device="cuda")
        w.chain_matmul(mm, y, in_slot=0, next=1, next_qm=nx)
        nx.chain_matmul(mm, z, in_slot=1)
        assert torch.equal(y, y_ref) and torch.equal(z, z_ref)
    w.close()
    nx.close()


@pytest.mark.parametrize("m", [1, 3, 4])
def test_swiglu_prepare_link(F, ctx, m):
    n_ff, cols = 512, 768
    gu = F.QMatrix.from_bytes(ctx, synth.matrix(12, 2 * n_ff, cols, seed=5), 12, 2 * n_ff, cols)
    dn = F.QMatrix.from_bytes(ctx, synth.matrix(14, 160, n_ff, seed=6), 14, 160, n_ff)
    x = cuda(synth.activations(m, cols, seed=7))
    f_ref = gu.try_matmul_swiglu(x)
    d_ref = dn.matmul(f_ref)
    ctx.chain_reserve(max(gu.scratch_bytes(m), dn.scratch_bytes(m)))
    mm = gu.prepare(x)
    f, d = torch.empty_like(f_ref), torch.empty_like(d_ref)
    gu.chain_matmul(mm, f, swiglu=True, in_slot=0, next=1, next_qm=dn)
    dn.chain_matmul(mm, d, in_slot=1)
    assert torch.equal(f, f_ref) and torch.equal(d, d_ref)
    gu.close()
    dn.close()


@pytest.mark.parametrize("m", [1, 2, 3, 4])
@pytest.mark.parametrize("ty,ty_next,weighted", [(12, 12, True), (14, 12, False), (12, 14, True)])
def test_residual_link_against_add_rmsnorm_and_the_oracle(F, ctx, ty, ty_next, weighted, m):
    hid, k, rows_next = 1280, 512, 208
    raw, raw_next = synth.matrix(ty, hid, k, seed=11), synth.matrix(ty_next, rows_next, hid, seed=12)
    w = F.QMatrix.from_bytes(ctx, raw, ty, hid, k)
    nx = F.QMatrix.from_bytes(ctx, raw_next, ty_next, rows_next, hid)
    rng = np.random.default_rng(m)
    x = synth.activations(m, k, seed=13)
    h0 = rng.standard_normal((m, hid)).astype(np.float32) * np.float32(3)
    wn = rng.uniform(0.5, 1.5, hid).astype(np.float32) if weighted else None
    # unchained: product, add + rmsnorm + prepare, product
    o = w.matmul(cuda(x))
    s_ref, n_ref = torch.empty_like(o), torch.empty_like(o)
    mm = nx.add_rmsnorm_prepare(cuda(h0), o, cuda(wn) if weighted else None, 1e-6, sum_out=s_ref, norm_out=n_ref)
    z_ref = nx.matmul_prepared(mm).clone()
    # chained
    ctx.chain_reserve(max(w.scratch_bytes(m), nx.scratch_bytes(m)))
    w.prepare(cuda(x))
    h = cuda(h0)
    o2 = torch.empty_like(o)
    z = torch.empty_like(z_ref)
    w.chain_matmul(m, o2, in_slot=0, next=2, next_qm=nx, h=h, norm_weight=cuda(wn) if weighted else None)
    nx.chain_matmul(m, z, in_slot=1, in_rms=True, eps=1e-6)
    assert torch.equal(o2, o) and torch.equal(h, s_ref)                       # the sum is one f32 add per element
    zr, zc = z_ref.cpu().numpy(), z.cpu().numpy()
    assert np.abs(zc - zr).max() <= 2e-6 * np.abs(zr).max()                   # 1/rms after the product: f32 rounding only
    # against the oracle: the reference's own sequence on the same bytes
    o_ref = O.matmul_q(raw, ty, hid, k, x)
    s_o, n_o = O.add_rmsnorm(h0, o_ref, wn, 1e-6)
    assert_close(zc, O.matmul_q(raw_next, ty_next, rows_next, hid, n_o), "chained residual link",
                 exact_product(raw_next, ty_next, rows_next, hid, n_o))
    w.close()
    nx.close()


@pytest.mark.parametrize("batch", [1, 2, 3, 4])
def test_chained_stack_equals_the_stack_kernel_by_kernel(F, ctx, batch):
    from ferric_b200.stack import DecodeStack, TPPlan
    plan = TPPlan.make(1, 0, hidden=768, n_ff=1024, q_out=512, kv_out=256)
    stacks = [DecodeStack(ctx, plan, n_layers=3, batch=batch, chain=c) for c in (False, True)]
    assert not stacks[0].chain and stacks[1].chain
    raws = []
    for l in range(3):
        mats = [(12, plan.q_rows + 2 * plan.kv_rows, 768), (12, 768, plan.q_rows), (12, 2 * plan.ff_rows, 768), (14, 768, plan.ff_rows)]
        raw = [synth.matrix(ty, r, c, seed=200 + 10 * l + i) for i, (ty, r, c) in enumerate(mats)]
        raws.append(list(zip(mats, raw)))
        qs = [F.QMatrix.from_bytes(ctx, rw, ty, r, c) for (ty, r, c), rw in zip(mats, raw)]
        for st in stacks:
            st.add_layer(*qs)
    h0 = np.random.default_rng(batch).standard_normal((batch, 768)).astype(np.float32)
    outs = []
    for st in stacks:
        st.reserve()
        st.h.copy_(cuda(h0))
        outs.append((st.step().cpu().numpy().copy(), st.xn.cpu().numpy().copy(), st.launches_per_step))
    (h_a, xn_a, launches_a), (h_b, xn_b, launches_b) = outs
    assert launches_b == 4 * 3 + 2 and launches_a == 8 * 3 + 1           # one launch per matrix (+ entry and exit norm)
    assert np.abs(h_a - h_b).max() <= 1e-5 * np.abs(h_a).max()
    assert np.abs(xn_a - xn_b).max() <= 1e-5 * np.abs(xn_a).max()
    # the oracle, layer by layer
    h = h0.copy()
    xn = O.add_rmsnorm(h, None, None, 1e-6)[1]
    for (q, o, gu, dn) in raws:
        qkv = O.matmul_q(q[1], *q[0], xn)
        oo = O.matmul_q(o[1], *o[0], np.ascontiguousarray(qkv[:, :plan.q_rows]))
        h, xn = O.add_rmsnorm(h, oo, None, 1e-6)
        f = O.swiglu(O.matmul_q(gu[1], *gu[0], xn), plan.ff_rows)
        h, xn = O.add_rmsnorm(h, O.matmul_q(dn[1], *dn[0], f), None, 1e-6)
    assert np.abs(h_b - h).max() <= 1e-4 + 1e-3 * np.abs(h).max()
    st = stacks[1]
    st.capture()
    st.h.copy_(cuda(h0))
    assert np.array_equal(st.run().cpu().numpy(), h_b)                    # graph replay == eager launches, bit for bit
    stacks[0].layers = []
    st.close()


@pytest.mark.parametrize("m", [1, 2, 4])
def test_pushed_residual_link_with_one_rank(F, ctx, m):
    """A group of one rank pushes to itself: product, exchange, residual add and preparation in ONE launch must
    equal the local residual link bit for bit -- both kinds, one of them twice running (the receive regions'
    parity double-buffer), both formats."""
    hid, k, rows_next = 1536, 768, 64
    grp = F.TPGroup(ctx, 0, 1, m, hid)
    grp.connect([grp.export()])
    nx = F.QMatrix.from_bytes(ctx, synth.matrix(12, rows_next, hid, seed=21), 12, rows_next, hid)
    rng = np.random.default_rng(m)
    for ty, kinds in ((12, (0, 0, 1)), (14, (1, 0, 1, 1))):
        w = F.QMatrix.from_bytes(ctx, synth.matrix(ty, hid, k, seed=ty), ty, hid, k)
        ctx.chain_reserve(max(w.scratch_bytes(m), nx.scratch_bytes(m)))
        for i, kind in enumerate(kinds):
            x = cuda(synth.activations(m, k, seed=10 * ty + i))
            h0 = cuda(rng.standard_normal((m, hid)).astype(np.float32))
            wn = cuda(rng.uniform(0.5, 1.5, hid).astype(np.float32))
            w.prepare(x)
            h1, o1, z1 = h0.clone(), torch.empty((m, hid), device="cuda"), torch.empty((m, rows_next), device="cuda")
            w.chain_matmul(m, o1, in_slot=0, next=2, next_qm=nx, h=h1, norm_weight=wn)
            nx.chain_matmul(m, z1, in_slot=1, in_rms=True)
            w.prepare(x)
            h2, z2 = h0.clone(), torch.empty_like(z1)
            grp.chain_matmul(kind, w, m, 0, nx, h2, wn)
            nx.chain_matmul(m, z2, in_slot=1, in_rms=True)
            grp.check()
            assert torch.equal(h1, h2) and torch.equal(z1, z2), (ty, i)
        w.close()
    nx.close()
    grp.close()


def test_chain_argument_errors(F):
    ctx = F.Context(0)
    w = F.QMatrix.from_bytes(ctx, synth.matrix(12, 512, 256, seed=1), 12, 512, 256)
    nx = F.QMatrix.from_bytes(ctx, synth.matrix(12, 32, 512, seed=2), 12, 32, 512)
    wide = F.QMatrix.from_bytes(ctx, synth.matrix(12, 32, 1024, seed=3), 12, 32, 1024)
    q8 = F.QMatrix.from_bytes(ctx, synth.matrix(8, 32, 256, seed=4), 8, 32, 256)
    y = torch.empty((5, 512), device="cuda")
    with pytest.raises(F.FerricError) as e:                      # no slots reserved yet
        w.chain_matmul(1, y)
    assert e.value.status == 1
    ctx.chain_reserve(max(w.scratch_bytes(4), nx.scratch_bytes(4)))
    w.prepare(torch.zeros((1, 256), device="cuda"))
    with pytest.raises(F.FerricError) as e:                      # more rows than one GEMV pass
        w.chain_matmul(5, y)
    assert e.value.status == 3
    with pytest.raises(F.FerricError) as e:                      # the next product would read more columns than there are
        w.chain_matmul(1, y, next=1, next_qm=wide)
    assert e.value.status == 3
    with pytest.raises(F.FerricError) as e:                      # a residual link needs the residual stream
        w.chain_matmul(1, y, next=2, next_qm=nx)
    assert e.value.status == 1
    with pytest.raises(F.FerricError) as e:
        q8.chain_matmul(1, y)
    assert e.value.status == 6
    with pytest.raises(F.FerricError) as e:
        w.chain_matmul(1, y, in_slot=2)
    assert e.value.status == 1
    for q in (w, nx, wide, q8):
        q.close()
    ctx.close()
