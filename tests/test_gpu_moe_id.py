"""The mixture-of-experts indexed products (crates/ferric-tensor/src/dtype.rs:1620-1677) through the C ABI against the
oracle's restatement: selected-expert gate|up + SwiGLU, and the selected experts' down projections with the router's
weighted sum fused.  Bar: 1e-3 relative + 1e-4 absolute, element-wise."""
import numpy as np
import pytest
import torch

from ferric_b200 import synth
from oracle import oracle as O
from test_gpu_parity import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F():
    import ferric_b200
    return ferric_b200


@pytest.fixture(scope="module")
def ctx(F):
    c = F.Context(0)
    yield c
    c.close()


def router(rng, t, k, n_expert):
    """[t, 2k]: k weights summing to one, then k distinct expert indices as f32 (Tensor::moe_topk's output form)."""
    selw = np.empty((t, 2 * k), dtype=np.float32)
    for i in range(t):
        w = rng.uniform(0.1, 1.0, k).astype(np.float32)
        selw[i, :k] = w / w.sum()
        selw[i, k:] = rng.choice(n_expert, size=k, replace=False).astype(np.float32)
    return selw


@pytest.mark.parametrize("ty", [12, 13, 14])
@pytest.mark.parametrize("t,k,n_expert,eff,cols", [(1, 8, 16, 64, 512), (3, 2, 5, 48, 256), (5, 4, 8, 128, 768)])
def test_selected_expert_gate_up_swiglu(F, ctx, ty, t, k, n_expert, eff, cols):
    rng = np.random.default_rng(t * 100 + k)
    raw = synth.matrix(ty, n_expert * 2 * eff, cols, seed=ty + t)
    x = synth.activations(t, cols, seed=3)
    selw = router(rng, t, k, n_expert)
    qm = F.QMatrix.from_bytes(ctx, raw, ty, n_expert * 2 * eff, cols)
    got = qm.matmul_swiglu_id(torch.from_numpy(x).cuda(), torch.from_numpy(selw).cuda(), k, eff).cpu().numpy()
    ref = O.matmul_q_swiglu_id(raw, ty, n_expert, eff, cols, x, selw, k)
    assert got.shape == (t, k, eff)
    assert_close(got, ref, "swiglu_id")
    # every (token, slot) equals the plain fused product on that expert's own rows, bit for bit
    vals, bb = synth.BLOCK[ty]
    rb = cols // vals * bb
    e = int(selw[t - 1, k + k - 1])
    one = F.QMatrix.from_bytes(ctx, raw[e * 2 * eff * rb:(e + 1) * 2 * eff * rb], ty, 2 * eff, cols)
    alone = one.try_matmul_swiglu(torch.from_numpy(x[t - 1:t]).cuda()).cpu().numpy()[0]
    assert np.array_equal(got[t - 1, k - 1], alone)
    one.close()
    qm.close()


@pytest.mark.parametrize("ty", [12, 14])
@pytest.mark.parametrize("t,k,n_expert,out_pe,cols", [(1, 8, 16, 256, 512), (4, 3, 6, 80, 256), (2, 1, 3, 512, 1024)])
def test_selected_expert_down_with_weighted_sum(F, ctx, ty, t, k, n_expert, out_pe, cols):
    rng = np.random.default_rng(t * 10 + k)
    raw = synth.matrix(ty, n_expert * out_pe, cols, seed=ty + k)
    x = rng.standard_normal((t, k, cols)).astype(np.float32)
    selw = router(rng, t, k, n_expert)
    qm = F.QMatrix.from_bytes(ctx, raw, ty, n_expert * out_pe, cols)
    got = qm.matmul_id_wsum(torch.from_numpy(x).cuda(), torch.from_numpy(selw).cuda(), out_pe).cpu().numpy()
    ref = O.matmul_q_id_wsum(raw, ty, n_expert, out_pe, cols, x, selw)
    assert got.shape == (t, out_pe)
    assert_close(got, ref, "id_wsum")
    if t == 1:                                                     # the reference's 2-D [k, in] form means one token
        got2 = qm.matmul_id_wsum(torch.from_numpy(x[0]).cuda(), torch.from_numpy(selw).cuda(), out_pe).cpu().numpy()
        assert np.array_equal(got, got2)
    qm.close()


def test_indexed_product_argument_errors(F, ctx):
    qm = F.QMatrix.from_bytes(ctx, synth.matrix(12, 4 * 64, 256, seed=1), 12, 4 * 64, 256)
    q8 = F.QMatrix.from_bytes(ctx, synth.matrix(8, 64, 256, seed=2), 8, 64, 256)
    x = torch.zeros((2, 256), device="cuda")
    sel = torch.zeros((2, 4), device="cuda")
    for bad, status in ((lambda: qm.matmul_swiglu_id(x, torch.zeros((2, 18), device="cuda"), 9, 32), 3),       # k > 8
                        (lambda: qm.matmul_swiglu_id(x, sel, 2, 24), 3),                                          # eff not a multiple of 16
                        (lambda: qm.matmul_swiglu_id(x, sel, 2, 48), 3),                                          # rows are not whole experts
                        (lambda: qm.matmul_swiglu_id(torch.zeros((2, 512), device="cuda"), sel, 2, 32), 3),       # inner dim
                        (lambda: q8.matmul_swiglu_id(x, sel, 2, 32), 2),
                        (lambda: qm.matmul_id_wsum(torch.zeros((2, 2, 256), device="cuda"), sel, 40), 3)):
        with pytest.raises(F.FerricError) as e:
            bad()
        assert e.value.status == status
    # an index outside the stack gives zeros, never a read outside the matrix
    sel_bad = torch.tensor([[0.5, 0.5, 1.0, 99.0], [0.5, 0.5, -3.0, 2.0]], device="cuda")
    y = qm.matmul_swiglu_id(torch.ones((2, 256), device="cuda"), sel_bad, 2, 32)
    assert torch.isfinite(y).all() and (y[0, 1] == 0).all() and (y[1, 0] == 0).all() and (y[0, 0] != 0).any()
    qm.close()
    q8.close()
