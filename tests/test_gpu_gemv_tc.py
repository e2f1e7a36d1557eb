"""GPU parity of the batched decode product on the tensor cores (more than 8 activation rows).

The kernel multiplies the quantised weights' integers with the activations rounded to 22-bit integers per
(row, super-block), split into two 11-bit limbs, on the tensor cores and scales per super-block in f32 -- at least the
precision of an f32 product -- so the bar is the decode bar: 1e-3 relative + 1e-4 absolute against the oracle's
dequantise-then-dot product (with the exact float64 product beside it, see test_gpu_parity.assert_close).  Every case
also reads the kernel's give-up word: no bounded wait may run out.

Shapes walk the kernel's branches: the two tile widths (up to 32 / 64 activation rows), more than one
activation tile, ragged weight rows (rows not a multiple of 128 or of 16), a K split (few row tiles, many
super-blocks) with its finish kernel, the fused SwiGLU finish, Q4_K's min term on the tensor core, Q6_K's two operand
planes with scales over the whole int8 range, and activations spanning many binades (one scale per row and
super-block).
"""
import os

import numpy as np
import pytest
import torch

from ferric_b200 import synth
from oracle import oracle as O
from test_gpu_parity import assert_close, exact_product

pytestmark = pytest.mark.gpu
NCPU = os.cpu_count() or 1


@pytest.fixture(scope="module")
def F():
    import ferric_b200
    return ferric_b200


@pytest.fixture(scope="module")
def ctx(F):
    c = F.Context(0)
    yield c
    c.close()


@pytest.fixture(autouse=True)
def tensor_core_path_from_nine_rows(monkeypatch):
    """By default this kernel takes over from 9 (Q4_K) or 13 (Q6_K) activation rows; the tests here run both from 9."""
    monkeypatch.setenv("FERRIC_CUDA_GEMV_TC_MIN_M", "9")


def run(F, ctx, raw, ty, rows, cols, x, swiglu=False):
    qm = F.QMatrix.from_bytes(ctx, raw, ty, rows, cols)
    xd = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    y = qm.try_matmul_swiglu(xd) if swiglu else qm.matmul(xd)
    assert qm.gemm_status() == 0
    out = y.cpu().numpy()
    qm.close()
    return out


@pytest.mark.parametrize("ty,rows,cols,m", [
    (12, 128, 256, 9),        # one CTA, one super-block, narrow tile
    (12, 200, 1024, 16),      # ragged rows
    (12, 1000, 2048, 33),     # widest tile, ragged rows
    (12, 272, 512, 64),
    (12, 130, 768, 70),       # two activation tiles of the widest kind, the second nearly empty
    (12, 256, 512, 128),      # two full activation tiles
    (12, 144, 512, 200),      # four activation tiles, the last partly filled
    (12, 256, 5120, 17),      # few row tiles, 20 super-blocks: K split + finish kernel
    (13, 200, 1024, 16),      # Q5_K: the Q4_K kernel with the fifth bit, ragged rows
    (13, 272, 512, 64),       # Q5_K, widest tile
    (13, 256, 5120, 17),      # Q5_K with a K split
    (14, 128, 256, 24),       # Q6_K: two operand planes
    (14, 200, 768, 40),       # Q6_K, two activation tiles (its tile holds 32 rows)
    (14, 640, 4352, 64),      # Q6_K with a K split
])
def test_shapes(F, ctx, ty, rows, cols, m):
    raw = synth.matrix(ty, rows, cols, seed=rows + cols + m)
    x = synth.activations(m, cols, seed=m + ty)
    ref = O.matmul_q(raw, ty, rows, cols, x, threads=NCPU)
    got = run(F, ctx, raw, ty, rows, cols, x)
    assert_close(got, ref, f"ty{ty} {rows}x{cols} m{m}", exact_product(raw, ty, rows, cols, x))


def test_q6k_full_int8_scales(F, ctx):
    """GGUF files use the whole int8 range for Q6_K scales; sc * (q - 32) then reaches 4064, which is why the kernel
    splits the scale into two digits."""
    rows, cols, m = 144, 512, 32
    rng = np.random.default_rng(11)
    raw = synth.q6k_blocks(rng, rows * cols // 256).reshape(-1, 210)
    raw[:, 192:208] = rng.integers(-128, 128, size=(raw.shape[0], 16), dtype=np.int64).astype(np.int8).view(np.uint8)
    raw[::7, 192:208] = np.array([-128, 127] * 8, dtype=np.int8).view(np.uint8)
    raw = raw.reshape(-1)
    x = synth.activations(m, cols, seed=3)
    ref = O.matmul_q(raw, 14, rows, cols, x, threads=NCPU)
    assert_close(run(F, ctx, raw, 14, rows, cols, x), ref, "q6k int8 scales", exact_product(raw, 14, rows, cols, x))


def test_q4k_min_term_at_its_extremes(F, ctx):
    """The min term is computed on the tensor core from the 6-bit mins and the sums of the activation limbs over each
    sub-block: all scales and mins at 63 with all quants at 15 (the largest operands), and all quants at 0 (only the
    min term is left), with activations of one sign so that the sub-block sums are as large as they get."""
    rows, cols, m = 144, 1024, 40
    rng = np.random.default_rng(5)
    nblocks = rows * cols // 256
    for qbyte in (0xFF, 0x00):
        raw = np.zeros((nblocks, 144), dtype=np.uint8)
        raw[:, 0:2] = rng.uniform(0.001, 0.01, nblocks).astype(np.float16).view(np.uint8).reshape(-1, 2)
        raw[:, 2:4] = rng.uniform(0.001, 0.01, nblocks).astype(np.float16).view(np.uint8).reshape(-1, 2)
        raw[:, 4:16] = 0xFF
        raw[:, 16:] = qbyte
        raw = raw.reshape(-1)
        x = np.abs(synth.activations(m, cols, seed=8)) + np.float32(0.5)
        ref = O.matmul_q(raw, 12, rows, cols, x, threads=NCPU)
        assert_close(run(F, ctx, raw, 12, rows, cols, x), ref, f"q4k extremes {qbyte:#x}", exact_product(raw, 12, rows, cols, x))


def test_fused_swiglu_finish(F, ctx):
    """gate|up + SwiGLU through the finish kernel against the unfused pair of calls: the reference's own bar for its
    fused kernel is max|d| / max|ref| < 1e-5 (crates/ferric-tensor/examples/ffn_fuse.rs:100-108)."""
    n_ff, cols, m = 384, 1024, 20
    raw = synth.matrix(12, 2 * n_ff, cols, seed=5)
    x = synth.activations(m, cols, seed=6)
    got = run(F, ctx, raw, 12, 2 * n_ff, cols, x, swiglu=True)
    assert got.shape == (m, n_ff)
    unfused = ctx.swiglu(torch.from_numpy(run(F, ctx, raw, 12, 2 * n_ff, cols, x)).cuda(), n_ff).cpu().numpy()
    assert np.abs(got - unfused).max() <= 1e-5 * np.abs(unfused).max()
    ref = O.swiglu(O.matmul_q(raw, 12, 2 * n_ff, cols, x, threads=NCPU), n_ff)
    assert np.abs(got - ref).max() <= 1e-4 * max(1.0, float(np.abs(ref).max()))


@pytest.mark.parametrize("ty,rows,cols,m", [(12, 256, 5120, 17), (14, 640, 4352, 64), (12, 200, 2048, 33)])
def test_k_cut_repeats_bit_for_bit(F, ctx, ty, rows, cols, m):
    """Few row tiles: K is cut across CTAs and a finish kernel adds the pieces in their order -- three launches
    (preparation, product, finish) and the same bits on every repeat, ragged rows included."""
    raw = synth.matrix(ty, rows, cols, seed=rows + m)
    x = synth.activations(m, cols, seed=cols + m)
    qm = F.QMatrix.from_bytes(ctx, raw, ty, rows, cols)
    xd = torch.from_numpy(x).cuda()
    before = ctx.launches()
    first = qm.matmul(xd).cpu().numpy()
    assert ctx.launches() - before == 3
    for _ in range(3):
        again = qm.matmul(xd).cpu().numpy()
        assert (again.view(np.uint32) == first.view(np.uint32)).all()
    assert qm.gemm_status() == 0
    qm.close()
    ref = O.matmul_q(raw, ty, rows, cols, x, threads=NCPU)
    assert_close(first, ref, f"k cut ty{ty} {rows}x{cols} m{m}", exact_product(raw, ty, rows, cols, x))


@pytest.mark.parametrize("ty", [12, 13])
@pytest.mark.parametrize("m", [20, 40])
def test_swiglu_fused_into_the_drain(F, ctx, m, ty):
    """With enough row tiles to fill the machine K is not cut, and each CTA pairs 64 gate rows with the 64 up rows of the
    same outputs and applies SwiGLU itself (no finish kernel)."""
    n_ff, cols = 64 * 150, 512
    raw = synth.matrix(ty, 2 * n_ff, cols, seed=31)
    x = synth.activations(m, cols, seed=32)
    qm = F.QMatrix.from_bytes(ctx, raw, ty, 2 * n_ff, cols)
    xd = torch.from_numpy(x).cuda()
    before = ctx.launches()
    got = qm.try_matmul_swiglu(xd).cpu().numpy()
    assert ctx.launches() - before == 2          # preparation + product
    assert qm.gemm_status() == 0
    qm.close()
    assert got.shape == (m, n_ff)
    ref = O.swiglu(O.matmul_q(raw, ty, 2 * n_ff, cols, x, threads=NCPU), n_ff)
    assert np.abs(got - ref).max() <= 1e-4 * max(1.0, float(np.abs(ref).max()))
    unfused = ctx.swiglu(torch.from_numpy(run(F, ctx, raw, ty, 2 * n_ff, cols, x)).cuda(), n_ff).cpu().numpy()
    assert np.abs(got - unfused).max() <= 1e-5 * np.abs(unfused).max()


def test_scaled_activations_zero_rows_and_outliers(F, ctx):
    """One scale per (activation row, super-block): ranges far outside f16, an all-zero row, an all-zero super-block
    and an outlier that sets its super-block's scale."""
    rows, cols, m = 160, 1024, 12
    raw = synth.matrix(12, rows, cols, seed=9)
    base = synth.activations(m, cols, seed=9)
    for scale in (1e-6, 3e4, 1e10):
        x = (base * np.float32(scale)).astype(np.float32)
        ref = O.matmul_q(raw, 12, rows, cols, x, threads=NCPU)
        assert_close(run(F, ctx, raw, 12, rows, cols, x) / scale, ref / scale, f"scale {scale}")
    x = base.copy()
    x[3] = 0.0
    x[5, 256:512] = 0.0
    x[7, 10] = 3e5
    got = run(F, ctx, raw, 12, rows, cols, x)
    assert (got[3] == 0).all()
    assert_close(got / 1e3, O.matmul_q(raw, 12, rows, cols, x, threads=NCPU) / 1e3, "outlier")


def test_same_result_as_the_gemv_passes(F, ctx, monkeypatch):
    """The tensor-core path keeps 22 bits of each activation under its super-block's largest, the mma.sync GEMV 28;
    both sum exact integer products.  Their results agree far inside the tolerance."""
    rows, cols, m = 256, 1024, 16
    raw = synth.matrix(12, rows, cols, seed=21)
    x = synth.activations(m, cols, seed=22)
    got = run(F, ctx, raw, 12, rows, cols, x)
    qm = F.QMatrix.from_bytes(ctx, raw, 12, rows, cols)
    xd = torch.from_numpy(x).cuda()
    halves = torch.cat([qm.matmul(xd[:8]), qm.matmul(xd[8:])]).cpu().numpy()   # 8 rows at a time: below the threshold, the GEMV
    qm.close()
    assert np.abs(got - halves).max() <= 1e-5 * np.abs(halves).max()


@pytest.mark.parametrize("batch", [12, 64])
def test_full_width_stack_replays_bit_for_bit(F, ctx, batch):
    """Four layers of the full-size stack (every SM busy, K cuts, fused SwiGLU drain, both tiles) at 12 and 64 tokens: the
    captured graph reproduces the eager step bit for bit on every replay, and no bounded wait runs out."""
    from ferric_b200.stack import DecodeStack, TPPlan
    st = DecodeStack(ctx, TPPlan.make(1, 0), n_layers=4, batch=batch)
    st.build_synthetic(seed=3)
    st.reserve()
    gen = torch.Generator(device="cuda").manual_seed(batch)
    h0 = torch.randn(st.h.shape, device="cuda", generator=gen)
    st.h.copy_(h0)
    ref = st.step().clone()
    xn_ref = st.xn.clone()
    assert bool(torch.isfinite(ref).all())
    st.capture()
    for _ in range(10):
        st.h.copy_(h0)
        out = st.run()
        torch.cuda.synchronize()
        assert torch.equal(out, ref) and torch.equal(st.xn, xn_ref)
    assert st.layers[0].wqkv.gemm_status() == 0
    st.close()
