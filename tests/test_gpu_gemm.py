"""GPU parity of the tensor-core prefill product (Q4_K / Q6_K / Q8_0 weights x bf16 activations).

The reference product for this configuration is: weights dequantised with the reference decoder and
rounded to bf16 (nearest even), activations bf16, f32 accumulation.  The tensor core sums in a
different order, so the comparison is done twice: against the exact float64 product of the same bf16
operands and against the oracle's sequential f32 sum (widened by that sum's own distance from the
exact value).

Tolerance: 1e-3 relative + 1e-4 absolute, plus the forward-error term of a dot product,
u * sum_k |x_k w_k| with u = 2^-21.  The tensor core adds each 16-term group into the f32 accumulator
with truncation, so a sum of K terms drifts by up to (K / 16) * 2^-23 of the running sum's magnitude;
on elements where thousands of O(1) terms cancel to ~1e-2 that drift (measured 1.2e-4 at K = 2048) is
above the bare absolute bar although it is 2e-6 of the row's scale.  u = 2^-21 is 8x tighter than the
worst case at K = 2048.  The reference's own kernel tests use max|d| / max|ref| < 1e-5
(crates/ferric-tensor/examples/q4_k.rs:52-55); that bar is asserted as well.
"""
import numpy as np
import pytest
import torch

from ferric_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

RTOL, ATOL, U_ACC = 1e-3, 1e-4, 2.0 ** -21


@pytest.fixture(scope="module")
def F():
    import ferric_b200
    return ferric_b200


@pytest.fixture(scope="module")
def ctx(F):
    c = F.Context(0)
    yield c
    c.close()


def bf16_to_f64(bits):
    return (np.asarray(bits, dtype=np.uint32) << 16).view(np.float32).astype(np.float64)


def blocks(ty, rng, n):
    if ty == 8:
        return synth.q8_0_blocks(rng, n // 32)
    return {12: synth.q4k_blocks, 13: synth.q5k_blocks, 14: synth.q6k_blocks}[ty](rng, n // 256)


def make_case(rows, cols, m, seed, ty=12):
    rng = np.random.default_rng(seed)
    raw = blocks(ty, rng, rows * cols)
    x = torch.from_numpy(rng.standard_normal((m, cols), dtype=np.float32)).to(torch.bfloat16)
    xbits = x.view(torch.int16).numpy().view(np.uint16)
    return raw, x, xbits


def exact_bf16_product(raw, rows, cols, xbits, ty=12):
    """(x . W^T, |x| . |W|^T) in float64 on the bf16 operands."""
    w = bf16_to_f64(O.deq_raw_bf16(raw, rows * cols, ty)).reshape(rows, cols)
    x = bf16_to_f64(xbits)
    return x @ w.T, np.abs(x) @ np.abs(w).T


def check(F, ctx, rows, cols, m, seed, oracle_rows=None, ty=12):
    raw, x, xbits = make_case(rows, cols, m, seed, ty)
    qm = F.QMatrix.from_bytes(ctx, raw, ty, rows, cols)
    y = qm.matmul_bf16(x.cuda())
    assert qm.gemm_status() == 0
    got = y.cpu().numpy().astype(np.float64)
    exact, mag = exact_bf16_product(raw, rows, cols, xbits, ty)
    e = np.abs(got - exact)
    tol = ATOL + RTOL * np.abs(exact) + U_ACC * mag
    w = int(np.argmax(e / tol))
    assert (e <= tol).all(), f"vs exact: worst |d|={e.flat[w]:.3e} at {np.unravel_index(w, e.shape)} (exact {exact.flat[w]:.6g})"
    # the oracle's own sequential f32 sum on a slice of the batch (it is a scalar loop)
    mo = min(m, oracle_rows or m)
    ref = O.matmul_q(raw, ty, rows, cols, xbits[:mo], threads=8, mode=O.MODE_BF16).astype(np.float64)
    e = np.abs(got[:mo] - ref)
    tol = ATOL + RTOL * np.abs(ref) + U_ACC * mag[:mo] + np.abs(ref - exact[:mo])
    assert (e <= tol).all(), f"vs oracle: worst ratio {(e / tol).max():.3f}"
    qm.close()
    return float(np.abs(got - exact).max() / np.abs(exact).max())


SHAPES = [
    (128, 256, 128),      # one CTA, one super-block
    (128, 1024, 128),     # pipeline wraps around its stages
    (256, 512, 256),      # N tile 256
    (144, 768, 40),       # ragged: rows not a multiple of 128, batch below one tile
    (16, 256, 1),         # smallest legal matrix
    (50, 512, 40),        # result pitch not a multiple of 16 bytes: element-wise epilogue instead of TMA stores
    (1000, 2048, 300),    # ragged rows; above 256 activation rows two CTAs pair up on a 256 x 512 tile
    (384, 512, 260),      # an odd number of 128-row tiles: the last pair has a padding CTA
    (128, 256, 700),      # one real CTA, its pair partner all padding, two N tiles
]


@pytest.mark.parametrize("ty", [12, 13, 14, 8])
@pytest.mark.parametrize("rows,cols,m", SHAPES)
def test_small_shapes(F, ctx, rows, cols, m, ty):
    rel = check(F, ctx, rows, cols, m, seed=rows + cols + m + ty, ty=ty)
    assert rel < 1e-5, rel   # the reference's kernel-test bar, max|d| / max|ref| (examples/q4_k.rs:52-55)


@pytest.mark.parametrize("m", [128, 512, 2048])
def test_prefill_config(F, ctx, m):
    """Prefill configuration: hidden 5120 -> 4096 rows (a q-projection slice), batch 128 / 512 / 2048."""
    check(F, ctx, 4096, 5120, m, seed=m, oracle_rows=32)


def bare_bar_stats(got, ref):
    """How far the plain bar |got - ref| <= 1e-4 + 1e-3 |ref| (no allowance for either side's rounding) is from holding:
    (elements over it, elements compared, worst error / bar)."""
    ratio = np.abs(got - ref) / (ATOL + RTOL * np.abs(ref))
    return int((ratio > 1.0).sum()), int(ratio.size), float(ratio.max())


@pytest.mark.parametrize("m", [128, 512, 2048])
def test_prefill_config_full_size(F, ctx, m):
    """configs[3] at its full size: W 17408 x 5120 Q4_K, bf16 activations [m, 5120].  The GPU computes every row; the
    float64 product and the oracle's sequential f32 product are formed on sampled row spans (rows are independent).  The
    number of sampled elements over the plain bar, and by how much, is printed."""
    rows, cols = 17408, 5120
    raw = synth.matrix_on_device(12, rows, cols, seed=3, device="cuda")
    qm = F.QMatrix.from_device_bytes(ctx, raw, 12, rows, cols)
    rb = cols // 256 * 144
    spans = [(0, 48), (8696, 8744), (17360, 17408)]
    host = {sp: raw[sp[0] * rb:sp[1] * rb].cpu().numpy() for sp in spans}
    del raw
    x = torch.from_numpy(synth.activations(m, cols, seed=3)).to(torch.bfloat16)
    xbits = x.view(torch.int16).numpy().view(np.uint16)
    y = qm.matmul_bf16(x.cuda())
    assert qm.gemm_status() == 0
    got_all = y.cpu().numpy().astype(np.float64)
    assert got_all.shape == (m, rows) and np.isfinite(got_all).all()
    over = total = 0
    worst = 0.0
    mo = min(m, 32)                                    # the oracle is a scalar loop: a slice of the batch
    for (lo, hi), rbytes in host.items():
        got = got_all[:, lo:hi]
        exact, mag = exact_bf16_product(rbytes, hi - lo, cols, xbits)
        e = np.abs(got - exact)
        tol = ATOL + RTOL * np.abs(exact) + U_ACC * mag
        assert (e <= tol).all(), f"rows {lo}:{hi} vs exact: worst ratio {(e / tol).max():.3f}"
        ref = O.matmul_q(rbytes, 12, hi - lo, cols, xbits[:mo], threads=8, mode=O.MODE_BF16).astype(np.float64)
        e = np.abs(got[:mo] - ref)
        tol = ATOL + RTOL * np.abs(ref) + U_ACC * mag[:mo] + np.abs(ref - exact[:mo])
        assert (e <= tol).all(), f"rows {lo}:{hi} vs oracle: worst ratio {(e / tol).max():.3f}"
        o, t, w = bare_bar_stats(got[:mo], ref)
        over, total, worst = over + o, total + t, max(worst, w)
    print(f"BARE-BAR config3 m={m}: {over} of {total} sampled elements over 1e-4 + 1e-3|ref|, worst ratio {worst:.2f}")
    qm.close()


def test_prefill_down_q6k(F, ctx):
    """The Q6_K down projection of the same layer (K = 17408), a 1024-row slice, batch 512."""
    check(F, ctx, 1024, 17408, 512, seed=5, oracle_rows=16, ty=14)


@pytest.mark.parametrize("ty", [12, 13, 14, 8])
def test_dequant_stage_is_bit_exact(F, ctx, ty):
    """x = identity columns: y[i, r] is then exactly the bf16 weight W[r, i] -- the dequant-to-bf16 stage
    inside the kernel must match the oracle's bf16 dequantisation bit for bit."""
    rows, cols = 256, 256
    rng = np.random.default_rng(7)
    raw = blocks(ty, rng, rows * cols)
    qm = F.QMatrix.from_bytes(ctx, raw, ty, rows, cols)
    x = torch.eye(cols, dtype=torch.bfloat16, device="cuda")
    y = qm.matmul_bf16(x)
    assert qm.gemm_status() == 0
    got = y.cpu().numpy()                                  # [cols, rows]
    want = (O.deq_raw_bf16(raw, rows * cols, ty).astype(np.uint32) << 16).view(np.float32).reshape(rows, cols)
    # a weight of -0.0 (Q6_K: q = 32 under a negative scale) reaches y as +0.0: it is summed with the +0.0 products
    # of the other columns.  Every other value must match bit for bit.
    want = want + np.float32(0.0)
    assert np.array_equal(np.ascontiguousarray(got.T).view(np.uint32), want.view(np.uint32))
    qm.close()


def test_q8_0_needs_256_column_multiples(F, ctx):
    """Q8_0 itself only needs columns in multiples of 32; the tensor-core product walks K in groups of 256 and declines
    other widths (the caller then uses matmul_q)."""
    rng = np.random.default_rng(1)
    raw = synth.q8_0_blocks(rng, 16 * 288 // 32)
    qm = F.QMatrix.from_bytes(ctx, raw, 8, 16, 288)
    with pytest.raises(F.FerricError):
        qm.matmul_bf16(torch.zeros(4, 288, dtype=torch.bfloat16, device="cuda"))
    qm.close()
