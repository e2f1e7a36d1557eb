"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on identical inputs.

Bars: dequantised weights bit-exact (f32 and bf16); dot products within 1e-3 relative + 1e-4
absolute of the reference product (dequantise, then sequential f32 dot).  The reference's own
kernel tests use max|d| / max|ref| < 1e-5 (crates/ferric-tensor/examples/q4_k.rs:52-55); that
figure is asserted too where the reference asserts it.
"""
import os

import numpy as np
import pytest
import torch

import np_decoders as D
from ferric_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

KAT = np.load(os.path.join(os.path.dirname(__file__), "golden", "kat.npz"))
RTOL, ATOL = 1e-3, 1e-4
NCPU = os.cpu_count() or 1


@pytest.fixture(scope="module")
def F():
    import ferric_b200
    return ferric_b200


@pytest.fixture(scope="module")
def ctx(F):
    c = F.Context(0)
    caps = c.caps()
    assert caps["cc_major"] >= 10, caps
    yield c
    c.close()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_close(got, ref, what="", exact=None):
    """|got - ref| <= 1e-4 + 1e-3 |ref|, element-wise.

    With `exact` (the same dequantised weights multiplied in float64) the reference's own f32
    rounding is taken out of the comparison: a sequential f32 sum over K = 17408 terms is itself
    ~1e-4 away from the exact value, and that distance is not the kernel's error.  Then the kernel
    must be within the tolerance of the exact product, and within the tolerance plus the
    reference's measured own deviation of the reference."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    err = np.abs(got - ref)
    tol = ATOL + RTOL * np.abs(ref)
    if exact is not None:
        exact = np.asarray(exact, dtype=np.float64)
        e2 = np.abs(got - exact)
        t2 = ATOL + RTOL * np.abs(exact)
        w2 = int(np.argmax(e2 / t2))
        assert (e2 <= t2).all(), f"{what}: vs exact, worst |d|={e2.flat[w2]:.3e} at {w2} (exact {exact.flat[w2]:.6g})"
        tol = tol + np.abs(ref - exact)
    worst = int(np.argmax(err / tol))
    assert (err <= tol).all(), f"{what}: worst |d|={err.flat[worst]:.3e} at {worst} (ref {ref.flat[worst]:.6g}, tol {tol.flat[worst]:.3e})"
    return float((err / tol).max())


def bare_bar(got, ref, what):
    """Print how far the plain bar |got - ref| <= 1e-4 + 1e-3 |ref| -- with no allowance for the reference product's own
    f32 rounding -- is from holding: elements over it and the worst error / bar ratio."""
    ratio = np.abs(np.asarray(got, np.float64) - np.asarray(ref, np.float64)) / (ATOL + RTOL * np.abs(np.asarray(ref, np.float64)))
    print(f"BARE-BAR {what}: {int((ratio > 1).sum())} of {ratio.size} elements over 1e-4 + 1e-3|ref|, worst ratio {ratio.max():.2f}")


def exact_product(raw, ty, rows, cols, x):
    """x . W^T with the oracle-dequantised weights (exact f32 values) accumulated in float64."""
    vals, bb = synth.BLOCK[ty]
    rb = cols // vals * bb
    x64 = np.asarray(x, dtype=np.float64)
    out = np.empty((x64.shape[0], rows), dtype=np.float64)
    for r0 in range(0, rows, 1024):
        n = min(1024, rows - r0)
        w = O.deq_raw(raw[r0 * rb:(r0 + n) * rb], n * cols, ty).reshape(n, cols).astype(np.float64)
        out[:, r0:r0 + n] = x64 @ w.T
    return out


def gpu_matmul(F, ctx, raw, ty, rows, cols, x):
    qm = F.QMatrix.from_bytes(ctx, raw, ty, rows, cols)
    y = qm.matmul(torch.from_numpy(np.ascontiguousarray(x)).cuda())
    torch.cuda.synchronize()
    out = y.cpu().numpy()
    qm.close()
    return out


def x_cos(m, k, f=0.013):
    return np.cos(np.arange(m * k, dtype=np.float32) * np.float32(f)).astype(np.float32).reshape(m, k)


# ------------------------------------------------------------------------------ decoders
@pytest.mark.parametrize("name,ty", [("q4k_fix", 12), ("q4k_rand", 12), ("q6k_fix", 14), ("q6k_rand", 14),
                                     ("q6k_wild", 14), ("q8_rand", 8), ("handbuilt_q4k", 12)])
def test_deq_raw_matches_golden_bits(F, ctx, name, ty):
    raw = KAT[name + "_raw"]
    want = bits(KAT["handbuilt_q4k_expected"]) if name == "handbuilt_q4k" else KAT[name + "_bits"]
    got = ctx.deq_raw(raw, want.size, ty)
    assert (bits(got) == want).all()


def test_deq_raw_partial_block_and_errors(F, ctx):
    raw = KAT["q4k_rand_raw"]
    got = ctx.deq_raw(raw, 300, 12)            # one whole block, the rest stays zero (vec![0.0; n])
    assert (bits(got[:256]) == KAT["q4k_rand_bits"][:256]).all() and (got[256:] == 0).all()
    with pytest.raises(F.FerricError) as e:
        ctx.deq_raw(raw, 256, 99)
    assert e.value.status == 2
    with pytest.raises(F.FerricError) as e:
        ctx.deq_raw(raw[:100], 256, 12)
    assert e.value.status == 3


@pytest.mark.parametrize("ty", [12, 13, 14, 8])
@pytest.mark.parametrize("rows,cols", [(1, 256), (16, 512), (17, 768), (100, 1024), (515, 2048)])
def test_loaded_matrix_dequantises_bit_exactly(F, ctx, ty, rows, cols):
    raw = synth.matrix(ty, rows, cols, seed=rows * 7 + cols + ty)
    qm = F.QMatrix.from_bytes(ctx, raw, ty, rows, cols)
    assert (qm.rows(), qm.cols(), qm.n_shards(), qm.ggml_type()) == (rows, cols, 1, ty)
    assert qm.nbytes() == raw.size == F.type_size(ty, rows * cols)
    want = O.deq_raw(raw, rows * cols, ty)
    got = qm.dequant().cpu().numpy().reshape(-1)
    assert (bits(got) == bits(want)).all()
    gb = qm.dequant(bf16=True).view(torch.int16).cpu().numpy().view(np.uint16).reshape(-1)
    assert (gb == O.deq_raw_bf16(raw, rows * cols, ty)).all()
    qm.close()


def test_fully_random_bytes_dequantise_bit_exactly(F, ctx):
    rng = np.random.default_rng(77)
    for ty in (12, 13, 14, 8):
        vals, bb = synth.BLOCK[ty]
        rows, cols = 48, 4 * 256
        raw = rng.integers(0, 256, size=rows * (cols // vals) * bb, dtype=np.uint8)
        want = O.deq_raw(raw, rows * cols, ty)
        qm = F.QMatrix.from_bytes(ctx, raw, ty, rows, cols)
        got = qm.dequant().cpu().numpy().reshape(-1)
        ok = np.isfinite(want)
        assert (bits(got)[ok] == bits(want)[ok]).all() and (np.isfinite(got) == ok).all()
        qm.close()


# ------------------------------------------------------------------------------ products
@pytest.mark.parametrize("ty,shapes", [(12, [(8, 256, 4), (13, 512, 1), (4096, 2048, 1)]),
                                       (14, [(8, 256, 4), (7, 512, 1), (2048, 1024, 1)]),
                                       (8, [(8, 256, 4), (13, 128, 1), (4096, 2048, 1)])])
def test_reference_kernel_examples(F, ctx, ty, shapes):
    """crates/ferric-tensor/examples/q4_k.rs, q6_k.rs, q8_0.rs: packed matmul vs dequant-then-f32."""
    for rows, k, m in shapes:
        if ty == 12:
            raw = np.concatenate([O.q4k_block(i + 1) for i in range(rows * k // 256)])
        elif ty == 14:
            raw = np.concatenate([O.q6k_block(i + 1) for i in range(rows * k // 256)])
        else:
            w = (np.sin(np.arange(rows * k, dtype=np.float32) * np.float32(0.021)) * np.float32(0.7)).astype(np.float32)
            raw = np.concatenate([O.quant_q8_0(w[r * k:(r + 1) * k]) for r in range(rows)])
        x = x_cos(m, k)
        ref = O.matmul_q(raw, ty, rows, k, x, threads=NCPU)
        got = gpu_matmul(F, ctx, raw, ty, rows, k, x)
        assert got.shape == (m, rows)
        assert_close(got, ref, f"ty{ty} {rows}x{k} m{m}")
        scale = max(np.abs(ref).max(), 1e-3)
        assert np.abs(got - ref).max() / scale < 1e-5


def test_config0_q4k_4096(F, ctx):
    raw = synth.matrix(12, 4096, 4096, seed=0)
    x = synth.activations(1, 4096, seed=0)
    ref = O.matmul_q(raw, 12, 4096, 4096, x, threads=NCPU)
    got = gpu_matmul(F, ctx, raw, 12, 4096, 4096, x)
    exact = exact_product(raw, 12, 4096, 4096, x)
    assert_close(got, ref, "config 0", exact)
    bare_bar(got, ref, "config0 q4k 4096x4096")
    # the reference's other accumulation orders (fused per-block rows, GPU kernel order) agree too
    assert_close(got, O.matmul_q(raw, 12, 4096, 4096, x, threads=NCPU, mode=O.MODE_FUSED), "config 0 fused order", exact)
    assert_close(got, O.matmul_q(raw, 12, 4096, 4096, x, threads=NCPU, mode=O.MODE_SHADER), "config 0 kernel order", exact)


@pytest.mark.parametrize("name,ty,rows,cols", [("q", 12, 5120, 5120), ("k", 12, 1024, 5120), ("gate", 12, 17408, 5120),
                                               ("down", 14, 5120, 17408)])
def test_config1_layer_matrices(F, ctx, name, ty, rows, cols):
    raw = synth.matrix(ty, rows, cols, seed=1 + len(name))
    x = synth.activations(1, cols, seed=1)
    ref = O.matmul_q(raw, ty, rows, cols, x, threads=NCPU)
    got = gpu_matmul(F, ctx, raw, ty, rows, cols, x)
    exact = exact_product(raw, ty, rows, cols, x)
    assert_close(got, ref, f"config 1 {name}", exact)
    bare_bar(got, ref, f"config1 {name} {rows}x{cols}")
    bare_bar(ref, exact, f"config1 {name}: the reference product itself against the float64 product")
    print(f"config 1 {name}: max|gpu-exact| {np.abs(got - exact).max():.2e}  max|cpu_ref-exact| {np.abs(ref - exact).max():.2e}")


def test_config2_output_head_rows_sampled(F, ctx):
    """151936 x 5120 Q6_K at batch 1 and 64.  The oracle runs on sampled row spans (rows are
    independent: crates/ferric-tensor/src/cpu_simd.rs:74-78); the GPU runs the whole matrix."""
    rows, cols = 151936, 5120
    raw = synth.matrix_on_device(14, rows, cols, seed=2, device="cuda")
    qm = F.QMatrix.from_device_bytes(ctx, raw, 14, rows, cols)
    row_bytes = cols // 256 * 210
    spans = [(0, 64), (75961, 76025), (151872, 151936)]
    host = {s: raw[s[0] * row_bytes:s[1] * row_bytes].cpu().numpy() for s in spans}
    del raw
    for m in (1, 64):
        x = synth.activations(m, cols, seed=2)
        y = qm.matmul(torch.from_numpy(x).cuda())
        torch.cuda.synchronize()
        y = y.cpu().numpy()
        assert y.shape == (m, rows) and np.isfinite(y).all()
        for (lo, hi), rb in host.items():
            ref = O.matmul_q(rb, 14, hi - lo, cols, x, threads=NCPU)
            assert_close(y[:, lo:hi], ref, f"config 2 m={m} rows {lo}:{hi}", exact_product(rb, 14, hi - lo, cols, x))
            bare_bar(y[:, lo:hi], ref, f"config2 head m={m} rows {lo}:{hi}")
    qm.close()


@pytest.mark.parametrize("m", [16, 64])
def test_config1_products_at_many_rows_full_size_rows_sampled(F, ctx, m):
    """The layer's two big products at their full size with 16 and 64 activation rows (the tensor-core decode kernel at
    both tiles): gate|up 34816 x 5120 Q4_K with SwiGLU in the kernel's drain (every SM busy, two waves) and down
    5120 x 17408 Q6_K with its K range cut across CTAs.  The oracle runs on sampled row spans."""
    n_ff, cols = 17408, 5120
    raw = synth.matrix_on_device(12, 2 * n_ff, cols, seed=5, device="cuda")
    qm = F.QMatrix.from_device_bytes(ctx, raw, 12, 2 * n_ff, cols)
    row_bytes = cols // 256 * 144
    spans = [(0, 32), (8711, 8743), (n_ff - 32, n_ff)]
    host = {s: (raw[s[0] * row_bytes:s[1] * row_bytes].cpu().numpy(),
                raw[(n_ff + s[0]) * row_bytes:(n_ff + s[1]) * row_bytes].cpu().numpy()) for s in spans}
    del raw
    x = synth.activations(m, cols, seed=m)
    y = qm.try_matmul_swiglu(torch.from_numpy(x).cuda()).cpu().numpy()
    assert y.shape == (m, n_ff) and np.isfinite(y).all() and qm.gemm_status() == 0
    for (lo, hi), (gate, up) in host.items():
        both = np.concatenate([gate, up])
        ref = O.swiglu(O.matmul_q(both, 12, 2 * (hi - lo), cols, x, threads=NCPU), hi - lo)
        assert np.abs(y[:, lo:hi] - ref).max() <= 1e-4 * max(1.0, float(np.abs(ref).max())), (lo, hi)
    qm.close()
    rows, cols = 5120, 17408
    raw = synth.matrix_on_device(14, rows, cols, seed=6, device="cuda")
    qm = F.QMatrix.from_device_bytes(ctx, raw, 14, rows, cols)
    row_bytes = cols // 256 * 210
    spans = [(0, 48), (2500, 2548), (rows - 48, rows)]
    host = {s: raw[s[0] * row_bytes:s[1] * row_bytes].cpu().numpy() for s in spans}
    del raw
    x = synth.activations(m, cols, seed=m + 1)
    y = qm.matmul(torch.from_numpy(x).cuda()).cpu().numpy()
    assert y.shape == (m, rows) and np.isfinite(y).all() and qm.gemm_status() == 0
    for (lo, hi), rb in host.items():
        ref = O.matmul_q(rb, 14, hi - lo, cols, x, threads=NCPU)
        assert_close(y[:, lo:hi], ref, f"down m={m} rows {lo}:{hi}", exact_product(rb, 14, hi - lo, cols, x))
    qm.close()


@pytest.mark.parametrize("ty", [12, 13, 14, 8])
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 9, 16, 17, 33, 64])
def test_batch_sizes(F, ctx, ty, m):
    rows, cols = 200, 1024
    raw = synth.matrix(ty, rows, cols, seed=40 + ty)
    x = synth.activations(m, cols, seed=m)
    ref = O.matmul_q(raw, ty, rows, cols, x, threads=NCPU)
    got = gpu_matmul(F, ctx, raw, ty, rows, cols, x)
    assert_close(got, ref, f"ty{ty} m{m}", exact_product(raw, ty, rows, cols, x))


@pytest.mark.parametrize("ty", [12, 13, 14, 8])
def test_edge_shapes_and_ranges(F, ctx, ty):
    vals = synth.BLOCK[ty][0]
    # ragged row counts around the 16-row tile, one block of K, and K deeper than one warp's share
    for rows, cols in [(1, 256), (15, 256), (16, 256), (17, 512), (31, 256), (33, 4352)]:
        raw = synth.matrix(ty, rows, cols, seed=rows + cols)
        x = synth.activations(2, cols, seed=rows)
        assert_close(gpu_matmul(F, ctx, raw, ty, rows, cols, x), O.matmul_q(raw, ty, rows, cols, x), f"{rows}x{cols}",
                     exact_product(raw, ty, rows, cols, x))
    rows, cols = 64, 1024
    raw = synth.matrix(ty, rows, cols, seed=9)
    base = synth.activations(3, cols, seed=9)
    for scale in (1e-6, 1.0, 3e4, 1e10):          # far outside f16 range: the split is per-block scaled
        x = (base * np.float32(scale)).astype(np.float32)
        ref = O.matmul_q(raw, ty, rows, cols, x)
        got = gpu_matmul(F, ctx, raw, ty, rows, cols, x)
        assert_close(got / scale, ref / scale, f"ty{ty} scale {scale}")
    x = base.copy()
    x[0, :] = 0.0                                    # an all-zero row
    x[1, 5] = 3e5                                    # one outlier inside a block
    assert_close(gpu_matmul(F, ctx, raw, ty, rows, cols, x) / 1e3, O.matmul_q(raw, ty, rows, cols, x) / 1e3, "outlier")
    # empty batch: nothing to do, nothing written
    qm = F.QMatrix.from_bytes(ctx, raw, ty, rows, cols)
    y = qm.matmul(torch.empty((0, cols), dtype=torch.float32, device="cuda"))
    assert tuple(y.shape) == (0, rows)
    if ty == 8:
        assert vals == 32
    qm.close()


def test_empty_matrix(F, ctx):
    qm = F.QMatrix.from_bytes(ctx, np.zeros(0, np.uint8), 12, 0, 256)
    assert qm.rows() == 0 and qm.nbytes() == 0
    y = qm.matmul(torch.zeros((2, 256), dtype=torch.float32, device="cuda"))
    assert tuple(y.shape) == (2, 0)
    qm.close()


def test_constructor_and_shape_errors(F, ctx):
    raw = synth.matrix(12, 4, 256, seed=1)
    with pytest.raises(F.FerricError) as e:
        F.QMatrix.from_bytes(ctx, raw, 2, 4, 256)          # Q4_0: no packed kernel here
    assert e.value.status == 2 and "no native matmul" in str(e.value)
    with pytest.raises(F.FerricError) as e:
        F.QMatrix.from_bytes(ctx, raw[:-1], 12, 4, 256)
    assert e.value.status == 3 and "byte length" in str(e.value)
    with pytest.raises(F.FerricError) as e:
        F.QMatrix.from_bytes(ctx, raw, 12, 8, 128)
    assert e.value.status == 3
    qm = F.QMatrix.from_bytes(ctx, raw, 12, 4, 256)
    with pytest.raises(F.FerricError) as e:
        qm.matmul(torch.zeros((1, 512), dtype=torch.float32, device="cuda"))
    assert e.value.status == 3 and "inner dim mismatch" in str(e.value)
    qm.close()


def test_host_buffer_entry_point(F, ctx):
    raw = synth.matrix(12, 300, 1024, seed=3)
    x = synth.activations(5, 1024, seed=3)
    qm = F.QMatrix.from_bytes(ctx, raw, 12, 300, 1024)
    assert_close(qm.matmul_host(x), O.matmul_q(raw, 12, 300, 1024, x), "host buffers")
    qm.close()


# ------------------------------------------------------------------------------ fused SwiGLU
@pytest.mark.parametrize("ty", [12, 14])
@pytest.mark.parametrize("t", [1, 8])
def test_fused_gate_up_swiglu(F, ctx, ty, t):
    """crates/ferric-tensor/examples/ffn_fuse.rs:60-108 (n_ff 3072, n_embd 1024, cos inputs)."""
    n_ff, n_embd = 3072, 1024
    nblk = n_embd // 256
    gen = O.q4k_block if ty == 12 else O.q6k_block
    raw = np.concatenate([gen(i + 1) for i in range(2 * n_ff * nblk)])
    h = (np.cos(np.arange(t * n_embd, dtype=np.float32) * np.float32(0.017)) * np.float32(0.3)).astype(np.float32).reshape(t, n_embd)
    qm = F.QMatrix.from_bytes(ctx, raw, ty, 2 * n_ff, n_embd)
    hx = torch.from_numpy(h).cuda()
    fused = qm.try_matmul_swiglu(hx)
    assert fused is not None and tuple(fused.shape) == (t, n_ff)
    unfused = ctx.swiglu(qm.matmul(hx), n_ff)
    torch.cuda.synchronize()
    fused, unfused = fused.cpu().numpy(), unfused.cpu().numpy()
    scale = max(np.abs(unfused).max(), 1e-3)
    assert np.abs(fused - unfused).max() / scale < 1e-5
    ref = O.swiglu(O.matmul_q(raw, ty, 2 * n_ff, n_embd, h, threads=NCPU), n_ff)
    assert np.abs(fused - ref).max() / max(np.abs(ref).max(), 1e-3) < 1e-5
    qm.close()


@pytest.mark.parametrize("t", [1, 3, 8])
def test_fused_gate_up_swiglu_q5k(F, ctx, t):
    """Q5_K gate|up takes the Q4_K kernel with the fifth bit OR-ed in; same bar as the reference's fused-vs-unfused
    check (crates/ferric-tensor/examples/ffn_fuse.rs:100-108)."""
    n_ff, n_embd = 1024, 1536
    raw = synth.matrix(13, 2 * n_ff, n_embd, seed=13)
    h = synth.activations(t, n_embd, seed=t)
    qm = F.QMatrix.from_bytes(ctx, raw, 13, 2 * n_ff, n_embd)
    hx = torch.from_numpy(h).cuda()
    fused = qm.try_matmul_swiglu(hx)
    assert fused is not None and tuple(fused.shape) == (t, n_ff)
    unfused = ctx.swiglu(qm.matmul(hx), n_ff).cpu().numpy()
    fused = fused.cpu().numpy()
    assert np.abs(fused - unfused).max() / max(np.abs(unfused).max(), 1e-3) < 1e-5
    ref = O.swiglu(O.matmul_q(raw, 13, 2 * n_ff, n_embd, h, threads=NCPU), n_ff)
    assert np.abs(fused - ref).max() / max(np.abs(ref).max(), 1e-3) < 1e-4
    qm.close()


def test_swiglu_declines_what_the_reference_declines(F, ctx):
    raw = synth.matrix(8, 64, 256, seed=1)
    qm = F.QMatrix.from_bytes(ctx, raw, 8, 64, 256)
    x = torch.from_numpy(synth.activations(1, 256, 1)).cuda()
    assert qm.try_matmul_swiglu(x) is None                   # Q8_0: the reference returns None
    got = qm.gate_up_swiglu(x).cpu().numpy()                 # ... and the caller falls back
    ref = O.swiglu(O.matmul_q(raw, 8, 64, 256, synth.activations(1, 256, 1)), 32)
    assert_close(got, ref, "unfused fallback")
    qm.close()


# ------------------------------------------------------------------------------ norms around the matmuls
@pytest.mark.parametrize("rows,d", [(1, 5120), (3, 1024), (8, 256)])
def test_add_rmsnorm_matches_reference_kernel(F, ctx, rows, d):
    rng = np.random.default_rng(rows + d)
    a = rng.standard_normal((rows, d)).astype(np.float32) * np.float32(3)
    b = rng.standard_normal((rows, d)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, d).astype(np.float32)
    ta, tb, tw = (torch.from_numpy(v).cuda() for v in (a, b, w))
    s_ref, n_ref = O.add_rmsnorm(a, b, w, 1e-6)
    s, n = ctx.add_rmsnorm(ta, tb, tw, 1e-6)
    assert (s.cpu().numpy().view(np.uint32) == s_ref.view(np.uint32)).all()          # the sum is one f32 add
    assert np.abs(n.cpu().numpy() - n_ref).max() <= 1e-5 * np.abs(n_ref).max()    # the mean of squares reassociates
    _, n2 = ctx.add_rmsnorm(ta, None, None, 1e-6)                                   # plain, weightless rmsnorm
    assert np.abs(n2.cpu().numpy() - O.add_rmsnorm(a, None, None, 1e-6)[1]).max() <= 1e-5 * np.abs(n_ref).max()


@pytest.mark.parametrize("ty", [12, 13, 14])
@pytest.mark.parametrize("m,d", [(1, 1536), (2, 1536), (5, 1536), (1, 5120), (8, 5120), (3, 2304)])
def test_fused_add_rmsnorm_prepare(F, ctx, ty, m, d):
    """(from 8 super-blocks per row on, the kernel spreads a row over a cluster of four CTAs)"""
    rows = 96
    raw = synth.matrix(ty, rows, d, seed=21)
    rng = np.random.default_rng(m)
    a = rng.standard_normal((m, d)).astype(np.float32) * np.float32(2)
    b = rng.standard_normal((m, d)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, d).astype(np.float32)
    qm = F.QMatrix.from_bytes(ctx, raw, ty, rows, d)
    ta, tb, tw = (torch.from_numpy(v).cuda() for v in (a, b, w))
    s_out, n_out = torch.empty_like(ta), torch.empty_like(ta)
    mm = qm.add_rmsnorm_prepare(ta, tb, tw, 1e-6, sum_out=s_out, norm_out=n_out)
    y = qm.matmul_prepared(mm).cpu().numpy()
    s_ref, n_ref = O.add_rmsnorm(a, b, w, 1e-6)
    assert (s_out.cpu().numpy().view(np.uint32) == s_ref.view(np.uint32)).all()
    assert np.abs(n_out.cpu().numpy() - n_ref).max() <= 1e-5 * np.abs(n_ref).max()
    # the product must be the unfused pair's: matmul_q of the norm this kernel produced
    y2 = qm.matmul(n_out).cpu().numpy()
    assert np.abs(y - y2).max() <= 1e-6 * max(np.abs(y2).max(), 1e-3)
    assert_close(y, O.matmul_q(raw, ty, rows, d, n_ref), "fused norm + prepare", exact_product(raw, ty, rows, d, n_ref))
    # in place on the residual stream, no norm written
    qm.add_rmsnorm_prepare(ta, tb, tw, 1e-6, sum_out=ta)
    y3 = qm.matmul_prepared(mm).cpu().numpy()
    assert (ta.cpu().numpy().view(np.uint32) == s_ref.view(np.uint32)).all() and np.array_equal(y3, y)
    qm.close()


@pytest.mark.parametrize("batch", [2, 6, 12, 40])
def test_decode_stack_step_matches_layerwise_oracle(F, ctx, batch):
    """Two small layers of the decode stack against the oracle, kernel by kernel semantics: one GEMV pass (2 tokens, the
    chained form), two passes (6), and the tensor-core decode kernel at its narrow and wide tile (12, 40 tokens: the
    step for more than 8 tokens, with the fused SwiGLU finish and K cuts of these small matrices)."""
    from ferric_b200.stack import DecodeStack, TPPlan
    plan = TPPlan.make(1, 0, hidden=512, n_ff=768, q_out=512, kv_out=256)
    st = DecodeStack(ctx, plan, n_layers=2, batch=batch)
    rng = np.random.default_rng(8)
    raws = []
    for l in range(2):
        mats = [(12, plan.q_rows + 2 * plan.kv_rows, 512), (12, 512, plan.q_rows), (12, 2 * plan.ff_rows, 512), (14, 512, plan.ff_rows)]
        raw = [synth.matrix(ty, r, c, seed=100 + 10 * l + i) for i, (ty, r, c) in enumerate(mats)]
        raws.append(list(zip(mats, raw)))
        st.add_layer(*[F.QMatrix.from_bytes(ctx, rw, ty, r, c) for (ty, r, c), rw in zip(mats, raw)])
    st.reserve()
    h0 = rng.standard_normal((batch, 512)).astype(np.float32)
    st.h.copy_(torch.from_numpy(h0).cuda())
    got = st.step().cpu().numpy()
    h = h0.copy()
    xn = O.add_rmsnorm(h, None, None, 1e-6)[1]
    for (q, o, gu, dn) in raws:
        qkv = O.matmul_q(q[1], *q[0], xn)
        oo = O.matmul_q(o[1], *o[0], np.ascontiguousarray(qkv[:, :plan.q_rows]))
        h, xn = O.add_rmsnorm(h, oo, None, 1e-6)
        f = O.swiglu(O.matmul_q(gu[1], *gu[0], xn), plan.ff_rows)
        dd = O.matmul_q(dn[1], *dn[0], f)
        h, xn = O.add_rmsnorm(h, dd, None, 1e-6)
    assert np.abs(got - h).max() <= 1e-4 + 1e-3 * np.abs(h).max()
    st.capture()
    st.h.copy_(torch.from_numpy(h0).cuda())
    got2 = st.run().cpu().numpy()
    assert np.array_equal(got, got2)           # graph replay == eager launches, bit for bit
    st.close()


def test_profile_buckets(F):
    """prof / prof_report (crates/ferric-tensor/src/lib.rs:3017-3046): time between marks lands in named buckets."""
    c = F.Context(0)
    qm = F.QMatrix.from_bytes(c, synth.matrix(12, 4096, 4096, seed=0), 12, 4096, 4096)
    x = torch.randn((1, 4096), device="cuda")
    c.prof("ignored")                                           # off: a no-op
    assert c.prof_report().strip().endswith("0.000 total)")
    c.prof_enable(True)
    c.prof("start")                                             # the first mark only starts the clock
    for _ in range(50):
        qm.matmul(x)
    c.prof("matmul_q")
    c.add_rmsnorm(x, None, None, 1e-6)
    c.prof("rmsnorm")
    rep = c.prof_report()
    lines = [l.split() for l in rep.splitlines()[1:]]
    assert [l[0] for l in lines] == ["matmul_q", "rmsnorm"] and float(lines[0][1]) > float(lines[1][1]) > 0
    assert "start" not in rep and c.prof_report().strip().endswith("0.000 total)")      # reset after a full report
    qm.close()
    c.close()


def test_dense_fallback_matrix(F, ctx):
    """QMatrix::from_dense (crates/ferric-tensor/src/dtype.rs:912-926): a format without a packed kernel reaches the
    matmul as an already dequantised f32 weight; the product is the reference's dense x . W^T."""
    rows, cols = 203, 1000                                         # neither a tile nor a vector multiple
    rng = np.random.default_rng(17)
    w = rng.standard_normal((rows, cols)).astype(np.float32) * np.float32(0.05)
    qm = F.QMatrix.from_dense(ctx, w)
    assert (qm.rows(), qm.cols(), qm.ggml_type(), qm.n_shards(), qm.nbytes()) == (rows, cols, 0, 1, rows * cols * 4)
    assert np.array_equal(qm.dequant().cpu().numpy(), w)
    for m in (1, 3, 9):
        x = synth.activations(m, cols, seed=m)
        got = qm.matmul(torch.from_numpy(x).cuda()).cpu().numpy()
        assert_close(got, O.matmul_bt(x, w), f"dense m={m}", x.astype(np.float64) @ w.astype(np.float64).T)
    assert qm.try_matmul_swiglu(torch.zeros((1, cols), device="cuda")) is None       # the reference's None
    with pytest.raises(F.FerricError) as e:
        qm.prepare(torch.zeros((1, cols), device="cuda"))
    assert e.value.status == 6
    qm.close()
    # dequantise a packed format on the host, load it dense: same product as the packed matrix within the bar
    raw = synth.matrix(12, 64, 512, seed=5)
    dense = F.QMatrix.from_dense(ctx, O.deq_raw(raw, 64 * 512, 12).reshape(64, 512))
    packed = F.QMatrix.from_bytes(ctx, raw, 12, 64, 512)
    x = torch.from_numpy(synth.activations(2, 512, seed=6)).cuda()
    assert_close(dense.matmul(x).cpu().numpy(), packed.matmul(x).cpu().numpy(), "dense vs packed")
    dense.close()
    packed.close()


# ------------------------------------------------------------------------------ shards
@pytest.mark.parametrize("ty", [12, 13, 14, 8])
def test_row_and_k_shards_compose(F, ctx, ty):
    rows, cols = 96, 2048
    vals, bb = synth.BLOCK[ty]
    raw = synth.matrix(ty, rows, cols, seed=11)
    x = synth.activations(2, cols, seed=11)
    full = O.matmul_q(raw, ty, rows, cols, x)
    xd = torch.from_numpy(x).cuda()
    # column-parallel: row ranges concatenate exactly like the reference's row shards + cat
    parts = []
    for r0, r1 in [(0, 40), (40, 41), (41, 96)]:
        qm = F.QMatrix.from_bytes_view(ctx, raw, ty, rows, cols, r0, r1 - r0, 0, cols)
        parts.append(qm.matmul(xd).cpu().numpy())
        qm.close()
    assert_close(np.concatenate(parts, axis=1), full, "row shards")
    # row-parallel: K ranges sum to the full product
    total = np.zeros_like(full, dtype=np.float64)
    for c0, c1 in [(0, 768), (768, 1024), (1024, 2048)]:
        qm = F.QMatrix.from_bytes_view(ctx, raw, ty, rows, cols, 0, rows, c0, c1 - c0)
        total += qm.matmul(xd[:, c0:c1].contiguous()).cpu().numpy()
        # each shard equals the oracle on the gathered K slice
        rb = raw.reshape(rows, cols // vals, bb)[:, c0 // vals:c1 // vals, :].reshape(-1)
        assert_close(qm.matmul(xd[:, c0:c1].contiguous()).cpu().numpy(), O.matmul_q(rb, ty, rows, c1 - c0, x[:, c0:c1]), "k shard")
        qm.close()
    assert_close(total, full, "k shards summed")


# ------------------------------------------------------------------------------ full-size properties
def test_linearity_at_full_size(F, ctx):
    rows, cols = 17408, 5120
    raw = synth.matrix_on_device(12, rows, cols, seed=5, device="cuda")
    qm = F.QMatrix.from_device_bytes(ctx, raw, 12, rows, cols)
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn((1, cols), device="cuda", generator=g)
    b = torch.randn((1, cols), device="cuda", generator=g)
    ya, yb, yab = qm.matmul(a), qm.matmul(b), qm.matmul(a + 2 * b)
    err = (yab - (ya + 2 * yb)).abs().max().item()
    assert err <= 1e-4 + 1e-3 * yab.abs().max().item()
    # the same rows whatever batch they ride in
    y4 = qm.matmul(torch.cat([a, b, a + 2 * b, a]))
    assert torch.equal(y4[0], y4[3])
    assert (y4[0] - ya[0]).abs().max().item() <= 1e-4 + 1e-3 * ya.abs().max().item()
    qm.close()


def test_launch_counter_counts_native_kernels(F, ctx):
    raw = synth.matrix(12, 32, 256, seed=1)
    qm = F.QMatrix.from_bytes(ctx, raw, 12, 32, 256)
    before = ctx.launches()
    qm.matmul(torch.zeros((1, 256), dtype=torch.float32, device="cuda"))
    assert ctx.launches() - before == 2          # activation preparation + GEMV
    qm.close()


# ------------------------------------------------------------------------------ unit-balanced Q6_K form
@pytest.mark.parametrize("ctas", [1, 3, 7, 0])
def test_q6k_unit_balanced_form(F, ctas, monkeypatch):
    """The Q6_K GEMV in its unit-balanced form: every warp takes an equal run of units, whatever the row tiles; runs
    that start or end inside a row tile leave partial sums that the last warp to arrive adds in warp order.  A forced
    small grid makes small matrices walk all of it: warps spanning several row tiles, row tiles cut into several
    pieces, a tile exactly one warp's run.  Same bar against the oracle, the same bits on every run, close to the
    other form, tickets back at zero (the repeated runs would fail otherwise)."""
    if ctas:
        monkeypatch.setenv("FERRIC_CUDA_GEMV_STREAM_CTAS", str(ctas))
    monkeypatch.setenv("FERRIC_CUDA_GEMV_STREAM", "1")     # opt-in: it measured no faster than the row-tile form
    c = F.Context(0)
    monkeypatch.setenv("FERRIC_CUDA_GEMV_STREAM", "0")
    c_off = F.Context(0)
    shapes = [(200, 1024, 1), (33, 4352, 2), (515, 2048, 5), (1000, 5120, 8), (96, 7168, 3), (16, 256 * 24, 1), (384, 256, 2)]
    if not ctas:
        shapes = [(5120, 17408, 1), (5120, 2304, 2), (4000, 5120, 4)]
    for rows, cols, m in shapes:
        raw = synth.matrix(14, rows, cols, seed=rows + ctas)
        x = synth.activations(m, cols, seed=m)
        xd = torch.from_numpy(x).cuda()
        qm = F.QMatrix.from_bytes(c, raw, 14, rows, cols)
        got = qm.matmul(xd).cpu().numpy()
        ref = O.matmul_q(raw, 14, rows, cols, x, threads=NCPU)
        assert_close(got, ref, f"{rows}x{cols} m{m} ctas{ctas}", exact_product(raw, 14, rows, cols, x))
        for _ in range(3):
            assert np.array_equal(qm.matmul(xd).cpu().numpy(), got)
        q2 = F.QMatrix.from_bytes(c_off, raw, 14, rows, cols)
        other = q2.matmul(xd).cpu().numpy()
        assert np.abs(other - got).max() <= 2e-6 * max(1.0, float(np.abs(ref).max())) + 1e-5 * np.abs(ref).max()
        qm.close()
        q2.close()
    c.close()
    c_off.close()
