"""Pins the CPU oracle: the reference's own known-answer tests, the committed golden vectors, and an
independently written numpy decoder.  No GPU needed."""
import os

import numpy as np
import pytest

import np_decoders as D
from ferric_b200 import synth
from oracle import oracle as O

KAT = np.load(os.path.join(os.path.dirname(__file__), "golden", "kat.npz"))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


# ---- crates/ferric-tensor/src/cpu_simd.rs:203-213 --------------------------------------------
def test_f16_decodes_subnormals_and_specials():
    assert O.f16_to_f32(0x0000) == 0.0
    assert O.f16_to_f32(0x3C00) == 1.0
    assert O.f16_to_f32(0xBC00) == -1.0
    assert abs(O.f16_to_f32(0x0001) - 5.9604645e-8) < 1e-14
    assert np.isinf(O.f16_to_f32(0x7C00))
    assert np.isinf(O.f16_to_f32(0xFC00)) and O.f16_to_f32(0xFC00) < 0
    assert np.isnan(O.f16_to_f32(0x7E00))
    for b, v in zip(KAT["f16_bits"], KAT["f16_vals"]):
        assert np.float32(O.f16_to_f32(int(b))) == v


def test_f16_decode_matches_numpy_on_every_bit_pattern():
    allb = np.arange(65536, dtype=np.uint16)
    want = allb.view(np.float16).astype(np.float32)
    got = np.array([O.f16_to_f32(int(b)) for b in allb], dtype=np.float32)
    nan = np.isnan(want)
    assert (np.isnan(got) == nan).all()
    assert (bits(got)[~nan] == bits(want)[~nan]).all()


def test_f16_encode_round_trips():
    vals = np.random.default_rng(1).standard_normal(2000).astype(np.float32) * np.float32(10)
    for v in list(vals) + [0.05, 0.06, 65504.0, 1e-7, 6e-8, 0.0]:
        assert O.f32_to_f16(v) == int(np.array([v], dtype=np.float32).astype(np.float16).view(np.uint16)[0])


# ---- crates/ferric-tensor/src/dtype.rs:4159-4163, examples/dtypes.rs:29-32 -------------------
def test_bf16_rne_matches_golden_and_torch():
    import torch

    x = KAT["bf16_in_bits"].view(np.float32)
    got = np.array([O.bf16_rne(v) for v in x], dtype=np.uint16)
    assert (got == KAT["bf16_out"]).all()
    t = torch.from_numpy(x.copy()).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert (got == t).all()  # the bias rule equals IEEE round-to-nearest-even on finite values


# ---- crates/ferric-gguf/src/lib.rs:471-494, dtype.rs:873-889 ---------------------------------
def test_type_size_and_block_bytes():
    assert O.type_size(O.GGML_Q4_K, 4096 * 4096) == 9_437_184
    assert O.type_size(O.GGML_Q6_K, 151936 * 5120) == 638_131_200
    assert O.type_size(O.GGML_Q8_0, 64) == 68
    assert O.type_size(O.GGML_F32, 8) == 32 and O.type_size(O.GGML_F16, 8) == 16 and O.type_size(O.GGML_BF16, 8) == 16
    with pytest.raises(O.OracleError):
        O.type_size(99, 256)
    assert O.block_bytes(8) == (32, 34) and O.block_bytes(12) == (256, 144) and O.block_bytes(14) == (256, 210)
    assert O.block_bytes(0) is None and O.block_bytes(23) is None


def test_deq_raw_rejects_unknown_type_and_short_buffer():
    with pytest.raises(O.OracleError) as e:
        O.deq_raw(np.zeros(144, np.uint8), 256, 99)
    assert e.value.code == O.FO_ERR_TYPE
    with pytest.raises(O.OracleError) as e:
        O.deq_raw(np.zeros(100, np.uint8), 256, O.GGML_Q4_K)
    assert e.value.code == O.FO_ERR_SHAPE


# ---- crates/ferric-gguf/examples/roundtrip.rs:54-87 ------------------------------------------
def test_handbuilt_q4k_block():
    got = O.deq_raw(KAT["handbuilt_q4k_raw"], 256, O.GGML_Q4_K)
    assert np.abs(got - KAT["handbuilt_q4k_expected"]).max() < 1e-3  # the reference's own bound
    assert (got == KAT["handbuilt_q4k_expected"]).all()               # and in fact exact


# ---- golden vectors (bit patterns) -----------------------------------------------------------
@pytest.mark.parametrize("name,ty,vals", [("q4k_fix", 12, 256), ("q4k_rand", 12, 256), ("q6k_fix", 14, 256),
                                          ("q6k_rand", 14, 256), ("q6k_wild", 14, 256), ("q8_rand", 8, 32)])
def test_decoders_match_golden_bits(name, ty, vals):
    raw, want = KAT[name + "_raw"], KAT[name + "_bits"]
    got = O.deq_raw(raw, want.size, ty)
    assert (bits(got) == want).all()
    gb = O.deq_raw_bf16(raw, want.size, ty)
    assert (gb == D.bf16_rne(want.view(np.float32))).all()


def test_fixture_generators_match_golden_bytes():
    assert (np.concatenate([O.q4k_block(s) for s in (1, 2, 3, 12345, 0xFFFFFFFF)]) == KAT["q4k_fix_raw"]).all()
    assert (np.concatenate([O.q6k_block(s) for s in (1, 2, 3, 12345, 0xFFFFFFFF)]) == KAT["q6k_fix_raw"]).all()


@pytest.mark.parametrize("ty", [8, 12, 14])
def test_decoders_match_numpy_on_random_blocks(ty):
    raw = synth.matrix(ty, 8, 1024, seed=ty)
    n = 8 * 1024
    assert (bits(O.deq_raw(raw, n, ty)) == bits(D.deq_raw(raw, n, ty))).all()
    # fully random bytes: every scale value, subnormal / large f16 d (skip blocks whose d is inf/nan)
    rng = np.random.default_rng(100 + ty)
    _, bb = synth.BLOCK[ty]
    raw = rng.integers(0, 256, size=64 * bb, dtype=np.uint8)
    n = 64 * synth.BLOCK[ty][0]
    a, b = O.deq_raw(raw, n, ty), D.deq_raw(raw, n, ty)
    ok = np.isfinite(b)
    assert (bits(a)[ok] == bits(b)[ok]).all() and (np.isfinite(a) == ok).all()


# ---- crates/ferric-gguf/examples/roundtrip.rs:13-16,47-52 ------------------------------------
def test_q8_0_quantise_round_trip():
    w = np.sin(np.arange(64, dtype=np.float32) * np.float32(0.3) + np.float32(2.0)).astype(np.float32)
    raw = O.quant_q8_0(w)
    assert raw.size == 68
    d = O.deq_raw(raw, 64, O.GGML_Q8_0)
    assert np.abs(d - w).max() / max(np.abs(w).max(), 1e-6) < 0.02


# ---- crates/ferric-tensor/examples/q4_k.rs:43-56, q6_k.rs:22-35, q8_0.rs:10-23 ---------------
def _x_cos(m, k):
    return np.cos(np.arange(m * k, dtype=np.float32) * np.float32(0.013)).astype(np.float32).reshape(m, k)


@pytest.mark.parametrize("ty,shapes", [(12, [(8, 256, 4), (13, 512, 1), (256, 2048, 1)]),
                                       (14, [(8, 256, 4), (7, 512, 1), (128, 1024, 1)]),
                                       (8, [(8, 256, 4), (13, 128, 1), (256, 2048, 1)])])
def test_packed_orders_agree_with_dequant_then_dot(ty, shapes):
    for rows, k, m in shapes:
        if ty == 12:
            raw = np.concatenate([O.q4k_block(i + 1) for i in range(rows * k // 256)])
        elif ty == 14:
            raw = np.concatenate([O.q6k_block(i + 1) for i in range(rows * k // 256)])
        else:
            w = (np.sin(np.arange(rows * k, dtype=np.float32) * np.float32(0.021)) * np.float32(0.7)).astype(np.float32)
            raw = np.concatenate([O.quant_q8_0(w[r * k:(r + 1) * k]) for r in range(rows)])
        x = _x_cos(m, k)
        ref = O.matmul_q(raw, ty, rows, k, x, mode=O.MODE_DEQUANT_DOT)
        # the literal reference: deq_raw -> matmul_bt
        wdq = O.deq_raw(raw, rows * k, ty).reshape(rows, k)
        assert (bits(ref) == bits(O.matmul_bt(x, wdq))).all()
        scale = max(np.abs(ref).max(), 1e-3)
        for mode in (O.MODE_FUSED, O.MODE_SHADER):
            got = O.matmul_q(raw, ty, rows, k, x, mode=mode)
            assert np.abs(got - ref).max() / scale < 1e-5, (ty, rows, k, m, mode)


# ---- crates/ferric-tensor/src/cpu_simd.rs:162-200 --------------------------------------------
def test_q8_0_matvec_matches_exact_values():
    for rows, cols in [(1, 32), (8, 64), (17, 256), (64, 512)]:
        raw, vals = O.q8_0_synth(rows, cols, rows * 13 + cols)
        x = ((np.arange(cols) * 37 % 101).astype(np.float32) - np.float32(50.0)) / np.float32(50.0)
        got = O.matmul_q(raw, 8, rows, cols, x, mode=O.MODE_FUSED)[0]
        want = (vals.reshape(rows, cols).astype(np.float64) @ x.astype(np.float64))
        scale = max(np.abs(want).max(), 1e-6)
        assert np.abs(got - want).max() / scale < 1e-5
        assert (bits(O.deq_raw(raw, rows * cols, 8)) == bits(vals)).all()


@pytest.mark.parametrize("ty", [8, 12, 14])
def test_threading_changes_nothing_about_the_answer(ty):
    raw = synth.matrix(ty, 64, 256, seed=7)
    x = np.sin(np.arange(256, dtype=np.float32) * np.float32(0.01))
    for mode in (O.MODE_DEQUANT_DOT, O.MODE_FUSED):
        one = O.matmul_q(raw, ty, 64, 256, x, threads=1, mode=mode)
        for t in (2, 3, 8, 64, 128):
            assert (bits(O.matmul_q(raw, ty, 64, 256, x, threads=t, mode=mode)) == bits(one)).all()


@pytest.mark.parametrize("ty", [8, 12, 14])
def test_spans_concatenate_to_the_whole(ty):
    raw = synth.matrix(ty, 40, 256, seed=3)
    x = ((np.arange(256) % 7).astype(np.float32)) - np.float32(3.0)
    whole = O.matmul_q(raw, ty, 40, 256, x, mode=O.MODE_FUSED)[0]
    for cut in (0, 1, 17, 39, 40):
        joined = np.concatenate([O.matvec_span(raw, ty, 40, 256, x, 0, cut, 2), O.matvec_span(raw, ty, 40, 256, x, cut, 40, 2)])
        assert (bits(joined) == bits(whole)).all()


def test_shape_errors_are_reported():
    raw = synth.matrix(12, 4, 256, seed=1)
    with pytest.raises(O.OracleError) as e:
        O.matmul_q(raw[:-1], 12, 4, 256, np.zeros(256, np.float32))
    assert e.value.code == O.FO_ERR_SHAPE
    with pytest.raises(O.OracleError):
        O.matmul_q(raw, 12, 4, 128, np.zeros(128, np.float32))   # cols not a multiple of 256
    with pytest.raises(O.OracleError):
        O.matmul_q(raw, 2, 4, 256, np.zeros(256, np.float32))    # no packed kernel for this type
    with pytest.raises(O.OracleError):
        O.matmul_q(raw, 12, 4, 256, np.zeros(512, np.float32))   # inner dim mismatch


def test_swiglu_and_bf16_product():
    rng = np.random.default_rng(4)
    gu = rng.standard_normal((3, 64)).astype(np.float32)
    out = O.swiglu(gu, 32)
    g, u = gu[:, :32].astype(np.float64), gu[:, 32:].astype(np.float64)
    assert np.allclose(out, g / (1 + np.exp(-g)) * u, rtol=1e-6, atol=1e-7)
    raw = synth.matrix(12, 16, 512, seed=5)
    xb = D.bf16_rne(rng.standard_normal((2, 512)).astype(np.float32))
    y = O.matmul_q(raw, 12, 16, 512, xb, mode=O.MODE_BF16)
    w = (D.bf16_rne(O.deq_raw(raw, 16 * 512, 12)).astype(np.uint32) << 16).view(np.float32).reshape(16, 512)
    xf = (xb.astype(np.uint32) << 16).view(np.float32)
    assert np.allclose(y, xf.astype(np.float64) @ w.astype(np.float64).T, rtol=1e-4, atol=1e-4)


# ------------------------------------------------------------------------------ Q5_K
# The reference holds no known-answer vector for Q5_K (its only check is fused-vs-unfused agreement,
# crates/ferric-tensor/examples/ffn_fuse.rs:100-108).  The oracle's decoder (restated from
# crates/ferric-gguf/src/lib.rs:690-716) is held against an independent numpy restatement and a hand-built block in the
# style of the reference's Q4_K one (crates/ferric-gguf/examples/roundtrip.rs:54-87).
def test_q5k_oracle_matches_independent_decoder_bit_for_bit():
    rng = np.random.default_rng(50)
    raw = synth.q5k_blocks(rng, 97).reshape(-1)
    n = 97 * 256
    assert O.type_size(13, n) == raw.size == 97 * 176
    assert np.array_equal(O.deq_raw(raw, n, 13).view(np.uint32), D.deq_q5_k(raw, n).view(np.uint32))
    wild = rng.integers(0, 256, size=40 * 176, dtype=np.uint8)          # any bytes: every (scale, min, bit) pattern
    wild.reshape(-1, 176)[:, 0:4] = synth.q5k_blocks(rng, 40)[:, 0:4]    # keep d, dmin finite
    assert np.array_equal(O.deq_raw(wild, 40 * 256, 13).view(np.uint32), D.deq_q5_k(wild, 40 * 256).view(np.uint32))


def test_q5k_hand_built_block():
    blk = np.zeros(176, dtype=np.uint8)
    blk[0:2] = np.array([1.0], dtype=np.float16).view(np.uint8)         # d = 1
    blk[2:4] = 0                                                         # dmin = 0
    sc = np.arange(1, 9)                                                 # scale of sub-block j = j + 1
    blk[4:16] = synth.pack_q4k_scales(sc[None, :], np.zeros((1, 8), dtype=np.int64))[0]
    i = np.arange(128)
    blk[48:176] = ((i % 8) | (((i + 3) % 8) << 4)).astype(np.uint8)
    blk[16:48] = (np.arange(32) * 37 + 5).astype(np.uint8)               # fifth bits
    got = O.deq_raw(blk, 256, 13)
    want = np.empty(256, dtype=np.float32)
    for grp in range(4):
        for l in range(32):
            b = int(blk[48 + 32 * grp + l])
            qh = int(blk[16 + l])
            want[64 * grp + l] = (grp * 2 + 1) * ((b & 15) + 16 * ((qh >> (2 * grp)) & 1))
            want[64 * grp + 32 + l] = (grp * 2 + 2) * ((b >> 4) + 16 * ((qh >> (2 * grp + 1)) & 1))
    assert np.array_equal(got, want)


def test_q5k_product_modes_and_sizes():
    rows, cols = 9, 512
    raw = synth.matrix(13, rows, cols, seed=3)
    x = synth.activations(2, cols, seed=4)
    w = O.deq_raw(raw, rows * cols, 13).reshape(rows, cols)
    ref = np.empty((2, rows), dtype=np.float32)
    for t in range(2):
        for r in range(rows):
            acc = np.float32(0)
            for c in range(cols):
                acc = np.float32(acc + np.float32(x[t, c] * w[r, c]))
            ref[t, r] = acc
    assert np.array_equal(O.matmul_q(raw, 13, rows, cols, x), ref)
    assert np.array_equal(O.matmul_q(raw, 13, rows, cols, x, threads=3), ref)
    assert O.block_bytes(13) == (256, 176)
