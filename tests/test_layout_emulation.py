"""CPU emulation of the GEMV kernels' data path: device layout, bit extraction, fragment maps.

The index functions come from the same header the CUDA kernels compile (``csrc/layout.h``, through
a g++ shim), and the code below restates, lane by lane, what ``prep_kernel`` and the int8
tensor-core GEMV kernels do.  The emulated products are checked against the oracle, and every
integer operand is checked against the weight / scale it must stand for, so a wrong map shows up
without a GPU.
"""
import ctypes as C
import os
import subprocess
import tempfile

import numpy as np
import pytest

from oracle import oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def shim():
    out = os.path.join(tempfile.mkdtemp(prefix="ferric_shim_"), "layout_shim.so")
    subprocess.check_call(["g++", "-O1", "-shared", "-fPIC", "-o", out, os.path.join(HERE, "cpu", "layout_shim.cpp")])
    lib = C.CDLL(out)
    for name in ("shim_q4k_unit_offset", "shim_q5k_unit_offset", "shim_q6k_unit_offset"):
        getattr(lib, name).restype = C.c_uint32
    return lib


def h16(bits):
    return float(np.array([bits & 0xFFFF], dtype=np.uint16).view(np.float16)[0])


def byte_of(word, i):
    return (int(word) >> (8 * i)) & 0xFF


def s8(b):
    return b - 256 if b >= 128 else b


def prep_row_block(xb):
    """prep_kernel for one (activation row, super-block): limbs [4, 256], 16-weight limb sums, 2^(e-6)."""
    amax = float(np.max(np.abs(xb)))
    e = 0
    if amax > 0 and np.isfinite(amax):
        _, e = np.frexp(np.float32(amax))
        e = min(max(int(e) + 1, -80), 120)
    to_int = np.float32(2.0) ** np.float32(27 - e)
    X = np.rint((xb.astype(np.float32) * to_int).astype(np.float32)).astype(np.int64)
    assert np.abs(X).max() <= 2 ** 27
    limbs = np.zeros((4, 256), dtype=np.int64)
    for j in (3, 2, 1):
        a = ((X + 64) & 127) - 64
        limbs[j] = a
        X = (X - a) >> 7
    limbs[0] = X
    assert np.abs(limbs).max() <= 64
    sums16 = limbs.reshape(4, 16, 16).sum(axis=2)
    return limbs, sums16, float(2.0 ** (e - 6))


def split_sum(S):
    s0 = ((S + 64) & 127) - 64
    s1 = (S - s0) >> 7
    assert -128 <= s0 < 128 and -128 <= s1 < 128 and 128 * s1 + s0 == S
    return s0, s1


def recombine(acc, m):
    """acc[16 rows, 8 columns] -> y[m, 16]: column 4*(row in tile) + limb, weight 2^(-7 limb)."""
    y = np.zeros((m, 16))
    for batch in range(m):
        for j in range(4):
            y[batch] += acc[:, 4 * batch + j] * 2.0 ** (-7 * j)
    return y


def emulate_q4k(shim, raw, cols, x):
    """y[m <= 2, 16] for one 16-row tile of raw Q4_K bytes, following gemv_q4k_kernel lane by lane."""
    nblk, m = cols // 256, x.shape[0]
    raw = raw.reshape(16, nblk, 144)
    units = np.zeros((nblk, shim.shim_q4k_unit_bytes()), dtype=np.uint8)
    seen = np.zeros(units.shape, dtype=np.int32)
    for r in range(16):
        for b in range(nblk):
            for byte in range(144):
                off = shim.shim_q4k_unit_offset(r, byte)
                units[b, off] = raw[r, b, byte]
                seen[b, off] += 1
    assert (seen == 1).all()
    acc = np.zeros((16, 8))
    for b in range(nblk):
        u32 = units[b].view(np.uint32)
        limbs, sums, ups = {}, {}, {}
        for brow in range(2):
            if brow < m:
                limbs[brow], s16, ups[brow] = prep_row_block(x[brow, b * 256:(b + 1) * 256])
                sums[brow] = s16.reshape(4, 8, 2).sum(axis=2)        # 32-weight sub-blocks
            else:
                limbs[brow], sums[brow], ups[brow] = np.zeros((4, 256), np.int64), np.zeros((4, 8), np.int64), 1.0
        ai = np.zeros((16, 8), dtype=np.int64)
        cm = np.zeros((16, 8), dtype=np.int64)
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            for hi8, rr in ((0, g), (1, g + 8)):
                h = u32[4 * rr:4 * rr + 4]
                u0, u1, u2 = int(h[1]), int(h[2]), int(h[3])
                sc_lo, m_lo = u0 & 0x3F3F3F3F, u1 & 0x3F3F3F3F
                sc_hi = (u2 & 0x0F0F0F0F) | ((u0 >> 2) & 0x30303030)
                m_hi = ((u2 >> 4) & 0x0F0F0F0F) | ((u1 >> 2) & 0x30303030)
                s12 = [int(v) for v in raw[rr, b, 4:16]]
                for p in range(4):
                    q = u32[(256 + 512 * (2 * hi8 + (p >> 1)) + 16 * lane) // 4:][:4]
                    w = [int(q[2 * (p & 1)]), int(q[2 * (p & 1) + 1])]
                    for n in range(2):
                        s = 2 * p + n
                        sc = byte_of(sc_lo if s < 4 else sc_hi, s & 3)
                        ref_sc = (s12[s] & 63) if s < 4 else ((s12[s + 4] & 0x0F) | ((s12[s - 4] >> 6) << 4))
                        assert sc == ref_sc
                        for part in range(2):          # a0/a1 (k 4t..) then a2/a3 (k 16+4t..)
                            a = ((w[part] >> 4) if n else w[part]) & 0x0F0F0F0F
                            for j in range(4):
                                i = 4 * part + j
                                wgt = shim.shim_q4k_frag_weight(s, t, i)
                                grp, nn, l = wgt >> 6, (wgt >> 5) & 1, wgt & 31
                                qb = int(raw[rr, b, 16 + 32 * grp + l])
                                assert byte_of(a, j) == ((qb >> 4) if nn else (qb & 0xF)), (s, t, i, wgt)
                                for col in range(8):
                                    ai[rr, col] += sc * byte_of(a, j) * limbs[col >> 2][col & 3][wgt]
                # mins step: k slot 4t+i <-> sub-block 4t+i, lanes t >= 2 contribute zeros
                mw = m_lo if t == 0 else m_hi if t == 1 else 0
                for i in range(4):
                    sb = 4 * t + i
                    if sb < 8:
                        ref_m = (s12[sb + 4] & 63) if sb < 4 else ((s12[sb + 4] >> 4) | ((s12[sb] >> 6) << 4))
                        assert byte_of(mw, i) == ref_m
                    for col in range(8):
                        S = int(sums[col >> 2][col & 3][sb]) if sb < 8 else 0
                        s0, s1 = split_sum(S)
                        cm[rr, col] += byte_of(mw, i) * (s0 + 128 * s1)
        for r in range(16):
            d, dmin = h16(int(u32[4 * r]) & 0xFFFF), h16(int(u32[4 * r]) >> 16)
            for col in range(8):
                up = ups[col >> 2]
                acc[r, col] += d * up * float(ai[r, col]) - dmin * up * float(cm[r, col])
    return recombine(acc, m)


def emulate_q6k(shim, raw, cols, x):
    nblk, m = cols // 256, x.shape[0]
    raw = raw.reshape(16, nblk, 210)
    units = np.zeros((nblk, shim.shim_q6k_unit_bytes()), dtype=np.uint8)
    seen = np.zeros(units.shape, dtype=np.int32)
    for r in range(16):
        for b in range(nblk):
            for byte in range(210):
                off = shim.shim_q6k_unit_offset(r, byte)
                units[b, off] = raw[r, b, byte]
                seen[b, off] += 1
    assert (seen == 1).all()
    acc = np.zeros((16, 8))
    for b in range(nblk):
        u8 = units[b]
        u32 = u8.view(np.uint32)
        limbs, sums, ups = {}, {}, {}
        for brow in range(2):
            if brow < m:
                limbs[brow], sums[brow], ups[brow] = prep_row_block(x[brow, b * 256:(b + 1) * 256])
            else:
                limbs[brow], sums[brow], ups[brow] = np.zeros((4, 256), np.int64), np.zeros((4, 16), np.int64), 1.0
        ai = np.zeros((16, 8), dtype=np.int64)
        co = np.zeros((16, 8), dtype=np.int64)
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            for hi8, rr in ((0, g), (1, g + 8)):
                scrow = u8[32 + 16 * rr:32 + 16 * rr + 16]
                assert (scrow == raw[rr, b, 192:208]).all()
                ql = [u32[(288 + 512 * (2 * hi8 + c) + 16 * lane) // 4:][:4] for c in range(2)]
                qh = u32[(2336 + 512 * hi8 + 16 * lane) // 4:][:4]
                for h in range(2):
                    for k in range(4):
                        for is_ in range(2):
                            wi, sb = 2 * h + is_, 8 * h + 2 * k + is_
                            lw, hw = int(ql[k & 1][wi]), int(qh[wi])
                            lo = ((lw >> 4) if (k & 2) else lw) & 0x0F0F0F0F
                            hs = [(hw << 4), (hw << 2), hw, (hw >> 2)][k] & 0x30303030
                            a = lo | hs
                            sc = s8(int(scrow[sb]))
                            for j in range(4):
                                wgt = shim.shim_q6k_frag_weight(sb, t, j)
                                half_, kk, l = wgt >> 7, (wgt >> 5) & 3, wgt & 31
                                assert (half_, kk, l >> 4) == (h, k, is_)
                                qlb = int(raw[rr, b, 64 * half_ + 32 * (kk & 1) + l])
                                lo4 = (qlb >> 4) if (kk & 2) else (qlb & 0xF)
                                h2 = (int(raw[rr, b, 128 + 32 * half_ + l]) >> (2 * kk)) & 3
                                assert byte_of(a, j) == (lo4 | (h2 << 4)), (sb, t, j, wgt)
                                assert sc == s8(int(raw[rr, b, 192 + 8 * half_ + (l >> 4) + 2 * kk]))
                                for col in range(8):
                                    ai[rr, col] += sc * byte_of(a, j) * limbs[col >> 2][col & 3][wgt]
                # offset step: k slot 4t+i <-> sub-block 4t+i, A = the raw scale bytes
                for i in range(4):
                    sb = 4 * t + i
                    for col in range(8):
                        s0, s1 = split_sum(int(sums[col >> 2][col & 3][sb]))
                        co[rr, col] += s8(int(scrow[sb])) * (s0 + 128 * s1)
        for r in range(16):
            g, hi8 = r & 7, r >> 3
            d = h16(int(u32[g]) >> (16 * hi8))
            assert d == O.f16_to_f32(int(raw[r, b, 208]) | (int(raw[r, b, 209]) << 8))
            for col in range(8):
                acc[r, col] += d * ups[col >> 2] * float(ai[r, col] - 32 * co[r, col])
    return recombine(acc, m)


def _tol_ok(got, ref):
    return np.all(np.abs(got - ref) <= 1e-4 + 1e-3 * np.abs(ref))


@pytest.mark.parametrize("m", [1, 2])
def test_q4k_kernel_model_matches_oracle(shim, m):
    cols = 512
    raw = np.concatenate([O.q4k_block(7 * i + 1) for i in range(16 * cols // 256)])
    rng = np.random.default_rng(5)
    x = rng.standard_normal((m, cols)).astype(np.float32) * np.float32(3.0)
    y = emulate_q4k(shim, raw, cols, x)
    ref = O.matmul_q(raw, O.GGML_Q4_K, 16, cols, x)
    assert _tol_ok(y, ref), np.abs(y - ref).max()
    exact = x.astype(np.float64) @ O.deq_raw(raw, 16 * cols, 12).reshape(16, cols).astype(np.float64).T
    assert np.abs(y - exact).max() < 2e-6 * np.abs(exact).max()      # limbs carry f32-level accuracy


@pytest.mark.parametrize("m", [1, 2])
def test_q6k_kernel_model_matches_oracle(shim, m):
    cols = 512
    rng = np.random.default_rng(9)
    raw = rng.integers(0, 256, size=16 * (cols // 256) * 210, dtype=np.uint8)   # full int8 scale range
    blocks = raw.reshape(-1, 210)
    blocks[:, 208:210] = np.frombuffer(
        rng.uniform(1e-4, 2e-3, size=blocks.shape[0]).astype(np.float16).tobytes(), dtype=np.uint8).reshape(-1, 2)
    x = rng.standard_normal((m, cols)).astype(np.float32) * np.float32(0.01)
    y = emulate_q6k(shim, raw, cols, x)
    ref = O.matmul_q(raw, O.GGML_Q6_K, 16, cols, x)
    assert _tol_ok(y, ref), np.abs(y - ref).max()
    exact = x.astype(np.float64) @ O.deq_raw(raw, 16 * cols, 14).reshape(16, cols).astype(np.float64).T
    assert np.abs(y - exact).max() < 2e-6 * np.abs(exact).max()


def test_limb_split_is_exact_for_the_blocks_largest_values():
    rng = np.random.default_rng(3)
    for scale in (1e-6, 1.0, 3e4, 1e10):
        xb = (rng.standard_normal(256) * scale).astype(np.float32)
        xb[7] = np.float32(0.0)
        limbs, sums16, up = prep_row_block(xb)
        X = limbs[0] * 2 ** 21 + limbs[1] * 2 ** 14 + limbs[2] * 2 ** 7 + limbs[3]
        back = X.astype(np.float64) * up * 2.0 ** -21
        assert np.abs(back - xb.astype(np.float64)).max() <= np.abs(xb).max() * 2.0 ** -26
        assert (sums16 == limbs.reshape(4, 16, 16).sum(axis=2)).all()


def test_fragment_maps_cover_each_weight_once(shim):
    seen = np.zeros(256, dtype=np.int32)
    for s in range(8):
        for t in range(4):
            assert [shim.shim_q4k_frag_weight(s, t, i) for i in range(8)] == list(range(32 * s + 8 * t, 32 * s + 8 * t + 8))
            for i in range(8):
                seen[shim.shim_q4k_frag_weight(s, t, i)] += 1
    assert (seen == 1).all()
    seen[:] = 0
    for sb in range(16):
        for t in range(4):
            for i in range(4):
                seen[shim.shim_q6k_frag_weight(sb, t, i)] += 1
    assert (seen == 1).all()


def test_q5k_unit_layout(shim):
    """The Q5_K unit is a bijection of 16 rows x 176 block bytes onto 2816 bytes; header and nibbles sit where the Q4_K
    unit has them, and lane 4g + t of the fifth-bit segment holds qh[8t .. 8t+8) of rows g and g + 8 -- the bits of the
    very weights (8t .. 8t+7 of every sub-block) whose nibbles the lane owns."""
    n = shim.shim_q5k_unit_bytes()
    assert n == 16 * 176
    seen = np.zeros(n, dtype=np.int32)
    for r in range(16):
        for byte in range(176):
            seen[shim.shim_q5k_unit_offset(r, byte)] += 1
    assert (seen == 1).all()
    for r in range(16):
        for byte in range(16):
            assert shim.shim_q5k_unit_offset(r, byte) == shim.shim_q4k_unit_offset(r, byte)
        for byte in range(128):
            assert shim.shim_q5k_unit_offset(r, 48 + byte) == shim.shim_q4k_unit_offset(r, 16 + byte)
        g, hi = r & 7, r >> 3
        for l in range(32):
            t, j = l >> 3, l & 7
            assert shim.shim_q5k_unit_offset(r, 16 + l) == 2304 + 16 * (4 * g + t) + 8 * hi + j
