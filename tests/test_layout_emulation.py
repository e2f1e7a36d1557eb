"""CPU emulation of the GEMV kernels' data path: device layout, bit extraction, fragment maps.

The index functions come from the same header the CUDA kernels compile (``csrc/layout.h``, through
a g++ shim), and the bit manipulation below restates the kernels' per-lane code.  The emulated
tensor-core products are checked against the oracle, and every f16 operand the kernels form is
checked to be exact, so a wrong map or an inexact multiplier shows up without a GPU.
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
    for name in ("shim_q4k_unit_offset", "shim_q6k_unit_offset"):
        getattr(lib, name).restype = C.c_uint32
    return lib


def h16(bits):
    """f16 bit pattern -> python float (exact)."""
    return float(np.array([bits & 0xFFFF], dtype=np.uint16).view(np.float16)[0])


def split(v, tail):
    """Head / scaled tail of the activation split, as the prep kernel does it."""
    head = np.float16(np.float32(v))
    if not tail:
        return float(head)
    return float(np.float16(np.float32((np.float32(v) - np.float32(head)) * np.float32(1024.0))))


def is_f16_exact(v):
    return float(np.float16(v)) == float(v)


def prep_block(xb, tail):
    """One (batch row, super-block): returns scaled head-or-tail values per weight, the 2^e factor."""
    amax = float(np.max(np.abs(xb)))
    e = 0
    if amax > 0 and np.isfinite(amax):
        _, e = np.frexp(np.float32(amax))
        e = max(int(e), -100)
    down = np.float32(2.0) ** np.float32(-e)
    xs = (xb.astype(np.float32) * down).astype(np.float32)
    vals = np.array([split(v, tail) for v in xs], dtype=np.float64)
    return vals, xs, float(2.0 ** e)


def byte_of(word, i):
    return (word >> (8 * i)) & 0xFF


def emulate_q4k(shim, raw, cols, x):
    """y[m, 16] for one 16-row tile of raw Q4_K bytes, following gemv_q4k_kernel lane by lane."""
    nblk = cols // 256
    m = x.shape[0]
    raw = raw.reshape(16, nblk, 144)
    unit_bytes = shim.shim_q4k_unit_bytes()
    units = np.zeros((nblk, unit_bytes), dtype=np.uint8)
    for r in range(16):
        for b in range(nblk):
            for byte in range(144):
                units[b, shim.shim_q4k_unit_offset(r, byte)] = raw[r, b, byte]
    acc = np.zeros((16, 8), dtype=np.float64)  # [row, mma column]
    for b in range(nblk):
        u32 = units[b].view(np.uint32)
        cw = np.zeros((16, 8))
        cm = np.zeros((16, 8))
        # B side (prep kernel): column col -> batch col>>1, tail if odd
        bvals, sums, ups = {}, {}, {}
        for col in range(8):
            batch, tail = col >> 1, col & 1
            if batch < m:
                v, xs, up = prep_block(x[batch, b * 256:(b + 1) * 256], tail)
                s32 = [float(np.float32(xs[32 * q:32 * q + 32].sum(dtype=np.float32))) for q in range(8)]
            else:
                v, s32, up = np.zeros(256), [0.0] * 8, 1.0
            bvals[col], ups[batch] = v, up
            sums[col] = [split(s, tail) for s in s32]
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            rows = {}
            for which, r in (("g", g), ("h", g + 8)):
                h = u32[4 * r:4 * r + 4]
                d, dmin = h16(int(h[0]) & 0xFFFF), h16(int(h[0]) >> 16)
                u0, u1, u2 = int(h[1]), int(h[2]), int(h[3])
                sc_lo, m_lo = u0 & 0x3F3F3F3F, u1 & 0x3F3F3F3F
                sc_hi = (u2 & 0x0F0F0F0F) | ((u0 >> 2) & 0x30303030)
                m_hi = ((u2 >> 4) & 0x0F0F0F0F) | ((u1 >> 2) & 0x30303030)
                p = t >> 1
                sc = {(X, n): byte_of(sc_hi if X else sc_lo, 2 * p + n) for X in range(2) for n in range(2)}
                mw = m_lo if t < 2 else m_hi
                mins = (byte_of(mw, 2 * (t & 1)), byte_of(mw, 2 * (t & 1) + 1))
                # the words this lane loaded for row r: segments 2*(r>>3)+X, 16 bytes at lane
                q = [u32[(256 + 512 * (2 * (r >> 3) + X) + 16 * lane) // 4:][:4] for X in range(2)]
                rows[which] = (d, dmin, sc, mins, q)
                # cross-check the scale unpack against the sub-block map
                for X in range(2):
                    for n in range(2):
                        j = shim.shim_q4k_frag_subblock(X, t, n)
                        s12 = raw[r, b, 4:16]
                        ref = (int(s12[j]) & 63) if j < 4 else ((int(s12[j + 4]) & 0x0F) | ((int(s12[j - 4]) >> 6) << 4))
                        assert sc[(X, n)] == ref
            for X in range(2):
                for i in range(4):
                    for n in range(2):
                        s = 8 * X + 2 * i + n
                        mask = 0x00F000F0 if n else 0x000F000F
                        for which, rr in (("g", g), ("h", g + 8)):
                            d, dmin, sc, mins, q = rows[which]
                            a = int(q[X][i])
                            for part, word in ((0, a), (1, a >> 8)):  # regs (k 2t..), (k 2t+8..)
                                v = (word & mask) | 0x64006400
                                mult = sc[(X, n)] / (16.0 if n else 1.0)
                                nbias = -1024.0 * sc[(X, n)] if n == 0 else -64.0 * sc[(X, n)]
                                assert is_f16_exact(mult) and is_f16_exact(nbias)
                                for half in range(2):
                                    av = h16(v >> (16 * half)) * mult + nbias  # fma, exact result below
                                    assert av == int(av) and 0 <= av <= 945 and is_f16_exact(av)
                                    j = 2 * part + half
                                    wgt = shim.shim_q4k_frag_weight(s, t, j)
                                    # the weight this operand must stand for
                                    grp, nn, l = wgt >> 6, (wgt >> 5) & 1, wgt & 31
                                    qb = int(raw[rr, b, 16 + 32 * grp + l])
                                    qq = int((qb >> 4) if nn else (qb & 0xF))
                                    assert av == sc[(X, n)] * qq, (s, t, j, wgt)
                                    for col in range(8):
                                        cw[rr, col] += av * bvals[col][wgt]
            # mins step: k slots 2t, 2t+1 <- sub-blocks 2t, 2t+1
            for which, rr in (("g", g), ("h", g + 8)):
                d, dmin, sc, mins, q = rows[which]
                for col in range(8):
                    cm[rr, col] += mins[0] * sums[col][2 * t] + mins[1] * sums[col][2 * t + 1]
        for r in range(16):
            d, dmin = h16(int(u32[4 * r]) & 0xFFFF), h16(int(u32[4 * r]) >> 16)
            for col in range(8):
                up = ups.get(col >> 1, 1.0)
                acc[r, col] += d * up * cw[r, col] - dmin * up * cm[r, col]
    y = np.zeros((m, 16))
    for batch in range(m):
        y[batch] = acc[:, 2 * batch] + acc[:, 2 * batch + 1] / 1024.0
    return y


def emulate_q6k(shim, raw, cols, x):
    nblk = cols // 256
    m = x.shape[0]
    raw = raw.reshape(16, nblk, 210)
    unit_bytes = shim.shim_q6k_unit_bytes()
    units = np.zeros((nblk, unit_bytes), dtype=np.uint8)
    seen = np.zeros((nblk, unit_bytes), dtype=np.int32)
    for r in range(16):
        for b in range(nblk):
            for byte in range(210):
                off = shim.shim_q6k_unit_offset(r, byte)
                units[b, off] = raw[r, b, byte]
                seen[b, off] += 1
    assert (seen == 1).all()  # the map is a bijection onto the unit
    acc = np.zeros((16, 8))
    for b in range(nblk):
        u8 = units[b]
        u32 = u8.view(np.uint32)
        cw = np.zeros((16, 8))
        cs = np.zeros((16, 8))
        bvals, sums, ups = {}, {}, {}
        for col in range(8):
            batch, tail = col >> 1, col & 1
            if batch < m:
                v, xs, up = prep_block(x[batch, b * 256:(b + 1) * 256], tail)
                s16 = [float(np.float32(xs[16 * q:16 * q + 16].sum(dtype=np.float32))) for q in range(16)]
            else:
                v, s16, up = np.zeros(256), [0.0] * 16, 1.0
            bvals[col], ups[batch] = v, up
            sums[col] = [split(s, tail) for s in s16]
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            for hi8, rr in ((0, g), (1, g + 8)):
                scw = int(u32[(32 + 128 * hi8 + 4 * lane) // 4])
                scs = [np.int8(np.uint8(byte_of(scw, k))).item() for k in range(4)]
                for k in range(4):
                    sb = shim.shim_q6k_frag_subblock(t, k)
                    assert scs[k] == np.int8(raw[rr, b, 192 + sb]).item()
                ql = [u32[(288 + 512 * (2 * hi8 + c) + 16 * lane) // 4:][:4] for c in range(2)]
                qh = u32[(2336 + 512 * hi8 + 16 * lane) // 4:][:4]
                for wi in range(4):
                    hq = int(qh[wi])
                    for c in range(2):
                        lq = int(ql[c][wi])
                        for n in range(2):
                            k = c + 2 * n
                            s = 4 * wi + k
                            m4 = 0x00F000F0 if n else 0x000F000F
                            m2 = 0x00030003 << (2 * k)
                            lo_mult = scs[k] / (16.0 if n else 1.0)
                            hi_mult = scs[k] * 16.0 / (4.0 ** k)
                            assert is_f16_exact(lo_mult) and is_f16_exact(hi_mult)
                            for part in range(2):
                                lw = (lq >> (8 * part)) & m4
                                hw = (hq >> (8 * part)) & m2
                                for half in range(2):
                                    lo_bits, hi_bits = (lw >> (16 * half)) & 0xFFFF, (hw >> (16 * half)) & 0xFFFF
                                    lo_v = h16(lo_bits) * lo_mult  # subnormal * f16, must stay exact
                                    hi_v = h16(hi_bits) * hi_mult
                                    assert is_f16_exact(lo_v) and is_f16_exact(hi_v)
                                    j = 2 * part + half
                                    wgt = shim.shim_q6k_frag_weight(s, t, j)
                                    # reference 6-bit value of that weight
                                    half_ = wgt >> 7
                                    kk, l = (wgt >> 5) & 3, wgt & 31
                                    qlb = int(raw[rr, b, 64 * half_ + 32 * (kk & 1) + l])
                                    lo4 = (qlb >> 4) if (kk & 2) else (qlb & 0xF)
                                    h2 = (int(raw[rr, b, 128 + 32 * half_ + l]) >> (2 * kk)) & 3
                                    is_ = l >> 4
                                    sc_ref = np.int8(raw[rr, b, 192 + 8 * half_ + is_ + 2 * kk]).item()
                                    assert sc_ref == scs[k]
                                    want = sc_ref * (int(lo4) | (int(h2) << 4))
                                    got = (lo_v + hi_v) * 2.0 ** 24
                                    assert got == want, (s, t, j, wgt, got, want)
                                    for col in range(8):
                                        cw[rr, col] += (lo_v + hi_v) * bvals[col][wgt]
                # sums step: slots (2t, 2t+1, 2t+8, 2t+9) <- sub-blocks sb(t, 0..3)
                for col in range(8):
                    for k in range(4):
                        cs[rr, col] += scs[k] * sums[col][shim.shim_q6k_frag_subblock(t, k)]
        for r in range(16):
            g, hi8 = r & 7, r >> 3
            d = h16(int(u32[g]) >> (16 * hi8))
            assert d == O.f16_to_f32(int(raw[r, b, 208]) | (int(raw[r, b, 209]) << 8))
            for col in range(8):
                up = ups.get(col >> 1, 1.0)
                acc[r, col] += d * up * (2.0 ** 24 * cw[r, col] - 32.0 * cs[r, col])
    y = np.zeros((m, 16))
    for batch in range(m):
        y[batch] = acc[:, 2 * batch] + acc[:, 2 * batch + 1] / 1024.0
    return y


def _tol_ok(got, ref):
    return np.all(np.abs(got - ref) <= 1e-4 + 1e-3 * np.abs(ref))


@pytest.mark.parametrize("m", [1, 3])
def test_q4k_kernel_model_matches_oracle(shim, m):
    cols = 512
    raw = np.concatenate([O.q4k_block(7 * i + 1) for i in range(16 * cols // 256)])
    rng = np.random.default_rng(5)
    x = rng.standard_normal((m, cols)).astype(np.float32) * np.float32(3.0)
    y = emulate_q4k(shim, raw, cols, x)
    ref = O.matmul_q(raw, O.GGML_Q4_K, 16, cols, x)
    assert _tol_ok(y, ref), np.abs(y - ref).max()


@pytest.mark.parametrize("m", [1, 4])
def test_q6k_kernel_model_matches_oracle(shim, m):
    cols = 512
    rng = np.random.default_rng(9)
    raw = rng.integers(0, 256, size=16 * (cols // 256) * 210, dtype=np.uint8)
    blocks = raw.reshape(-1, 210)
    blocks[:, 208:210] = np.frombuffer(
        rng.uniform(1e-4, 2e-3, size=blocks.shape[0]).astype(np.float16).tobytes(), dtype=np.uint8).reshape(-1, 2)
    x = rng.standard_normal((m, cols)).astype(np.float32) * np.float32(0.01)
    y = emulate_q6k(shim, raw, cols, x)
    ref = O.matmul_q(raw, O.GGML_Q6_K, 16, cols, x)
    assert _tol_ok(y, ref), np.abs(y - ref).max()


def test_q4k_unit_map_is_a_bijection(shim):
    seen = np.zeros(shim.shim_q4k_unit_bytes(), dtype=np.int32)
    for r in range(16):
        for byte in range(144):
            seen[shim.shim_q4k_unit_offset(r, byte)] += 1
    assert (seen == 1).all()


def test_fragment_maps_cover_each_weight_once(shim):
    for fn in (shim.shim_q4k_frag_weight, shim.shim_q6k_frag_weight):
        seen = np.zeros(256, dtype=np.int32)
        for s in range(16):
            for t in range(4):
                base = fn(s, t, 0)
                assert base % 4 == 0  # the prep kernel reads one aligned float4 per (step, lane)
                assert sorted(fn(s, t, j) - base for j in range(4)) == [0, 1, 2, 3]
                assert [fn(s, t, j) - base for j in range(4)] == [0, 2, 1, 3]
                for j in range(4):
                    seen[fn(s, t, j)] += 1
        assert (seen == 1).all()
