"""Vectorised numpy decoders for Q4_K / Q6_K / Q8_0, written independently of ``oracle/ferric_oracle.c``.

They follow the published GGUF K-quant block layouts (the same ones the reference's decoders
implement, crates/ferric-gguf/src/lib.rs:608-615, :721-746, :793-825) with f32 arithmetic in the
reference's operation order, and exist to cross-check the C oracle and to produce golden vectors.
"""
import numpy as np


def _f16(b2: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b2).view(np.float16).astype(np.float32).reshape(-1)


def deq_q8_0(raw: np.ndarray, n: int) -> np.ndarray:
    blk = raw[: n // 32 * 34].reshape(-1, 34)
    d = _f16(blk[:, 0:2])
    q = blk[:, 2:].view(np.int8).astype(np.float32)
    out = np.zeros(n, dtype=np.float32)
    out[: blk.shape[0] * 32] = (q * d[:, None]).reshape(-1)
    return out


def q4k_scales_mins(s: np.ndarray):
    """[n, 12] packed bytes -> ([n, 8] scales, [n, 8] mins)."""
    s = s.astype(np.uint8)
    sc = np.empty((s.shape[0], 8), dtype=np.uint8)
    mn = np.empty((s.shape[0], 8), dtype=np.uint8)
    sc[:, :4] = s[:, 0:4] & 63
    mn[:, :4] = s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 0x0F) | ((s[:, 0:4] >> 6) << 4)
    mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return sc, mn


def deq_q4_k(raw: np.ndarray, n: int) -> np.ndarray:
    blk = raw[: n // 256 * 144].reshape(-1, 144)
    nb = blk.shape[0]
    d, dmin = _f16(blk[:, 0:2]), _f16(blk[:, 2:4])
    sc, mn = q4k_scales_mins(blk[:, 4:16])
    qs = blk[:, 16:].reshape(nb, 4, 32)
    q = np.stack([qs & 0x0F, qs >> 4], axis=2).reshape(nb, 8, 32).astype(np.float32)  # sub-blocks 0..7
    d1 = (d[:, None] * sc.astype(np.float32)).astype(np.float32)
    mm = (dmin[:, None] * mn.astype(np.float32)).astype(np.float32)
    val = ((d1[:, :, None] * q).astype(np.float32) - mm[:, :, None]).astype(np.float32)
    out = np.zeros(n, dtype=np.float32)
    out[: nb * 256] = val.reshape(-1)
    return out


def deq_q6_k(raw: np.ndarray, n: int) -> np.ndarray:
    blk = raw[: n // 256 * 210].reshape(-1, 210)
    nb = blk.shape[0]
    ql = blk[:, 0:128].reshape(nb, 2, 2, 32)       # [half, which 32-run, l]
    qh = blk[:, 128:192].reshape(nb, 2, 32)        # [half, l]
    sc = blk[:, 192:208].view(np.int8).astype(np.float32).reshape(nb, 2, 8)
    d = _f16(blk[:, 208:210])
    out = np.zeros((nb, 2, 4, 32), dtype=np.float32)  # [half, k, l] -> weight 128*half + 32*k + l
    for k in range(4):
        lo = ql[:, :, k & 1, :]
        lo = (lo >> 4) if (k & 2) else (lo & 0x0F)
        hi = (qh >> (2 * k)) & 3
        q = (lo | (hi << 4)).astype(np.int32) - 32
        scale = np.stack([sc[:, :, 2 * k], sc[:, :, 2 * k + 1]], axis=2)  # is = 0, 1
        scale = np.repeat(scale, 16, axis=2)                              # per l
        t = (d[:, None, None] * scale).astype(np.float32)
        out[:, :, k, :] = (t * q.astype(np.float32)).astype(np.float32)
    res = np.zeros(n, dtype=np.float32)
    res[: nb * 256] = out.reshape(-1)
    return res


def deq_raw(raw, n: int, ty: int) -> np.ndarray:
    raw = np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, np.ndarray) else raw.reshape(-1)
    return {8: deq_q8_0, 12: deq_q4_k, 14: deq_q6_k}[ty](raw, n)


def bf16_rne(x: np.ndarray) -> np.ndarray:
    """The reference's add-bias rounding (crates/ferric-tensor/src/dtype.rs:4159-4163) on f32 bit patterns."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFFFFFF
    return (r >> 16).astype(np.uint16)


def deq_q5_k(raw: np.ndarray, n: int) -> np.ndarray:
    """Q5_K: 176-byte blocks [d][dmin][scales 12][qh 32][qs 128]; Q4_K with a fifth bit from qh (bit j of qh[l]
    belongs to value l of sub-block j)."""
    blk = raw[: n // 256 * 176].reshape(-1, 176)
    nb = blk.shape[0]
    d, dmin = _f16(blk[:, 0:2]), _f16(blk[:, 2:4])
    sc, mn = q4k_scales_mins(blk[:, 4:16])
    qh = blk[:, 16:48]                                                      # [nb, 32]
    qs = blk[:, 48:].reshape(nb, 4, 32)
    lo4 = np.stack([qs & 0x0F, qs >> 4], axis=2).reshape(nb, 8, 32)       # sub-blocks 0..7
    bit = ((qh[:, None, :] >> np.arange(8, dtype=np.uint8)[None, :, None]) & 1).astype(np.uint8)
    q = (lo4 + 16 * bit).astype(np.float32)
    d1 = (d[:, None] * sc.astype(np.float32)).astype(np.float32)
    mm = (dmin[:, None] * mn.astype(np.float32)).astype(np.float32)
    val = ((d1[:, :, None] * q).astype(np.float32) - mm[:, :, None]).astype(np.float32)
    out = np.zeros(n, dtype=np.float32)
    out[: nb * 256] = val.reshape(-1)
    return out
