"""Regenerates ``tests/golden/kat.npz``: known-answer vectors for the packed-quant decoders.

    python tests/golden/make_golden.py

The reference (Rust) cannot be built or run in this image, so the vectors come from two sources
that do not pass through the code under test:
  * the reference's own known-answer tests, restated from their text -- the hand-built Q4_K block
    of crates/ferric-gguf/examples/roundtrip.rs:54-87 with the expected values its own formula
    gives, and the f16 specials of crates/ferric-tensor/src/cpu_simd.rs:203-213;
  * the independent numpy decoders in tests/np_decoders.py applied to blocks from the reference's
    fixture generators (q4k_block / q6k_block, crates/ferric-tensor/examples/q4_k.rs:13-37,
    q6_k.rs:9-17, restated here in Python) and to seeded random blocks.
Values are stored as f32 BIT PATTERNS (uint32) so comparisons are exact.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import np_decoders as D  # noqa: E402
from ferric_b200 import synth  # noqa: E402

M32 = 0xFFFFFFFF


def f16_bytes(x: float) -> bytes:
    return np.array([x], dtype=np.float32).astype(np.float16).tobytes()


def q4k_block(seed: int) -> np.ndarray:
    d = np.float32(0.05) + np.float32(0.01) * np.float32(seed % 7)
    dmin = np.float32(0.02) + np.float32(0.005) * np.float32(seed % 5)
    b = bytearray(f16_bytes(d) + f16_bytes(dmin))
    s = [0] * 12
    for j in range(8):
        sc = ((seed * 2654435761 + j * 40503) & M32) % 64
        mn = ((seed * 40503 + j * 2654435761) & M32) % 64
        if j < 4:
            s[j] |= sc & 63
            s[j + 4] |= mn & 63
        else:
            s[j + 4] |= (sc & 0x0F) | ((mn & 0x0F) << 4)
            s[j - 4] |= (sc >> 4) << 6
            s[j] |= (mn >> 4) << 6
    b += bytes(s)
    b += bytes(((seed + i * 2246822519) & M32) % 256 for i in range(128))
    return np.frombuffer(bytes(b), dtype=np.uint8)


def q6k_block(seed: int) -> np.ndarray:
    b = bytearray(210)
    for i in range(128):
        b[i] = ((seed + i * 2246822519) & M32) % 256
    for i in range(64):
        b[128 + i] = ((seed * 40503 + i * 97) & M32) % 256
    for i in range(16):
        b[192 + i] = ((((seed + i * 7) & M32) % 64) - 32) & 0xFF
    d = np.float32(0.04) + np.float32(0.01) * np.float32(seed % 6)
    b[208:210] = f16_bytes(d)
    return np.frombuffer(bytes(b), dtype=np.uint8)


def handbuilt_q4k():
    """roundtrip.rs:54-87: d = 1, dmin = 0, scales[0..8] = 1, qs[i] = (i%8) | (((i+3)%8) << 4)."""
    scales = [1] * 8 + [0] * 4
    qs = [((i % 256) % 8 & 0x0F) | ((((i % 256) + 3) % 8) << 4) for i in range(128)]
    blk = f16_bytes(1.0) + f16_bytes(0.0) + bytes(scales) + bytes(qs)

    def get(j):
        return scales[j] & 63 if j < 4 else (scales[j + 4] & 0x0F) | ((scales[j - 4] >> 6) << 4)

    exp = np.zeros(256, dtype=np.float32)
    y = q = is_ = 0
    for _ in range(4):
        s1, s2 = float(get(is_)), float(get(is_ + 1))
        for l in range(32):
            exp[y + l] = s1 * (qs[q + l] & 0x0F)
            exp[y + l + 32] = s2 * (qs[q + l] >> 4)
        y, q, is_ = y + 64, q + 32, is_ + 2
    return np.frombuffer(blk, dtype=np.uint8), exp


def main():
    rng = np.random.default_rng(20240607)
    hb_raw, hb_exp = handbuilt_q4k()
    q4k_fix = np.concatenate([q4k_block(s) for s in (1, 2, 3, 12345, 0xFFFFFFFF)])
    q6k_fix = np.concatenate([q6k_block(s) for s in (1, 2, 3, 12345, 0xFFFFFFFF)])
    q4k_rand = synth.q4k_blocks(rng, 6).reshape(-1)
    q6k_rand = synth.q6k_blocks(rng, 6).reshape(-1)
    q6k_wild = rng.integers(0, 256, size=4 * 210, dtype=np.uint8)  # full int8 scale range, any f16 d
    q6k_wild.reshape(4, 210)[:, 208:210] = np.array([[0x00, 0x3C], [0x01, 0x00], [0xFF, 0x03], [0x00, 0xBC]],
                                                      dtype=np.uint8)  # 1.0, min subnormal, max subnormal, -1.0
    q8_rand = synth.q8_0_blocks(rng, 12).reshape(-1)
    bf16_in = np.concatenate([rng.standard_normal(64).astype(np.float32) * np.float32(3.0),
                              np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38, 1e-40, -2.5],
                                       dtype=np.float32)])
    out = {
        "f16_bits": np.array([0x0000, 0x3C00, 0xBC00, 0x0001, 0x7C00, 0xFC00, 0x03FF, 0x0400, 0x7BFF], dtype=np.uint16),
        "f16_vals": np.array([0.0, 1.0, -1.0, 5.9604645e-8, np.inf, -np.inf, 6.097555e-05, 6.1035156e-05, 65504.0],
                             dtype=np.float32),
        "handbuilt_q4k_raw": hb_raw, "handbuilt_q4k_expected": hb_exp,
        "q4k_fix_raw": q4k_fix, "q4k_fix_bits": D.deq_q4_k(q4k_fix, 5 * 256).view(np.uint32),
        "q6k_fix_raw": q6k_fix, "q6k_fix_bits": D.deq_q6_k(q6k_fix, 5 * 256).view(np.uint32),
        "q4k_rand_raw": q4k_rand, "q4k_rand_bits": D.deq_q4_k(q4k_rand, 6 * 256).view(np.uint32),
        "q6k_rand_raw": q6k_rand, "q6k_rand_bits": D.deq_q6_k(q6k_rand, 6 * 256).view(np.uint32),
        "q6k_wild_raw": q6k_wild, "q6k_wild_bits": D.deq_q6_k(q6k_wild, 4 * 256).view(np.uint32),
        "q8_rand_raw": q8_rand, "q8_rand_bits": D.deq_q8_0(q8_rand, 12 * 32).view(np.uint32),
        "bf16_in_bits": bf16_in.view(np.uint32), "bf16_out": D.bf16_rne(bf16_in),
    }
    np.savez_compressed(os.path.join(HERE, "kat.npz"), **out)
    print("wrote", os.path.join(HERE, "kat.npz"), {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
