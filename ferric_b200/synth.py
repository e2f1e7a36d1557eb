"""Seeded synthetic GGUF block generators for the benchmark and parity configurations.

The reference measures on Qwen / Bonsai GGUF checkpoints that are not available offline; these
generators produce valid Q4_K / Q6_K / Q8_0 block bytes with those models' shapes and the value
distributions the benchmark configurations name: d, dmin ~ U(1e-4, 2e-3) rounded to f16; 6-bit
scales and mins ~ U{0..63}, packed with the 12-byte encoder the reference's own test fixtures use
(crates/ferric-tensor/examples/q4_k.rs:19-33); 4-bit quants ~ U{0..15}; Q6_K high bits ~ U{0..3}
and int8 scales ~ U{-32..31}; activations ~ N(0, 1).
"""
from __future__ import annotations

import numpy as np

GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = 8, 12, 14
GGML_Q5_K = 13
BLOCK = {GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144), GGML_Q5_K: (256, 176), GGML_Q6_K: (256, 210)}


def _f16_bytes(rng: np.random.Generator, n: int, lo: float = 1e-4, hi: float = 2e-3) -> np.ndarray:
    return rng.uniform(lo, hi, size=n).astype(np.float32).astype(np.float16).view(np.uint8).reshape(n, 2)


def pack_q4k_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """[n, 8] six-bit scales and mins -> [n, 12] bytes in the GGUF K-quant packing."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    s = np.zeros((sc.shape[0], 12), dtype=np.uint8)
    s[:, 0:4] = sc[:, 0:4] & 63
    s[:, 4:8] = mn[:, 0:4] & 63
    s[:, 8:12] = (sc[:, 4:8] & 0x0F) | ((mn[:, 4:8] & 0x0F) << 4)
    s[:, 0:4] |= (sc[:, 4:8] >> 4) << 6
    s[:, 4:8] |= (mn[:, 4:8] >> 4) << 6
    return s


def q4k_blocks(rng: np.random.Generator, nblk: int) -> np.ndarray:
    out = np.empty((nblk, 144), dtype=np.uint8)
    out[:, 0:2] = _f16_bytes(rng, nblk)
    out[:, 2:4] = _f16_bytes(rng, nblk)
    out[:, 4:16] = pack_q4k_scales(rng.integers(0, 64, size=(nblk, 8)), rng.integers(0, 64, size=(nblk, 8)))
    q = rng.integers(0, 16, size=(nblk, 256), dtype=np.uint8).reshape(nblk, 4, 2, 32)
    out[:, 16:144] = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).reshape(nblk, 128)
    return out


def q5k_blocks(rng: np.random.Generator, nblk: int) -> np.ndarray:
    """Q5_K: the Q4_K header and nibbles plus 32 bytes whose bit j is the fifth bit of value l of sub-block j."""
    out = np.empty((nblk, 176), dtype=np.uint8)
    q4 = q4k_blocks(rng, nblk)
    out[:, 0:16] = q4[:, 0:16]
    out[:, 16:48] = rng.integers(0, 256, size=(nblk, 32), dtype=np.uint8)
    out[:, 48:176] = q4[:, 16:144]
    return out


def q6k_blocks(rng: np.random.Generator, nblk: int) -> np.ndarray:
    out = np.empty((nblk, 210), dtype=np.uint8)
    lo = rng.integers(0, 16, size=(nblk, 2, 128), dtype=np.uint8)
    out[:, 0:128] = lo[:, 0, :] | (lo[:, 1, :] << 4)
    hi = rng.integers(0, 4, size=(nblk, 4, 64), dtype=np.uint8)
    out[:, 128:192] = hi[:, 0] | (hi[:, 1] << 2) | (hi[:, 2] << 4) | (hi[:, 3] << 6)
    out[:, 192:208] = rng.integers(-32, 32, size=(nblk, 16)).astype(np.int8).view(np.uint8)
    out[:, 208:210] = _f16_bytes(rng, nblk)
    return out


def q8_0_blocks(rng: np.random.Generator, nblk: int) -> np.ndarray:
    out = np.empty((nblk, 34), dtype=np.uint8)
    out[:, 0:2] = _f16_bytes(rng, nblk)
    out[:, 2:34] = rng.integers(-127, 128, size=(nblk, 32)).astype(np.int8).view(np.uint8)
    return out


def matrix(ggml_type: int, rows: int, cols: int, seed: int) -> np.ndarray:
    """Raw GGUF block bytes of a [rows, cols] weight, row-major [out, in]."""
    vals, _ = BLOCK[ggml_type]
    assert cols % vals == 0
    rng = np.random.default_rng(seed)
    nblk = rows * (cols // vals)
    gen = {GGML_Q4_K: q4k_blocks, GGML_Q5_K: q5k_blocks, GGML_Q6_K: q6k_blocks, GGML_Q8_0: q8_0_blocks}[ggml_type]
    return gen(rng, nblk).reshape(-1)


def activations(m: int, cols: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed ^ 0x5EED).standard_normal((m, cols)).astype(np.float32)


# ---- device-side generation (torch), for matrices too large to build on the host in reasonable time
def matrix_on_device(ggml_type: int, rows: int, cols: int, seed: int, device):
    """The same distributions, generated with torch on `device`; returns a uint8 CUDA tensor."""
    import torch

    vals, nbytes = BLOCK[ggml_type]
    nblk = rows * (cols // vals)
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    out = torch.randint(0, 256, (nblk, nbytes), dtype=torch.uint8, device=device, generator=g)

    def f16_field(n):
        v = torch.empty(n, dtype=torch.float32, device=device).uniform_(1e-4, 2e-3, generator=g)
        return v.to(torch.float16).view(torch.uint8).reshape(n, 2)

    if ggml_type in (GGML_Q4_K, GGML_Q5_K):
        # uniform bytes already give uniform 6-bit scales/mins, nibbles and fifth bits
        out[:, 0:2] = f16_field(nblk)
        out[:, 2:4] = f16_field(nblk)
    elif ggml_type == GGML_Q6_K:
        sc = torch.randint(-32, 32, (nblk, 16), dtype=torch.int8, device=device, generator=g)
        out[:, 192:208] = sc.view(torch.uint8)
        out[:, 208:210] = f16_field(nblk)
    else:
        out[:, 0:2] = f16_field(nblk)
    return out.reshape(-1)
