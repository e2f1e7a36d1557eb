"""ctypes binding of the CPU oracle (``ferric_oracle.c``).

TEST INFRASTRUCTURE.  Only ``tests/``, the smoke check and the bench's CPU-baseline leg may import
this module; the product package never does.  Every function mirrors a ``fo_*`` entry point whose C
source cites the reference file:line it restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libferric_oracle.so")

GGML_F32, GGML_F16, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K, GGML_BF16 = 0, 1, 8, 12, 14, 30
MODE_DEQUANT_DOT, MODE_FUSED, MODE_SHADER, MODE_BF16 = 0, 1, 2, 3
FO_OK, FO_ERR_TYPE, FO_ERR_SHAPE, FO_ERR_ARG = 0, -1, -2, -3


class OracleError(Exception):
    """A reference ``Err(String)`` / ``assert!`` condition, carried as the oracle's status code."""

    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: oracle status {code}")
        self.code = code


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (``-ffp-contract=off``) if the library is missing or stale."""
    src = os.path.join(_HERE, "ferric_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libferric_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        L = _lib
        L.fo_f16_to_f32.restype = C.c_float
        L.fo_f16_to_f32.argtypes = [C.c_uint16]
        L.fo_f32_to_f16.restype = C.c_uint16
        L.fo_f32_to_f16.argtypes = [C.c_float]
        L.fo_bf16_rne.restype = C.c_uint16
        L.fo_bf16_rne.argtypes = [C.c_float]
        L.fo_type_size.argtypes = [C.c_uint32, C.c_size_t, C.POINTER(C.c_size_t)]
        L.fo_block_bytes.argtypes = [C.c_uint32, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
        L.fo_deq_raw.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_uint32, C.c_void_p]
        L.fo_deq_raw_bf16.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_uint32, C.c_void_p]
        L.fo_matmul_bt.restype = None
        L.fo_matmul_bt.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_float, C.c_void_p]
        L.fo_matmul_q.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32, C.c_size_t, C.c_size_t,
                                  C.c_void_p, C.c_size_t, C.c_void_p, C.c_int, C.c_int]
        L.fo_matvec_span.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32, C.c_size_t, C.c_size_t,
                                     C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_int, C.c_int]
        L.fo_swiglu.restype = None
        L.fo_swiglu.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]
        L.fo_add_rmsnorm.restype = None
        L.fo_add_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p]
        L.fo_quant_q8_0.restype = None
        L.fo_quant_q8_0.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        L.fo_q4k_block.restype = None
        L.fo_q4k_block.argtypes = [C.c_uint32, C.c_void_p]
        L.fo_q6k_block.restype = None
        L.fo_q6k_block.argtypes = [C.c_uint32, C.c_void_p]
        L.fo_q8_0_synth.restype = None
        L.fo_q8_0_synth.argtypes = [C.c_size_t, C.c_size_t, C.c_uint32, C.c_void_p, C.c_void_p]
    return _lib


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _bytes(raw) -> np.ndarray:
    return np.ascontiguousarray(np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, np.ndarray) else raw, dtype=np.uint8)


def f16_to_f32(bits: int) -> float:
    return float(lib().fo_f16_to_f32(int(bits) & 0xFFFF))


def f32_to_f16(x: float) -> int:
    return int(lib().fo_f32_to_f16(float(np.float32(x))))


def bf16_rne(x: float) -> int:
    return int(lib().fo_bf16_rne(float(np.float32(x))))


def type_size(ty: int, n: int) -> int:
    out = C.c_size_t(0)
    rc = lib().fo_type_size(ty, n, C.byref(out))
    if rc != FO_OK:
        raise OracleError(rc, f"unsupported ggml type {ty}")
    return out.value


def block_bytes(ty: int):
    v, b = C.c_size_t(0), C.c_size_t(0)
    if lib().fo_block_bytes(ty, C.byref(v), C.byref(b)) != FO_OK:
        return None
    return v.value, b.value


def deq_raw(raw, n: int, ty: int) -> np.ndarray:
    raw = _bytes(raw)
    out = np.empty(n, dtype=np.float32)
    rc = lib().fo_deq_raw(_p(raw), raw.size, n, ty, _p(out))
    if rc != FO_OK:
        raise OracleError(rc, f"deq_raw(ty={ty}, n={n}, len={raw.size})")
    return out


def deq_raw_bf16(raw, n: int, ty: int) -> np.ndarray:
    raw = _bytes(raw)
    out = np.empty(n, dtype=np.uint16)
    rc = lib().fo_deq_raw_bf16(_p(raw), raw.size, n, ty, _p(out))
    if rc != FO_OK:
        raise OracleError(rc, f"deq_raw_bf16(ty={ty}, n={n})")
    return out


def matmul_bt(a: np.ndarray, b: np.ndarray, scale: float = 1.0) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    m, k = a.shape
    n, k2 = b.shape
    assert k == k2
    c = np.empty((m, n), dtype=np.float32)
    lib().fo_matmul_bt(_p(a), _p(b), m, n, k, scale, _p(c))
    return c


def matmul_q(raw, ty: int, rows: int, cols: int, x: np.ndarray, threads: int = 1,
             mode: int = MODE_DEQUANT_DOT) -> np.ndarray:
    """y[m, rows] = x[m, cols] . W^T on raw GGUF block bytes; see ``fo_matmul_q`` for the modes."""
    raw = _bytes(raw)
    if mode == MODE_BF16:
        x = np.ascontiguousarray(x, dtype=np.uint16)
    else:
        x = np.ascontiguousarray(x, dtype=np.float32)
    if x.ndim == 1:
        x = x[None, :]
    m = x.shape[0]
    if x.shape[1] != cols:
        raise OracleError(FO_ERR_SHAPE, f"inner dim mismatch: x[..,{x.shape[1]}] vs W[..,{cols}]")
    y = np.empty((m, rows), dtype=np.float32)
    rc = lib().fo_matmul_q(_p(raw), raw.size, ty, rows, cols, _p(x), m, _p(y), threads, mode)
    if rc != FO_OK:
        raise OracleError(rc, f"matmul_q(ty={ty}, rows={rows}, cols={cols}, len={raw.size})")
    return y


def matvec_span(raw, ty: int, rows: int, cols: int, x: np.ndarray, lo: int, hi: int, threads: int = 1,
                mode: int = MODE_FUSED) -> np.ndarray:
    raw = _bytes(raw)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(max(hi - lo, 0), dtype=np.float32)
    rc = lib().fo_matvec_span(_p(raw), raw.size, ty, rows, cols, _p(x), lo, hi, _p(y), threads, mode)
    if rc != FO_OK:
        raise OracleError(rc, "matvec_span")
    return y


def swiglu(gu: np.ndarray, d: int) -> np.ndarray:
    gu = np.ascontiguousarray(gu, dtype=np.float32)
    t = gu.size // (2 * d)
    out = np.empty((t, d), dtype=np.float32)
    lib().fo_swiglu(_p(gu), t, d, _p(out))
    return out


def _expert_rows(raw: np.ndarray, ty: int, cols: int, row0: int, nrows: int) -> np.ndarray:
    vals, bb = block_bytes(ty)
    rb = cols // vals * bb
    return raw[row0 * rb:(row0 + nrows) * rb]


def matmul_q_swiglu_id(raw, ty: int, n_expert: int, eff: int, cols: int, x: np.ndarray, selw: np.ndarray, k: int,
                       mode: int = MODE_DEQUANT_DOT) -> np.ndarray:
    """``Tensor::matmul_q4_k_swiglu_id`` (crates/ferric-tensor/src/dtype.rs:1620-1637, kernel :2463-2516): the stack
    holds every expert's gate|up rows, expert-major; for token t and slot s the expert is ``u32(selw[t, k + s])``
    (:2508), its gate row o is ``e * 2 eff + o`` and its up row ``e * 2 eff + eff + o`` (:2509-2512), and the result is
    ``silu(g) * u`` (:2513).  Returns [t, k, eff]."""
    raw = _bytes(raw)
    x = np.ascontiguousarray(x, dtype=np.float32)
    t = x.shape[0]
    out = np.empty((t, k, eff), dtype=np.float32)
    for ti in range(t):
        for s in range(k):
            e = int(np.uint32(selw[ti, k + s]))
            assert 0 <= e < n_expert
            gu = matmul_q(_expert_rows(raw, ty, cols, e * 2 * eff, 2 * eff), ty, 2 * eff, cols, x[ti:ti + 1], mode=mode)
            out[ti, s] = swiglu(gu, eff)[0]
    return out


def matmul_q_id_wsum(raw, ty: int, n_expert: int, out_pe: int, cols: int, x: np.ndarray, selw: np.ndarray,
                     mode: int = MODE_DEQUANT_DOT) -> np.ndarray:
    """``Tensor::matmul_q6_k_id_wsum`` (crates/ferric-tensor/src/dtype.rs:1660-1677, kernel :2538-2566): x is
    [t, k, in]; row t of the result is ``total = total + selw[t, s] * acc_s`` over the slots in order (:2562), acc_s
    being expert ``u32(selw[t, k + s])``'s down rows times x[t, s] (:2553-2561).  Returns [t, out_pe]."""
    raw = _bytes(raw)
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.ndim == 2:
        x = x[None]
    t, k = x.shape[0], x.shape[1]
    out = np.zeros((t, out_pe), dtype=np.float32)
    for ti in range(t):
        total = np.zeros(out_pe, dtype=np.float32)
        for s in range(k):
            e = int(np.uint32(selw[ti, k + s]))
            assert 0 <= e < n_expert
            acc = matmul_q(_expert_rows(raw, ty, cols, e * out_pe, out_pe), ty, out_pe, cols, x[ti, s:s + 1], mode=mode)[0]
            total = (total + np.float32(selw[ti, s]) * acc).astype(np.float32)
        out[ti] = total
    return out


def add_rmsnorm(a: np.ndarray, b=None, w=None, eps: float = 1e-6):
    """(sum, norm) as the reference's add_rmsnorm kernel computes them; b=None is plain rmsnorm."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    d = a.shape[-1]
    rows = a.size // d
    b = None if b is None else np.ascontiguousarray(b, dtype=np.float32)
    w = None if w is None else np.ascontiguousarray(w, dtype=np.float32)
    s, n = np.empty_like(a), np.empty_like(a)
    lib().fo_add_rmsnorm(_p(a), _p(b) if b is not None else None, _p(w) if w is not None else None, eps, rows, d,
                         _p(s), _p(n))
    return s, n


def quant_q8_0(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty((x.size + 31) // 32 * 34, dtype=np.uint8)
    lib().fo_quant_q8_0(_p(x), x.size, _p(out))
    return out


def q4k_block(seed: int) -> np.ndarray:
    out = np.empty(144, dtype=np.uint8)
    lib().fo_q4k_block(seed & 0xFFFFFFFF, _p(out))
    return out


def q6k_block(seed: int) -> np.ndarray:
    out = np.empty(210, dtype=np.uint8)
    lib().fo_q6k_block(seed & 0xFFFFFFFF, _p(out))
    return out


def q8_0_synth(rows: int, cols: int, seed: int):
    raw = np.empty(rows * (cols // 32) * 34, dtype=np.uint8)
    vals = np.empty(rows * cols, dtype=np.float32)
    lib().fo_q8_0_synth(rows, cols, seed & 0xFFFFFFFF, _p(raw), _p(vals))
    return raw, vals
