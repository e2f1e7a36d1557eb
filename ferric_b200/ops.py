"""Python mirror of the reference's QMatrix / matmul_q operator interface (see package docstring)."""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import numpy as np
import torch

from . import _lib

GGML_F32, GGML_F16, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K, GGML_BF16 = 0, 1, 8, 12, 14, 30


class FerricError(RuntimeError):
    """A failing C-ABI call: ``status`` is the FERRIC_* code, the text is ferric_cuda_last_error().

    Stands for the reference's ``Err(String)`` (unsupported type) and its ``assert!`` panics
    (shape errors), crates/ferric-tensor/src/dtype.rs:855, :1389-1390, :1429.
    """

    def __init__(self, status: int, where: str):
        msg = _lib.load().ferric_cuda_last_error().decode("utf-8", "replace")
        super().__init__(f"{where}: {_lib.STATUS_NAMES[status] if 0 <= status < 8 else status}: {msg}")
        self.status = status


def _check(status: int, where: str) -> None:
    if status != _lib.OK:
        raise FerricError(status, where)


def type_size(ggml_type: int, n: int) -> int:
    """``ferric_gguf::type_size`` (crates/ferric-gguf/src/lib.rs:471-494)."""
    out = C.c_size_t(0)
    _check(_lib.load().ferric_gguf_type_size(ggml_type, n, C.byref(out)), "type_size")
    return out.value


def _as_u8(raw) -> np.ndarray:
    if isinstance(raw, np.ndarray):
        return np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    return np.frombuffer(raw, dtype=np.uint8)


class Context:
    """A device + stream, the counterpart of ``ferric_core::Context`` (crates/ferric-core/src/lib.rs:19-43).

    ``stream=None`` makes the context own a stream; ``stream="torch"`` binds it to torch's current
    stream on that device so operator calls order with surrounding torch work.
    """

    def __init__(self, device: int = 0, stream: Optional[object] = "torch"):
        self._lib = _lib.load()
        self.device = int(device)
        h = C.c_void_p()
        if stream is None:
            _check(self._lib.ferric_cuda_ctx_create(self.device, C.byref(h)), "Context")
        else:
            if stream == "torch":
                stream = torch.cuda.current_stream(self.device).cuda_stream
            _check(self._lib.ferric_cuda_ctx_create_on_stream(self.device, C.c_void_p(int(stream)), C.byref(h)),
                   "Context")
        self._h = h

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.ferric_cuda_ctx_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_stream(self, cuda_stream: int) -> None:
        _check(self._lib.ferric_cuda_ctx_set_stream(self._h, C.c_void_p(int(cuda_stream))), "set_stream")

    def use_torch_stream(self) -> None:
        self.set_stream(torch.cuda.current_stream(self.device).cuda_stream)

    def sync(self) -> None:
        _check(self._lib.ferric_cuda_ctx_sync(self._h), "sync")

    def caps(self) -> dict:
        c = _lib.Caps()
        _check(self._lib.ferric_cuda_ctx_caps(self._h, C.byref(c)), "caps")
        return {k: getattr(c, k) for k, _ in _lib.Caps._fields_}

    def launches(self) -> int:
        return int(self._lib.ferric_cuda_ctx_launches(self._h))

    def prof_enable(self, on: bool = True) -> None:
        """Switch the per-op timing buckets on or off (the reference's FERRIC_PROFILE)."""
        _check(self._lib.ferric_cuda_prof_enable(self._h, int(on)), "prof_enable")

    def prof(self, label: str) -> None:
        """``prof(ctx, label)`` (crates/ferric-tensor/src/lib.rs:3017-3031): sync, charge the time since the last mark to `label`."""
        _check(self._lib.ferric_cuda_prof(self._h, label.encode()), "prof")

    def prof_report(self) -> str:
        """``prof_report()`` (:3033-3046): the buckets, largest first, as text; resets them."""
        n = C.c_size_t()
        _check(self._lib.ferric_cuda_prof_report(self._h, None, 0, C.byref(n)), "prof_report")
        buf = C.create_string_buffer(n.value + 1)
        _check(self._lib.ferric_cuda_prof_report(self._h, buf, n.value + 1, C.byref(n)), "prof_report")
        return buf.value.decode()

    def reserve_scratch(self, nbytes: int) -> None:
        _check(self._lib.ferric_cuda_ctx_reserve_scratch(self._h, nbytes), "reserve_scratch")

    def chain_reserve(self, slot_bytes: int) -> None:
        """Size the two prepared-activation slots chained products use (``ferric_cuda_chain_reserve``)."""
        _check(self._lib.ferric_cuda_chain_reserve(self._h, slot_bytes), "chain_reserve")

    def deq_raw(self, raw, n: int, ggml_type: int) -> np.ndarray:
        """``ferric_gguf::deq_raw`` (crates/ferric-gguf/src/lib.rs:497-520), decoded on the device."""
        raw = _as_u8(raw)
        out = np.empty(n, dtype=np.float32)
        _check(self._lib.ferric_gguf_deq_raw(self._h, raw.ctypes.data, raw.size, n, ggml_type, out.ctypes.data),
               "deq_raw")
        return out

    def add_rmsnorm(self, a: torch.Tensor, b: Optional[torch.Tensor] = None, weight: Optional[torch.Tensor] = None,
                    eps: float = 1e-6, sum_out: Optional[torch.Tensor] = None,
                    norm_out: Optional[torch.Tensor] = None):
        """``a.add_rmsnorm(b, weight, eps) -> (sum, norm)`` (crates/ferric-tensor/src/lib.rs:372-384);
        ``b=None`` is plain ``rmsnorm`` (:346-353), ``weight=None`` the weightless form (:340-344)."""
        a = a.contiguous()
        d = a.shape[-1]
        rows = a.numel() // d
        if norm_out is None:
            norm_out = torch.empty_like(a)
        if b is not None and sum_out is None:
            sum_out = torch.empty_like(a)
        _check(self._lib.ferric_cuda_add_rmsnorm(
            self._h, a.data_ptr(), b.contiguous().data_ptr() if b is not None else None,
            weight.contiguous().data_ptr() if weight is not None else None, float(eps), rows, d,
            sum_out.data_ptr() if sum_out is not None else None, norm_out.data_ptr()), "add_rmsnorm")
        return (sum_out if sum_out is not None else a), norm_out

    def swiglu(self, gu: torch.Tensor, d: int) -> torch.Tensor:
        """``Tensor::swiglu`` (crates/ferric-tensor/src/lib.rs:726-737)."""
        gu = gu.contiguous()
        t = gu.numel() // (2 * d)
        out = torch.empty((t, d), dtype=torch.float32, device=gu.device)
        _check(self._lib.ferric_cuda_swiglu(self._h, gu.data_ptr(), t, d, out.data_ptr()), "swiglu")
        return out


class QMatrix:
    """A packed-quant weight matrix (``ferric_tensor::QMatrix``, crates/ferric-tensor/src/dtype.rs:865-931)."""

    def __init__(self, ctx: Context, handle: C.c_void_p):
        self.ctx = ctx
        self._lib = ctx._lib
        self._h = handle

    @staticmethod
    def block_bytes(ggml_type: int):
        """(values per block, bytes per block) or None (crates/ferric-tensor/src/dtype.rs:873-889)."""
        v, b = C.c_size_t(0), C.c_size_t(0)
        rc = _lib.load().ferric_cuda_qmatrix_block_bytes(ggml_type, C.byref(v), C.byref(b))
        if rc == _lib.UNSUPPORTED:
            return None
        _check(rc, "block_bytes")
        return v.value, b.value

    @classmethod
    def from_bytes(cls, ctx: Context, raw, ggml_type: int, rows: int, cols: int) -> "QMatrix":
        """``QMatrix::from_bytes`` (crates/ferric-tensor/src/dtype.rs:893-908): raw GGUF block bytes, [out, in]."""
        raw = _as_u8(raw)
        h = C.c_void_p()
        _check(ctx._lib.ferric_cuda_qmatrix_from_bytes(ctx._h, raw.ctypes.data, raw.size, ggml_type, rows, cols,
                                                       C.byref(h)), "QMatrix.from_bytes")
        return cls(ctx, h)

    @classmethod
    def from_bytes_view(cls, ctx: Context, raw, ggml_type: int, rows: int, cols: int, row0: int, nrows: int,
                        col0: int, ncols: int) -> "QMatrix":
        """A tensor-parallel shard (row range x K range) of the full tensor's bytes."""
        raw = _as_u8(raw)
        h = C.c_void_p()
        _check(ctx._lib.ferric_cuda_qmatrix_from_bytes_view(ctx._h, raw.ctypes.data, raw.size, ggml_type, rows, cols,
                                                            row0, nrows, col0, ncols, C.byref(h)),
               "QMatrix.from_bytes_view")
        return cls(ctx, h)

    @classmethod
    def from_device_bytes(cls, ctx: Context, raw: torch.Tensor, ggml_type: int, rows: int, cols: int) -> "QMatrix":
        """As ``from_bytes`` for block bytes already in device memory (a uint8 CUDA tensor)."""
        assert raw.is_cuda and raw.dtype == torch.uint8 and raw.is_contiguous()
        h = C.c_void_p()
        _check(ctx._lib.ferric_cuda_qmatrix_from_device_bytes(ctx._h, raw.data_ptr(), raw.numel(), ggml_type, rows,
                                                              cols, C.byref(h)), "QMatrix.from_device_bytes")
        return cls(ctx, h)

    @classmethod
    def from_dense(cls, ctx: Context, w: np.ndarray) -> "QMatrix":
        """``QMatrix::from_dense`` (crates/ferric-tensor/src/dtype.rs:912-926): an already dequantised row-major
        [rows, cols] weight, the fallback for formats without a packed kernel."""
        w = np.ascontiguousarray(w, dtype=np.float32)
        h = C.c_void_p()
        _check(ctx._lib.ferric_cuda_qmatrix_from_dense(ctx._h, w.ctypes.data, w.shape[0], w.shape[1], C.byref(h)), "QMatrix.from_dense")
        return cls(ctx, h)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.ferric_cuda_qmatrix_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def rows(self) -> int:
        return int(self._lib.ferric_cuda_qmatrix_rows(self._h))

    def cols(self) -> int:
        return int(self._lib.ferric_cuda_qmatrix_cols(self._h))

    def nbytes(self) -> int:
        return int(self._lib.ferric_cuda_qmatrix_nbytes(self._h))

    def n_shards(self) -> int:
        return int(self._lib.ferric_cuda_qmatrix_n_shards(self._h))

    def ggml_type(self) -> int:
        return int(self._lib.ferric_cuda_qmatrix_ggml_type(self._h))

    def scratch_bytes(self, m: int) -> int:
        return int(self._lib.ferric_cuda_qmatrix_scratch_bytes(self._h, m))

    # -- operators -------------------------------------------------------------------------
    def _x2d(self, x: torch.Tensor, allow_row_stride: bool = False) -> torch.Tensor:
        if not x.is_cuda or x.dtype != torch.float32:
            raise TypeError("activations must be a float32 CUDA tensor")
        if x.dim() == 1:
            x = x[None, :]
        if allow_row_stride and x.dim() == 2 and x.stride(1) == 1 and x.stride(0) >= x.shape[1] \
                and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0:
            return x
        return x.contiguous()

    def matmul(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x.matmul_q(&w)``: y[m, rows] = x[m, cols] . W^T (crates/ferric-tensor/src/dtype.rs:935-944).

        A column slice of a wider row-major tensor is consumed in place (row stride passed through);
        ``out`` may likewise be a column slice of a wider result tensor."""
        x = self._x2d(x, allow_row_stride=True)
        m = x.shape[0]
        y = out if out is not None else torch.empty((m, self.rows()), dtype=torch.float32, device=x.device)
        assert y.stride(-1) == 1
        ldx = x.stride(0) if m > 1 else 0
        ldy = y.stride(0) if (y.dim() == 2 and m > 1) else 0
        _check(self._lib.ferric_cuda_matmul_q_ld(self.ctx._h, self._h, x.data_ptr(), m, x.shape[1], ldx,
                                                 y.data_ptr(), ldy), "matmul_q")
        return y

    def matmul_noalloc(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``matmul`` for hosts that must not allocate: the library's fixed scratch array is used and the
        caller supplies ``out``.  Contiguous inputs only; fails if the product needs more than 2 MiB of scratch."""
        if not (x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()):
            raise TypeError("matmul_noalloc needs contiguous float32 CUDA tensors")
        m = 1 if x.dim() == 1 else x.shape[0]
        _check(self._lib.ferric_cuda_matmul_q_noalloc(self.ctx._h, self._h, x.data_ptr(), m, x.shape[-1],
                                                      out.data_ptr()), "matmul_q_noalloc")
        return out

    def matmul_bf16(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Prefill product on the tensor cores: ``x`` [m, cols] bfloat16, result [m, rows] float32 with the
        weights rounded to bf16 (``Tensor::matmul_q4_k_coop``, ferric-tensor/src/dtype.rs:1818-1834).  Q4_K, Q5_K, Q6_K and Q8_0."""
        if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()):
            raise TypeError("matmul_bf16 needs a contiguous 2-D bfloat16 CUDA tensor")
        m = x.shape[0]
        if out is None:
            out = torch.empty((m, self.rows()), dtype=torch.float32, device=x.device)
        _check(self._lib.ferric_cuda_matmul_q_bf16(self.ctx._h, self._h, x.data_ptr(), m, x.shape[1], out.data_ptr()),
               "matmul_q_bf16")
        return out

    def gemm_status(self) -> int:
        """Synchronise and return the tensor-core kernel's give-up code (0 = every wait completed); raises on non-zero."""
        code = C.c_int32(0)
        _check(self._lib.ferric_cuda_gemm_status(self.ctx._h, C.byref(code)), "gemm_status")
        return code.value

    def prepare(self, x: torch.Tensor) -> int:
        """First half of ``matmul``: convert x into the context's activation scratch; returns m."""
        x = self._x2d(x, allow_row_stride=True)
        m = x.shape[0]
        _check(self._lib.ferric_cuda_prepare_x(self.ctx._h, self._h, x.data_ptr(), m, x.shape[1],
                                               x.stride(0) if m > 1 else 0), "prepare_x")
        return m

    def add_rmsnorm_prepare(self, a: torch.Tensor, b: Optional[torch.Tensor] = None,
                            weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                            sum_out: Optional[torch.Tensor] = None, norm_out: Optional[torch.Tensor] = None) -> int:
        """``(sum, norm) = a.add_rmsnorm(b, weight, eps)`` fused with ``prepare(norm)``; returns m."""
        m = a.numel() // a.shape[-1]
        assert a.shape[-1] == self.cols() and a.is_contiguous()
        ptr = lambda t: t.data_ptr() if t is not None else None
        _check(self._lib.ferric_cuda_add_rmsnorm_prepare(self.ctx._h, self._h, a.data_ptr(), ptr(b), ptr(weight),
                                                         float(eps), m, ptr(sum_out), ptr(norm_out)),
               "add_rmsnorm_prepare")
        return m

    def matmul_prepared(self, m: int, out: Optional[torch.Tensor] = None, swiglu: bool = False) -> torch.Tensor:
        """Second half of ``matmul`` / ``try_matmul_swiglu`` on the activations last prepared on the context."""
        n = self.rows() // 2 if swiglu else self.rows()
        y = out if out is not None else torch.empty((m, n), dtype=torch.float32,
                                                    device=torch.device("cuda", self.ctx.device))
        ldy = y.stride(0) if (y.dim() == 2 and m > 1) else 0
        _check(self._lib.ferric_cuda_matmul_q_prepared(self.ctx._h, self._h, m, y.data_ptr(), ldy, int(swiglu)),
               "matmul_q_prepared")
        return y

    def _link(self, m: int, out: Optional[torch.Tensor], swiglu: bool, in_slot: int, in_rms: bool, eps: float, next: int,
              next_qm: Optional["QMatrix"], h: Optional[torch.Tensor], norm_weight: Optional[torch.Tensor]) -> "_lib.ChainLink":
        ptr = lambda t: t.data_ptr() if t is not None else None
        ldy = out.stride(0) if (out is not None and out.dim() == 2 and m > 1) else 0
        return _lib.ChainLink(self._h, int(swiglu), in_slot, int(in_rms), float(eps), ptr(out), ldy, next,
                              next_qm._h if next_qm is not None else None, ptr(h), ptr(norm_weight))

    def chain_matmul(self, m: int, out: torch.Tensor, swiglu: bool = False, in_slot: int = 0, in_rms: bool = False,
                     eps: float = 1e-6, next: int = 0, next_qm: Optional["QMatrix"] = None, h: Optional[torch.Tensor] = None,
                     norm_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One link of a decoder layer's chain (``ferric_cuda_chain_matmul``): the product from prepared-activation
        slot ``in_slot``, then, in the same launch, what the next product needs -- ``next=1`` prepares the result for
        ``next_qm``, ``next=2`` adds it to the residual stream ``h`` first and leaves the 1/rms factor to the next link
        (``in_rms``).  Returns ``out``."""
        link = self._link(m, out, swiglu, in_slot, in_rms, eps, next, next_qm, h, norm_weight)
        _check(self._lib.ferric_cuda_chain_matmul(self.ctx._h, C.byref(link), m), "chain_matmul")
        return out

    def matmul_host(self, x: np.ndarray) -> np.ndarray:
        """The same product with host buffers (copies in, runs, copies out, synchronises)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        y = np.empty((x.shape[0], self.rows()), dtype=np.float32)
        _check(self._lib.ferric_cuda_matmul_q_host(self.ctx._h, self._h, x.ctypes.data, x.shape[0], x.shape[1],
                                                   y.ctypes.data), "matmul_q_host")
        return y

    def try_matmul_swiglu(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """``x.try_matmul_swiglu(&w)`` (crates/ferric-tensor/src/dtype.rs:949-959); None when not fusable."""
        x = self._x2d(x)
        m = x.shape[0]
        y = out if out is not None else torch.empty((m, self.rows() // 2), dtype=torch.float32, device=x.device)
        rc = self._lib.ferric_cuda_matmul_q_swiglu(self.ctx._h, self._h, x.data_ptr(), m, x.shape[1], y.data_ptr())
        if rc == _lib.UNSUPPORTED:
            return None
        _check(rc, "matmul_q_swiglu")
        return y

    def matmul_swiglu_id(self, x: torch.Tensor, selw: torch.Tensor, k: int, eff: int) -> torch.Tensor:
        """``x.matmul_q4_k_swiglu_id(w, selw, k, eff)`` (crates/ferric-tensor/src/dtype.rs:1620-1637): this matrix stacks
        every expert's gate|up rows; ``selw`` [t, 2k] holds the router's weights, then the expert indices as f32.
        Returns [t, k, eff]."""
        x, selw = x.contiguous(), selw.contiguous()
        t = x.shape[0]
        y = torch.empty((t, k, eff), dtype=torch.float32, device=x.device)
        _check(self._lib.ferric_cuda_matmul_q_swiglu_id(self.ctx._h, self._h, x.data_ptr(), t, x.shape[1], selw.data_ptr(), k, eff,
                                                        y.data_ptr()), "matmul_q_swiglu_id")
        return y

    def matmul_id_wsum(self, x: torch.Tensor, selw: torch.Tensor, out_pe: int) -> torch.Tensor:
        """``x.matmul_q6_k_id_wsum(w, selw, out_pe)`` (crates/ferric-tensor/src/dtype.rs:1660-1677): ``x`` is [t, k, in]
        (2-D [k, in] means one token); returns [t, out_pe], the selected experts' down products summed with the
        router's weights."""
        x, selw = x.contiguous(), selw.contiguous()
        if x.dim() == 2:
            x = x[None]
        t, k = x.shape[0], x.shape[1]
        y = torch.empty((t, out_pe), dtype=torch.float32, device=x.device)
        _check(self._lib.ferric_cuda_matmul_q_id_wsum(self.ctx._h, self._h, x.data_ptr(), t, k, x.shape[2], selw.data_ptr(), out_pe,
                                                      y.data_ptr()), "matmul_q_id_wsum")
        return y

    def gate_up_swiglu(self, x: torch.Tensor) -> torch.Tensor:
        """``Proj::gate_up_swiglu`` (crates/ferric-llama/src/qwen3.rs:219-227): fused if possible."""
        y = self.try_matmul_swiglu(x)
        if y is not None:
            return y
        return self.ctx.swiglu(self.matmul(x), self.rows() // 2)

    def dequant(self, bf16: bool = False) -> torch.Tensor:
        """deq_raw of the loaded weight on the device: f32 [rows, cols], or bf16 bit patterns (int16 view)."""
        dev = torch.device("cuda", self.ctx.device)
        if bf16:
            out = torch.empty((self.rows(), self.cols()), dtype=torch.bfloat16, device=dev)
            _check(self._lib.ferric_cuda_dequant_bf16(self.ctx._h, self._h, out.data_ptr()), "dequant_bf16")
        else:
            out = torch.empty((self.rows(), self.cols()), dtype=torch.float32, device=dev)
            _check(self._lib.ferric_cuda_dequant_f32(self.ctx._h, self._h, out.data_ptr()), "dequant_f32")
        return out


class Proj:
    """``Proj`` (crates/ferric-llama/src/qwen3.rs:192-228): q|k|v or gate|up as one fused matrix when the parts share a
    quant format, else one matrix per part with the results written side by side."""

    def __init__(self, ctx: Context, handle: C.c_void_p):
        self.ctx, self._lib, self._h = ctx, ctx._lib, handle

    @classmethod
    def from_parts(cls, ctx: Context, parts) -> "Proj":
        """A projection over matrices already built; it takes ownership of them."""
        table = (C.c_void_p * len(parts))(*[q._h.value for q in parts])
        h = C.c_void_p()
        _check(ctx._lib.ferric_cuda_proj_from_parts(table, len(parts), C.byref(h)), "proj_from_parts")
        for q in parts:
            q._h = None
        return cls(ctx, h)

    def n_parts(self) -> int:
        return int(self._lib.ferric_cuda_proj_n_parts(self._h))

    def fused(self) -> bool:
        return self.n_parts() == 1

    def rows(self) -> int:
        return int(self._lib.ferric_cuda_proj_rows(self._h))

    def cols(self) -> int:
        return int(self._lib.ferric_cuda_proj_cols(self._h))

    def part_types(self):
        return [int(self._lib.ferric_cuda_qmatrix_ggml_type(self._lib.ferric_cuda_proj_part(self._h, i))) for i in range(self.n_parts())]

    def matmul(self, x: torch.Tensor) -> torch.Tensor:
        """``Proj::matmul`` (:209-218)."""
        x = x.contiguous() if x.dim() == 2 else x[None, :].contiguous()
        y = torch.empty((x.shape[0], self.rows()), dtype=torch.float32, device=x.device)
        _check(self._lib.ferric_cuda_proj_matmul(self.ctx._h, self._h, x.data_ptr(), x.shape[0], x.shape[1], y.data_ptr()), "proj_matmul")
        return y

    def gate_up_swiglu(self, x: torch.Tensor, n_ff: int) -> torch.Tensor:
        """``Proj::gate_up_swiglu`` (:221-228)."""
        x = x.contiguous() if x.dim() == 2 else x[None, :].contiguous()
        y = torch.empty((x.shape[0], n_ff), dtype=torch.float32, device=x.device)
        _check(self._lib.ferric_cuda_proj_gate_up_swiglu(self.ctx._h, self._h, x.data_ptr(), x.shape[0], x.shape[1], n_ff, y.data_ptr()),
               "proj_gate_up_swiglu")
        return y

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.ferric_cuda_proj_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _DevView:
    """A raw device pointer dressed as a CUDA array, so torch can wrap it without copying."""

    def __init__(self, ptr: int, shape, typestr: str = "<f4"):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 3, "strides": None}


class TPGroup:
    """One rank's end of the tensor-parallel exchange (``ferric_cuda_tp_*``): the all-reduce of the o / down
    partial sums over CUDA-IPC peer memory.  ``exchange`` hands the 64-byte IPC handles round the ranks; any
    all-gather of bytes will do (``torch.distributed.all_gather_object`` here)."""

    def __init__(self, ctx: Context, rank: int, world: int, rows: int, cols: int):
        self.ctx, self.rank, self.world, self.rows, self.cols = ctx, rank, world, rows, cols
        self._lib = ctx._lib
        h = C.c_void_p()
        _check(self._lib.ferric_cuda_tp_create(ctx._h, rank, world, rows * cols, C.byref(h)), "tp_create")
        self._h = h
        self._views = {}

    def export(self) -> bytes:
        buf = (C.c_uint8 * 64)()
        _check(self._lib.ferric_cuda_tp_export(self._h, buf), "tp_export")
        return bytes(buf)

    def connect(self, handles) -> None:
        blob = b"".join(handles)
        assert len(blob) == 64 * self.world
        _check(self._lib.ferric_cuda_tp_connect(self._h, blob), "tp_connect")

    @staticmethod
    def connect_local(groups) -> None:
        """Connect groups that all live in this process (rank order, one per rank)."""
        table = (C.c_void_p * len(groups))(*[g._h.value for g in groups])
        for g in groups:
            _check(g._lib.ferric_cuda_tp_connect_local(g._h, table), "tp_connect_local")

    def connect_with_torch_distributed(self) -> None:
        import torch.distributed as dist
        handles = [None] * self.world
        dist.all_gather_object(handles, self.export())
        self.connect(handles)
        dist.barrier()

    def partial(self, kind: int) -> torch.Tensor:
        """This rank's exchange buffer `kind` as a [rows, cols] f32 tensor: the ``out`` of the row-parallel matmul."""
        if kind not in self._views:
            ptr = self._lib.ferric_cuda_tp_partial(self._h, kind)
            self._views[kind] = torch.as_tensor(_DevView(ptr, (self.rows, self.cols)),
                                                device=torch.device("cuda", self.ctx.device))
        return self._views[kind]

    def signal(self, kind: int) -> None:
        _check(self._lib.ferric_cuda_tp_signal(self.ctx._h, self._h, kind), "tp_signal")

    def add_rmsnorm_prepare(self, kind: int, qm: "QMatrix", a: torch.Tensor, weight: Optional[torch.Tensor] = None,
                            eps: float = 1e-6, sum_out: Optional[torch.Tensor] = None,
                            norm_out: Optional[torch.Tensor] = None, pushed: bool = False) -> int:
        """``qm.add_rmsnorm_prepare(a, b, ..)`` with b = the all-reduced exchange `kind`: the buffers the ranks
        signalled, or (``pushed``) what they pushed with ``matmul_push``."""
        m = a.numel() // a.shape[-1]
        ptr = lambda t: t.data_ptr() if t is not None else None
        fn = self._lib.ferric_cuda_tp_add_rmsnorm_prepare_pushed if pushed else self._lib.ferric_cuda_tp_add_rmsnorm_prepare
        _check(fn(self.ctx._h, self._h, kind, qm._h, a.data_ptr(), ptr(weight), float(eps), m, ptr(sum_out), ptr(norm_out)),
               "tp_add_rmsnorm_prepare")
        return m

    def allreduce_add_rmsnorm(self, kind: int, partial: torch.Tensor, a: torch.Tensor, weight: Optional[torch.Tensor] = None,
                              eps: float = 1e-6, sum_out: Optional[torch.Tensor] = None,
                              norm_out: Optional[torch.Tensor] = None, steps: int = 7) -> None:
        """(sum, norm) = add_rmsnorm(a, all-reduce(partial)) through the two-step pushed all-reduce; for many rows.
        `steps`: 1 scatter, 2 reduce, 4 consume (a host driving several ranks on one GPU runs them one at a time)."""
        rows, d = a.numel() // a.shape[-1], a.shape[-1]
        ptr = lambda t: t.data_ptr() if t is not None else None
        _check(self._lib.ferric_cuda_tp_allreduce_add_rmsnorm_steps(self.ctx._h, self._h, kind, partial.data_ptr(), a.data_ptr(),
                                                                    ptr(weight), float(eps), rows, d, ptr(sum_out), ptr(norm_out), steps),
               "tp_allreduce_add_rmsnorm")

    def matmul_scatter(self, kind: int, qm: "QMatrix", x: torch.Tensor) -> bool:
        """The row-parallel product x . W^T of this rank, scattered as step 1 of exchange `kind` of the two-step all-reduce
        (by the product's own finish kernel where its K range is cut across CTAs: returns True); continue with
        ``allreduce_add_rmsnorm(.., steps=6)``."""
        assert x.dtype == torch.float32 and x.is_cuda and x.stride(-1) == 1
        m = x.numel() // x.shape[-1]
        fused = C.c_int32(0)
        _check(self._lib.ferric_cuda_tp_matmul_scatter(self.ctx._h, self._h, kind, qm._h, x.data_ptr(), m,
                                                       x.stride(0) if x.dim() > 1 else 0, C.byref(fused)), "tp_matmul_scatter")
        return bool(fused.value)

    def matmul_push(self, kind: int, qm: "QMatrix", x: torch.Tensor) -> None:
        """The row-parallel product x . W^T of this rank, stored by the kernel's epilogue into every rank's receive
        region for exchange `kind` instead of a local buffer."""
        assert x.dtype == torch.float32 and x.is_cuda and x.stride(-1) == 1
        m = x.numel() // x.shape[-1]
        ldx = x.stride(0) if x.dim() == 2 else x.shape[-1]
        _check(self._lib.ferric_cuda_tp_matmul_push(self.ctx._h, self._h, kind, qm._h, x.data_ptr(), m, ldx), "tp_matmul_push")

    def chain_matmul(self, kind: int, qm: "QMatrix", m: int, in_slot: int, next_qm: "QMatrix", h: torch.Tensor,
                     norm_weight: Optional[torch.Tensor] = None) -> None:
        """A residual chain link whose product is row-parallel (``ferric_cuda_tp_chain_matmul``): push, all-reduce,
        residual add and preparation of the next product in one launch."""
        link = qm._link(m, None, False, in_slot, False, 0.0, 2, next_qm, h, norm_weight)
        _check(self._lib.ferric_cuda_tp_chain_matmul(self.ctx._h, self._h, kind, C.byref(link), m), "tp_chain_matmul")

    def check(self) -> None:
        """Synchronise and raise if a wait on a peer ran out."""
        t = C.c_int32(0)
        _check(self._lib.ferric_cuda_tp_status(self.ctx._h, self._h, C.byref(t)), "tp_status")

    def reset(self) -> None:
        """After a time-out: clear this rank's status, counters and receive regions (every rank must)."""
        _check(self._lib.ferric_cuda_tp_reset(self.ctx._h, self._h), "tp_reset")

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._views = {}
            self._lib.ferric_cuda_tp_free(self._h)
            self._h = None


class Gguf:
    """A parsed GGUF file: ``ferric_gguf::parse`` / ``GgufFile::open`` (crates/ferric-gguf/src/lib.rs:105-132, :533-554).

    ``Gguf(path)`` memory-maps a file; ``Gguf.parse(data)`` reads one already in memory (the bytes are kept alive by
    this object).  ``metadata`` is a dict of Python values, ``tensors`` a list of dicts in file order."""

    def __init__(self, path: Optional[str] = None, _data: Optional[np.ndarray] = None):
        self._lib = _lib.load()
        self._data = _data
        h = C.c_void_p()
        if _data is not None:
            _check(self._lib.ferric_gguf_parse(_data.ctypes.data, _data.size, C.byref(h)), "gguf_parse")
        else:
            _check(self._lib.ferric_gguf_open(os.fsencode(path), C.byref(h)), "gguf_open")
        self._h = h
        self.tensors = [self._info_at(i) for i in range(self._lib.ferric_gguf_n_tensors(h))]
        self.metadata = {k: self._meta(k) for k in self._keys()}

    @classmethod
    def parse(cls, data) -> "Gguf":
        return cls(_data=np.ascontiguousarray(np.frombuffer(bytes(data), dtype=np.uint8) if not isinstance(data, np.ndarray) else data,
                                              dtype=np.uint8))

    @property
    def data_start(self) -> int:
        return self._lib.ferric_gguf_data_start(self._h)

    @staticmethod
    def _unpack(t: "_lib.GgufTensor") -> dict:
        return {"name": t.name.decode("utf-8", "replace"), "dims": [int(t.dims[i]) for i in range(t.n_dims)],
                "ggml_type": int(t.ggml_type), "offset": int(t.offset), "n_elements": int(t.n_elements), "nbytes": int(t.nbytes)}

    def _info_at(self, i: int) -> dict:
        t = _lib.GgufTensor()
        _check(self._lib.ferric_gguf_tensor_at(self._h, i, C.byref(t)), "gguf_tensor_at")
        return self._unpack(t)

    def tensor(self, name: str) -> Optional[dict]:
        """``Gguf::tensor`` (:444): None when the file has no such tensor."""
        t = _lib.GgufTensor()
        if self._lib.ferric_gguf_tensor_by_name(self._h, name.encode(), C.byref(t)) != _lib.OK:
            return None
        return self._unpack(t)

    def raw(self, name: str) -> np.ndarray:
        """``Gguf::raw`` (:447-453): the tensor's packed bytes, a read-only view into the file."""
        p, n = C.c_void_p(), C.c_size_t()
        _check(self._lib.ferric_gguf_raw(self._h, name.encode(), C.byref(p), C.byref(n)), "gguf_raw")
        if n.value == 0:
            return np.zeros(0, dtype=np.uint8)
        arr = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(n.value,))
        arr.flags.writeable = False
        return arr

    def _str(self, fn, *args) -> str:
        n = C.c_size_t()
        _check(fn(self._h, *args, None, 0, C.byref(n)), "gguf_meta")
        buf = C.create_string_buffer(n.value + 1)
        _check(fn(self._h, *args, buf, n.value + 1, C.byref(n)), "gguf_meta")
        return buf.raw[:n.value].decode("utf-8", "replace")

    def _keys(self):
        return [self._str(self._lib.ferric_gguf_meta_key_at, i) for i in range(self._lib.ferric_gguf_n_meta(self._h))]

    def _meta(self, key: str):
        k, kind = key.encode(), C.c_int32()
        _check(self._lib.ferric_gguf_meta_kind(self._h, k, C.byref(kind)), "gguf_meta_kind")
        if kind.value == 0:
            v = C.c_uint64()
            _check(self._lib.ferric_gguf_meta_u64(self._h, k, C.byref(v)), "gguf_meta_u64")
            return v.value
        if kind.value == 1:
            v = C.c_int64()
            _check(self._lib.ferric_gguf_meta_i64(self._h, k, C.byref(v)), "gguf_meta_i64")
            return v.value
        if kind.value == 2:
            v = C.c_double()
            _check(self._lib.ferric_gguf_meta_f64(self._h, k, C.byref(v)), "gguf_meta_f64")
            return v.value
        if kind.value == 3:
            v = C.c_int32()
            _check(self._lib.ferric_gguf_meta_bool(self._h, k, C.byref(v)), "gguf_meta_bool")
            return bool(v.value)
        if kind.value == 4:
            return self._str(self._lib.ferric_gguf_meta_str, k)
        n = C.c_size_t()
        _check(self._lib.ferric_gguf_meta_arr_len(self._h, k, C.byref(n)), "gguf_meta_arr_len")
        out = []
        for i in range(n.value):
            v = C.c_double()
            if self._lib.ferric_gguf_meta_arr_f64(self._h, k, i, C.byref(v)) == _lib.OK:
                out.append(v.value)
            else:
                out.append(self._str(self._lib.ferric_gguf_meta_arr_str, k, i))
        return out

    def qmatrix(self, ctx: Context, *names: str) -> "QMatrix":
        """``qm`` / ``qm_cat`` (crates/ferric-llama/src/qwen35.rs:366-402): one weight, or several stacked along rows."""
        arr = (C.c_char_p * len(names))(*[n.encode() for n in names])
        h = C.c_void_p()
        _check(self._lib.ferric_cuda_qmatrix_from_gguf(ctx._h, self._h, arr, len(names), C.byref(h)), "qmatrix_from_gguf")
        return QMatrix(ctx, h)

    def proj(self, ctx: Context, *names: str) -> "Proj":
        """``Proj::load`` (crates/ferric-llama/src/qwen3.rs:199-208): fused when the named weights share a format, split otherwise."""
        arr = (C.c_char_p * len(names))(*[n.encode() for n in names])
        h = C.c_void_p()
        _check(self._lib.ferric_cuda_proj_from_gguf(ctx._h, self._h, arr, len(names), C.byref(h)), "proj_from_gguf")
        return Proj(ctx, h)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.ferric_gguf_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
