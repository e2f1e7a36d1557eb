"""ctypes loader for ``libferric_cuda.so`` (the C ABI declared in ``include/ferric_cuda.h``).

The library is looked for next to this file, where ``ferric_b200.build`` puts it.  There is no
fallback: if it is missing or does not load, importing the operators fails with the reason.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FERRIC_CUDA_LIB points the loader at another build of the same library (kernel A/B comparisons)
LIB_PATH = os.environ.get("FERRIC_CUDA_LIB") or os.path.join(_HERE, "libferric_cuda.so")

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED_TYPE, ERR_SHAPE, ERR_CUDA, ERR_OOM, UNSUPPORTED, ERR_TIMEOUT = range(8)
STATUS_NAMES = ["OK", "ERR_INVALID_ARG", "ERR_UNSUPPORTED_TYPE", "ERR_SHAPE", "ERR_CUDA", "ERR_OOM", "UNSUPPORTED",
                "ERR_TIMEOUT"]


class Caps(C.Structure):
    _fields_ = [("device", C.c_int32), ("sm_count", C.c_int32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("l2_bytes", C.c_uint64), ("total_mem_bytes", C.c_uint64), ("max_smem_per_block", C.c_uint64)]


_P, _SZ, _U32, _I32 = C.c_void_p, C.c_size_t, C.c_uint32, C.c_int32


class ChainLink(C.Structure):
    """``ferric_chain_link`` of include/ferric_cuda.h."""
    _fields_ = [("qm", C.c_void_p), ("swiglu", C.c_int32), ("in_slot", C.c_int32), ("in_rms", C.c_int32), ("eps", C.c_float),
                ("y_dev", C.c_void_p), ("ldy", C.c_size_t), ("next", C.c_int32), ("next_qm", C.c_void_p),
                ("h_dev", C.c_void_p), ("norm_weight_dev", C.c_void_p)]


class GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4), ("ggml_type", C.c_uint32),
                ("offset", C.c_uint64), ("n_elements", C.c_uint64), ("nbytes", C.c_uint64)]


# name -> (restype, argtypes); every symbol include/ferric_cuda.h declares
SIGNATURES = {
    "ferric_cuda_last_error": (C.c_char_p, []),
    "ferric_gguf_type_size": (_I32, [_U32, _SZ, C.POINTER(_SZ)]),
    "ferric_gguf_deq_raw": (_I32, [_P, _P, _SZ, _SZ, _U32, _P]),
    "ferric_cuda_ctx_create": (_I32, [C.c_int, C.POINTER(_P)]),
    "ferric_cuda_ctx_create_on_stream": (_I32, [C.c_int, _P, C.POINTER(_P)]),
    "ferric_cuda_ctx_set_stream": (_I32, [_P, _P]),
    "ferric_cuda_ctx_stream": (_P, [_P]),
    "ferric_cuda_ctx_sync": (_I32, [_P]),
    "ferric_cuda_ctx_free": (None, [_P]),
    "ferric_cuda_ctx_caps": (_I32, [_P, C.POINTER(Caps)]),
    "ferric_cuda_ctx_reserve_scratch": (_I32, [_P, _SZ]),
    "ferric_cuda_ctx_launches": (C.c_uint64, [_P]),
    "ferric_cuda_prof_enable": (_I32, [_P, _I32]),
    "ferric_cuda_prof": (_I32, [_P, C.c_char_p]),
    "ferric_cuda_prof_report": (_I32, [_P, _P, _SZ, C.POINTER(_SZ)]),
    "ferric_cuda_qmatrix_block_bytes": (_I32, [_U32, C.POINTER(_SZ), C.POINTER(_SZ)]),
    "ferric_cuda_qmatrix_from_bytes": (_I32, [_P, _P, _SZ, _U32, _SZ, _SZ, C.POINTER(_P)]),
    "ferric_cuda_qmatrix_from_bytes_view": (_I32, [_P, _P, _SZ, _U32, _SZ, _SZ, _SZ, _SZ, _SZ, _SZ, C.POINTER(_P)]),
    "ferric_cuda_qmatrix_from_device_bytes": (_I32, [_P, _P, _SZ, _U32, _SZ, _SZ, C.POINTER(_P)]),
    "ferric_cuda_qmatrix_from_dense": (_I32, [_P, _P, _SZ, _SZ, C.POINTER(_P)]),
    "ferric_cuda_qmatrix_rows": (_SZ, [_P]),
    "ferric_cuda_qmatrix_cols": (_SZ, [_P]),
    "ferric_cuda_qmatrix_nbytes": (_SZ, [_P]),
    "ferric_cuda_qmatrix_n_shards": (_SZ, [_P]),
    "ferric_cuda_qmatrix_ggml_type": (_U32, [_P]),
    "ferric_cuda_qmatrix_free": (None, [_P]),
    "ferric_cuda_qmatrix_scratch_bytes": (_SZ, [_P, _SZ]),
    "ferric_cuda_matmul_q": (_I32, [_P, _P, _P, _SZ, _SZ, _P]),
    "ferric_cuda_matmul_q_ld": (_I32, [_P, _P, _P, _SZ, _SZ, _SZ, _P, _SZ]),
    "ferric_cuda_prepare_x": (_I32, [_P, _P, _P, _SZ, _SZ, _SZ]),
    "ferric_cuda_matmul_q_prepared": (_I32, [_P, _P, _SZ, _P, _SZ, _I32]),
    "ferric_cuda_add_rmsnorm": (_I32, [_P, _P, _P, _P, C.c_float, _SZ, _SZ, _P, _P]),
    "ferric_cuda_add_rmsnorm_prepare": (_I32, [_P, _P, _P, _P, _P, C.c_float, _SZ, _P, _P]),
    "ferric_cuda_matmul_q_noalloc": (_I32, [_P, _P, _P, _SZ, _SZ, _P]),
    "ferric_cuda_matmul_q_bf16": (_I32, [_P, _P, _P, _SZ, _SZ, _P]),
    "ferric_cuda_gemm_status": (_I32, [_P, C.POINTER(_I32)]),
    "ferric_cuda_matmul_q_host": (_I32, [_P, _P, _P, _SZ, _SZ, _P]),
    "ferric_cuda_matmul_q_swiglu": (_I32, [_P, _P, _P, _SZ, _SZ, _P]),
    "ferric_cuda_swiglu": (_I32, [_P, _P, _SZ, _SZ, _P]),
    "ferric_cuda_matmul_q_swiglu_id": (_I32, [_P, _P, _P, _SZ, _SZ, _P, _SZ, _SZ, _P]),
    "ferric_cuda_matmul_q_id_wsum": (_I32, [_P, _P, _P, _SZ, _SZ, _SZ, _P, _SZ, _P]),
    "ferric_cuda_tp_create": (_I32, [_P, _I32, _I32, _SZ, C.POINTER(_P)]),
    "ferric_cuda_tp_export": (_I32, [_P, _P]),
    "ferric_cuda_tp_connect": (_I32, [_P, _P]),
    "ferric_cuda_tp_partial": (_P, [_P, _I32]),
    "ferric_cuda_tp_signal": (_I32, [_P, _P, _I32]),
    "ferric_cuda_tp_add_rmsnorm_prepare": (_I32, [_P, _P, _I32, _P, _P, _P, C.c_float, _SZ, _P, _P]),
    "ferric_cuda_tp_connect_local": (_I32, [_P, C.POINTER(_P)]),
    "ferric_cuda_tp_matmul_push": (_I32, [_P, _P, _I32, _P, _P, _SZ, _SZ]),
    "ferric_cuda_tp_add_rmsnorm_prepare_pushed": (_I32, [_P, _P, _I32, _P, _P, _P, C.c_float, _SZ, _P, _P]),
    "ferric_cuda_tp_allreduce_add_rmsnorm": (_I32, [_P, _P, _I32, _P, _P, _P, C.c_float, _SZ, _SZ, _P, _P]),
    "ferric_cuda_tp_allreduce_add_rmsnorm_steps": (_I32, [_P, _P, _I32, _P, _P, _P, C.c_float, _SZ, _SZ, _P, _P, _I32]),
    "ferric_cuda_tp_matmul_scatter": (_I32, [_P, _P, _I32, _P, _P, _SZ, _SZ, _P]),
    "ferric_cuda_tp_status": (_I32, [_P, _P, C.POINTER(_I32)]),
    "ferric_cuda_tp_reset": (_I32, [_P, _P]),
    "ferric_cuda_tp_chain_matmul": (_I32, [_P, _P, _I32, C.POINTER(ChainLink), _SZ]),
    "ferric_cuda_chain_reserve": (_I32, [_P, _SZ]),
    "ferric_cuda_chain_matmul": (_I32, [_P, C.POINTER(ChainLink), _SZ]),
    "ferric_cuda_tp_free": (None, [_P]),
    "ferric_gguf_parse": (_I32, [_P, _SZ, C.POINTER(_P)]),
    "ferric_gguf_open": (_I32, [C.c_char_p, C.POINTER(_P)]),
    "ferric_gguf_free": (None, [_P]),
    "ferric_gguf_n_tensors": (_SZ, [_P]),
    "ferric_gguf_data_start": (_SZ, [_P]),
    "ferric_gguf_n_meta": (_SZ, [_P]),
    "ferric_gguf_tensor_at": (_I32, [_P, _SZ, C.POINTER(GgufTensor)]),
    "ferric_gguf_tensor_by_name": (_I32, [_P, C.c_char_p, C.POINTER(GgufTensor)]),
    "ferric_gguf_raw": (_I32, [_P, C.c_char_p, C.POINTER(_P), C.POINTER(_SZ)]),
    "ferric_gguf_meta_key_at": (_I32, [_P, _SZ, _P, _SZ, C.POINTER(_SZ)]),
    "ferric_gguf_meta_kind": (_I32, [_P, C.c_char_p, C.POINTER(_I32)]),
    "ferric_gguf_meta_u64": (_I32, [_P, C.c_char_p, C.POINTER(C.c_uint64)]),
    "ferric_gguf_meta_i64": (_I32, [_P, C.c_char_p, C.POINTER(C.c_int64)]),
    "ferric_gguf_meta_f64": (_I32, [_P, C.c_char_p, C.POINTER(C.c_double)]),
    "ferric_gguf_meta_bool": (_I32, [_P, C.c_char_p, C.POINTER(_I32)]),
    "ferric_gguf_meta_str": (_I32, [_P, C.c_char_p, _P, _SZ, C.POINTER(_SZ)]),
    "ferric_gguf_meta_arr_len": (_I32, [_P, C.c_char_p, C.POINTER(_SZ)]),
    "ferric_gguf_meta_arr_str": (_I32, [_P, C.c_char_p, _SZ, _P, _SZ, C.POINTER(_SZ)]),
    "ferric_gguf_meta_arr_f64": (_I32, [_P, C.c_char_p, _SZ, C.POINTER(C.c_double)]),
    "ferric_cuda_qmatrix_from_gguf": (_I32, [_P, _P, C.POINTER(C.c_char_p), _SZ, C.POINTER(_P)]),
    "ferric_cuda_proj_from_gguf": (_I32, [_P, _P, C.POINTER(C.c_char_p), _SZ, C.POINTER(_P)]),
    "ferric_cuda_proj_from_parts": (_I32, [C.POINTER(_P), _SZ, C.POINTER(_P)]),
    "ferric_cuda_proj_n_parts": (_SZ, [_P]),
    "ferric_cuda_proj_rows": (_SZ, [_P]),
    "ferric_cuda_proj_cols": (_SZ, [_P]),
    "ferric_cuda_proj_part": (_P, [_P, _SZ]),
    "ferric_cuda_proj_free": (None, [_P]),
    "ferric_cuda_proj_matmul": (_I32, [_P, _P, _P, _SZ, _SZ, _P]),
    "ferric_cuda_proj_gate_up_swiglu": (_I32, [_P, _P, _P, _SZ, _SZ, _SZ, _P]),
    "ferric_cuda_dequant_f32": (_I32, [_P, _P, _P]),
    "ferric_cuda_dequant_bf16": (_I32, [_P, _P, _P]),
}

_lib = None


def load() -> C.CDLL:
    """Load the CUDA library and bind every declared entry point; raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is not built; run `python -m ferric_b200.build` "
                          "(this backend has no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the .so lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
