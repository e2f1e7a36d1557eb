"""ferric_b200 -- a B200-native (sm_100a) backend for Ferric's packed-quant GGUF matmul path.

Host-side mirror of the reference's operator surface, over the C ABI in ``include/ferric_cuda.h``:

=====================================================  ===========================================
reference (dcharlot-physicalai-bmi/ferric)              here
=====================================================  ===========================================
``ferric_gguf::type_size`` / ``deq_raw``                ``type_size`` / ``Context.deq_raw``
``ferric_core::Context``                                ``Context``
``ferric_tensor::QMatrix::{block_bytes,from_bytes}``    ``QMatrix.block_bytes`` / ``QMatrix.from_bytes``
``Tensor::matmul_q`` / ``try_matmul_swiglu``            ``QMatrix.matmul`` / ``QMatrix.try_matmul_swiglu``
``Tensor::swiglu``                                      ``Context.swiglu``
``ferric_gguf::parse`` / ``GgufFile::open``, ``qm``     ``Gguf.parse`` / ``Gguf(path)``, ``Gguf.qmatrix``
``ferric_llama::Proj::{load,matmul,gate_up_swiglu}``     ``Gguf.proj`` / ``Proj.matmul`` / ``Proj.gate_up_swiglu``
=====================================================  ===========================================

PyTorch is used only for device memory and streams; all arithmetic runs in ``libferric_cuda.so``.
"""
from .ops import (Context, FerricError, Gguf, Proj, QMatrix, TPGroup, GGML_Q4_K, GGML_Q6_K, GGML_Q8_0, type_size)  # noqa: F401
