"""The C-ABI library builds, loads and exports every symbol the public header declares.

No compute calls: these run without a GPU.  On a GPU-less host the context constructor must fail
loudly (there is no CPU fallback behind the ABI)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from ferric_b200 import build, _lib
    build.build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ferric_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ferric_(?:cuda|gguf)_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(lib):
    from ferric_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in ferric_cuda.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_type_size_matches_reference_table(lib):
    import ferric_b200 as F
    assert F.type_size(12, 4096 * 4096) == 9_437_184
    assert F.type_size(14, 151936 * 5120) == 638_131_200
    assert F.type_size(8, 64) == 68
    assert F.type_size(0, 8) == 32 and F.type_size(1, 8) == 16 and F.type_size(30, 8) == 16
    with pytest.raises(F.FerricError) as e:
        F.type_size(99, 256)
    assert e.value.status == 2 and "unsupported ggml type 99" in str(e.value)


def test_block_bytes_table(lib):
    # crates/ferric-tensor/src/dtype.rs:4207-4214: 8 / 12 / 14 are packed; float types are dense by design
    import ferric_b200 as F
    assert F.QMatrix.block_bytes(8) == (32, 34)
    assert F.QMatrix.block_bytes(12) == (256, 144)
    assert F.QMatrix.block_bytes(14) == (256, 210)
    for ty in (0, 1, 30, 35, 41):
        assert F.QMatrix.block_bytes(ty) is None


def test_null_handles_are_rejected_not_dereferenced(lib):
    h = C.c_void_p()
    assert lib.ferric_cuda_qmatrix_from_bytes(None, None, 0, 12, 0, 0, C.byref(h)) == 1
    assert lib.ferric_cuda_matmul_q(None, None, None, 1, 256, None) == 1
    assert lib.ferric_cuda_ctx_sync(None) == 1
    assert lib.ferric_cuda_qmatrix_rows(None) == 0
    lib.ferric_cuda_qmatrix_free(None)
    lib.ferric_cuda_ctx_free(None)
    assert b"NULL" in lib.ferric_cuda_last_error()


def test_no_gpu_means_a_loud_failure_not_a_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.ferric_cuda_ctx_create(0, C.byref(h)) == 4
    assert not h.value
    assert b"no CPU fallback" in lib.ferric_cuda_last_error()


def test_product_package_does_not_touch_the_oracle():
    pkg = os.path.join(ROOT, "ferric_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"
