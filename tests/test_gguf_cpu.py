"""GGUF ingest on the CPU: the parser against files built by tests/gguf_writer.py, and the behaviours the reference's
reader pins (crates/ferric-gguf/src/lib.rs:105-132, :387-431): total over arbitrary bytes, "not a GGUF file",
"GGUF header truncated or malformed", `general.alignment`, tensor bytes exactly as stored, the two stride refusals."""
import os
import struct

import numpy as np
import pytest

import gguf_writer as W
from ferric_b200 import synth
from ferric_b200.ops import FerricError, Gguf

META = [("general.architecture", W.STR, "qwen3"), ("qwen3.block_count", W.U32, 2), ("x.i8", W.I8, -5), ("x.u16", W.U16, 65535),
        ("x.i16", W.I16, -300), ("x.i32", W.I32, -70000), ("x.u64", W.U64, 2 ** 40), ("x.i64", W.I64, -2 ** 40),
        ("x.f32", W.F32, 0.5), ("x.f64", W.F64, 1e-300), ("x.bool", W.BOOL, True), ("x.u8", W.U8, 200),
        ("tokenizer.ggml.tokens", W.ARR, (W.STR, ["<s>", "hello", "wörld"])), ("x.arr_f32", W.ARR, (W.F32, [1.0, -2.5])),
        ("x.arr_i32", W.ARR, (W.I32, [3, -4, 5]))]


def tensors(rng):
    q4 = synth.q4k_blocks(rng, 4 * 512 // 256).tobytes()       # [out 4, in 512] listed as dims [512, 4]
    q6 = synth.q6k_blocks(rng, 3 * 256 // 256).tobytes()
    q8 = synth.q8_0_blocks(rng, 5 * 64 // 32).tobytes()
    f32 = np.arange(7, dtype=np.float32).tobytes()
    return [("blk.0.attn_q.weight", [512, 4], 12, q4), ("blk.0.ffn_down.weight", [256, 3], 14, q6),
            ("blk.0.attn_k.weight", [64, 5], 8, q8), ("output_norm.weight", [7], 0, f32)]


def test_parse_metadata_and_tensors():
    rng = np.random.default_rng(0)
    ts = tensors(rng)
    g = Gguf.parse(W.build(META, ts))
    assert g.metadata["general.architecture"] == "qwen3" and g.metadata["qwen3.block_count"] == 2
    assert g.metadata["x.i8"] == -5 and g.metadata["x.u16"] == 65535 and g.metadata["x.i16"] == -300
    assert g.metadata["x.i32"] == -70000 and g.metadata["x.u64"] == 2 ** 40 and g.metadata["x.i64"] == -2 ** 40
    assert g.metadata["x.f32"] == 0.5 and g.metadata["x.f64"] == 1e-300 and g.metadata["x.bool"] is True and g.metadata["x.u8"] == 200
    assert g.metadata["tokenizer.ggml.tokens"] == ["<s>", "hello", "wörld"]
    assert g.metadata["x.arr_f32"] == [1.0, -2.5] and g.metadata["x.arr_i32"] == [3.0, -4.0, 5.0]
    assert list(g.metadata)[:2] == ["general.architecture", "qwen3.block_count"]          # file order kept
    assert [t["name"] for t in g.tensors] == [t[0] for t in ts]
    assert g.data_start % 32 == 0
    for (name, dims, ty, data), info in zip(ts, g.tensors):
        assert info["dims"] == dims and info["ggml_type"] == ty and info["nbytes"] == len(data)
        assert info["offset"] % 32 == 0
        assert g.raw(name).tobytes() == data                                               # exactly as stored
        assert g.tensor(name) == info
    assert g.tensor("nope") is None
    with pytest.raises(FerricError, match="no tensor 'nope'"):
        g.raw("nope")
    g.close()


@pytest.mark.parametrize("align", [32, 64, 4096])
def test_alignment_key_moves_the_data_section(align):
    rng = np.random.default_rng(1)
    ts = tensors(rng)
    g = Gguf.parse(W.build(META, ts, alignment=align))
    assert g.data_start % align == 0
    assert all(t["offset"] % align == 0 for t in g.tensors)
    for name, _, _, data in ts:
        assert g.raw(name).tobytes() == data


def test_open_maps_a_file(tmp_path):
    rng = np.random.default_rng(2)
    ts = tensors(rng)
    big = META + [("tokenizer.ggml.merges", W.ARR, (W.STR, ["a b"] * 50000))]            # a header of over a megabyte
    path = os.path.join(tmp_path, "m.gguf")
    with open(path, "wb") as f:
        f.write(W.build(big, ts))
    g = Gguf(path)
    assert len(g.metadata["tokenizer.ggml.merges"]) == 50000
    for name, _, _, data in ts:
        assert g.raw(name).tobytes() == data
    g.close()
    with pytest.raises(FerricError, match="cannot open"):
        Gguf(os.path.join(tmp_path, "missing.gguf"))


def test_rejects_what_is_not_gguf():
    with pytest.raises(FerricError, match="not a GGUF file"):
        Gguf.parse(b"GGML" + b"\0" * 64)
    with pytest.raises(FerricError, match="not a GGUF file"):
        Gguf.parse(b"GG")


def test_truncated_or_malformed_headers_are_rejected_not_trusted():
    rng = np.random.default_rng(3)
    data = W.build(META, tensors(rng))
    g = Gguf.parse(data)
    header_len = g.data_start
    g.close()
    for cut in list(range(4, 64)) + list(range(64, header_len - 40, 37)):
        with pytest.raises(FerricError, match="truncated or malformed"):
            Gguf.parse(data[:cut])
    # a string length, an array count and a tensor count far beyond the file must not allocate or read out of bounds
    bad = bytearray(data)
    bad[24:32] = struct.pack("<Q", 2 ** 62)                       # length of the first key
    with pytest.raises(FerricError, match="truncated or malformed"):
        Gguf.parse(bytes(bad))
    bad = bytearray(data)
    bad[8:16] = struct.pack("<Q", 2 ** 40)                        # tensor count
    with pytest.raises(FerricError, match="truncated or malformed"):
        Gguf.parse(bytes(bad))
    bad = W.build([("k", 99, 0)] if False else [], [])            # unknown metadata value type
    bad = b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + W._s("k") + struct.pack("<I", 99)
    with pytest.raises(FerricError, match="truncated or malformed"):
        Gguf.parse(bad)


def test_random_bytes_never_fault():
    rng = np.random.default_rng(4)
    for n in (0, 1, 7, 24, 100, 5000):
        blob = b"GGUF" + rng.integers(0, 256, n, dtype=np.uint8).tobytes()
        try:
            Gguf.parse(blob).close()
        except FerricError:
            pass


def test_stride_guards():
    rng = np.random.default_rng(5)
    q4 = synth.q4k_blocks(rng, 8).tobytes()                       # 8 super-blocks = 1152 bytes
    f32 = np.zeros(8, dtype=np.float32).tobytes()
    # declared larger than the file leaves before the next tensor: the reader's stride is too big for this file
    with pytest.raises(FerricError, match="leaves only"):
        Gguf.parse(W.build([], [("a", [256, 16], 12, q4), ("b", [8], 0, f32)]))
    # the last tensor running past the end of the file
    with pytest.raises(FerricError, match="leaves only"):
        Gguf.parse(W.build([], [("b", [8], 0, f32), ("a", [256, 16], 12, q4)]))
    # more than twice the bytes reserved (and far beyond padding): the reader's stride is too small
    with pytest.raises(FerricError, match="more than twice"):
        Gguf.parse(W.build([], [("a", [256, 2], 12, q4), ("b", [8], 0, f32)]))
    # ordinary padding between tensors is fine, and so is a type this library has no layout for (it fails when read)
    g = Gguf.parse(W.build([], [("a", [256, 8], 12, q4), ("odd", [32], 2, b"\0" * 18), ("b", [8], 0, f32)], pad_between=40))
    assert g.tensor("odd")["nbytes"] == 0
    with pytest.raises(FerricError):
        g.raw("odd")
    assert g.raw("a").tobytes() == q4


def test_dims_whose_product_wraps_are_refused_before_any_size_arithmetic():
    """Hostile dims: rows = 2^60 + 1 with 256 columns of Q4_K multiply to a byte count that wraps to 144 in 64 bits and
    would pass every later length check; the parser refuses the header (status FERRIC_ERR_SHAPE), so no allocation is
    sized and no kernel is launched from such a record.  The matrix constructor applies the same rule to its own
    arguments, which needs no device: it fails on the size before it looks for one."""
    rng = np.random.default_rng(6)
    q4 = synth.q4k_blocks(rng, 1).tobytes()                        # 144 bytes: what the wrapped product asks for
    for dims in ([256, 2 ** 60 + 1], [2 ** 32, 2 ** 32], [2 ** 63, 2], [256, 2 ** 63]):
        with pytest.raises(FerricError) as e:
            Gguf.parse(W.build([], [("a", dims, 12, q4)]))
        assert e.value.status == 3 and "overflow" in str(e.value)
    # an honest large count still parses (it is then refused for not fitting the file)
    with pytest.raises(FerricError, match="leaves only"):
        Gguf.parse(W.build([], [("a", [256, 2 ** 40], 12, q4)]))
    from ferric_b200 import _lib
    import ctypes as C
    lib = _lib.load()
    out = C.c_size_t(0)
    assert lib.ferric_gguf_type_size(0, 2 ** 63, C.byref(out)) == 3          # n * 4 would wrap
    assert lib.ferric_gguf_type_size(12, 2 ** 63, C.byref(out)) == 0 and out.value == 2 ** 63 // 256 * 144
