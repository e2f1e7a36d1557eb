"""A minimal GGUF writer for the tests (the reference has no writer; the layout follows the reader,
crates/ferric-gguf/src/lib.rs:105-132: magic, version, tensor count, metadata count, key / type / value
records, tensor records (name, n_dims, dims, ggml type, offset), padding to `general.alignment`, data)."""
import struct

U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def _val(ty, v) -> bytes:
    fmt = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", U64: "<Q", I64: "<q", F64: "<d"}
    if ty in fmt:
        return struct.pack(fmt[ty], v)
    if ty == BOOL:
        return struct.pack("<B", 1 if v else 0)
    if ty == STR:
        return _s(v)
    if ty == ARR:
        et, items = v
        return struct.pack("<IQ", et, len(items)) + b"".join(_val(et, x) for x in items)
    raise ValueError(ty)


def build(meta, tensors, alignment=None, version=3, pad_between=0) -> bytes:
    """meta: list of (key, type, value); tensors: list of (name, dims, ggml_type, bytes).  Returns the file bytes."""
    meta = list(meta)
    if alignment is not None:
        meta.append(("general.alignment", U32, alignment))
    align = alignment or 32
    head = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(meta))
    for k, ty, v in meta:
        head += _s(k) + struct.pack("<I", ty) + _val(ty, v)
    offsets, off = [], 0
    for _, _, _, data in tensors:
        offsets.append(off)
        off += len(data) + pad_between
        off = (off + align - 1) // align * align
    for (name, dims, ty, _), o in zip(tensors, offsets):
        head += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ty, o)
    head += b"\0" * ((len(head) + align - 1) // align * align - len(head))
    body = bytearray(off)
    for (_, _, _, data), o in zip(tensors, offsets):
        body[o:o + len(data)] = data
    return head + bytes(body)
