"""A minimal GGUF v3 writer for the tests (the container layout of the public GGUF specification: header, metadata
key-value pairs, tensor infos, padding to general.alignment, tensor data).  Test infrastructure only."""
import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)


def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def _value(t: int, v) -> bytes:
    fmt = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}
    if t in fmt:
        return struct.pack(fmt[t], v)
    if t == STR:
        return _s(v.encode() if isinstance(v, str) else v)
    if t == ARR:
        et, items = v
        return struct.pack("<IQ", et, len(items)) + b"".join(_value(et, x) for x in items)
    raise ValueError(t)


def write_gguf(path, metadata, tensors, alignment=32, version=3, magic=b"GGUF", pad_tail=0):
    """metadata: list of (key, type, value); tensors: list of (name, dims (fastest axis first), ggml_type, bytes)."""
    out = bytearray()
    out += magic + struct.pack("<IQQ", version, len(tensors), len(metadata))
    for k, t, v in metadata:
        out += _s(k.encode()) + struct.pack("<I", t) + _value(t, v)
    off = 0
    offsets = []
    tensors = [(n, d, t, np.ascontiguousarray(a).tobytes()) for n, d, t, a in tensors]
    for name, dims, gt, data in tensors:
        out += _s(name.encode()) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", gt, off)
        offsets.append(off)
        off += (len(data) + alignment - 1) // alignment * alignment
    out += b"\0" * ((-len(out)) % alignment)
    base = len(out)
    for (name, dims, gt, data), o in zip(tensors, offsets):
        out += b"\0" * (base + o - len(out))
        out += data
    out += b"\0" * pad_tail
    with open(path, "wb") as f:
        f.write(out)
    return bytes(out)
