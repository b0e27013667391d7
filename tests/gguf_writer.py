"""Minimal GGUF v3 writer for the loader tests (little-endian; see the layout in mlx_native_b200/gguf.py)."""
import struct

import numpy as np

_TYPE_IDS = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7, "str": 8, "arr": 9, "u64": 10,
             "i64": 11, "f64": 12}
_FMT = {"u8": "B", "i8": "b", "u16": "H", "i16": "h", "u32": "I", "i32": "i", "f32": "f", "u64": "Q", "i64": "q", "f64": "d"}


def _s(text: str) -> bytes:
    b = text.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _value(kind, v) -> bytes:
    if kind in _FMT:
        return struct.pack("<" + _FMT[kind], v)
    if kind == "bool":
        return struct.pack("<B", 1 if v else 0)
    if kind == "str":
        return _s(v)
    if kind == "arr":
        ekind, items = v
        return struct.pack("<IQ", _TYPE_IDS[ekind], len(items)) + b"".join(_value(ekind, x) for x in items)
    raise ValueError(kind)


def write_gguf(path, metadata, tensors, *, magic=0x46554747, version=3, alignment=None):
    """metadata: list of (key, kind, value); tensors: list of (name, shape outermost-first, ggml type id, bytes)."""
    md = list(metadata)
    tensors = [(n, sh, tid, d if isinstance(d, (bytes, bytearray)) else np.ascontiguousarray(d).tobytes())
               for (n, sh, tid, d) in tensors]
    if alignment is not None:
        md.append(("general.alignment", "u32", alignment))
    al = alignment or 32
    head = struct.pack("<IIQQ", magic, version, len(tensors), len(md))
    for key, kind, v in md:
        head += _s(key) + struct.pack("<I", _TYPE_IDS[kind]) + _value(kind, v)
    offsets, pos = [], 0
    for _, _, _, data in tensors:
        pos = (pos + al - 1) // al * al
        offsets.append(pos)
        pos += len(data)
    for (name, shape, tid, _), off in zip(tensors, offsets):
        head += _s(name) + struct.pack("<I", len(shape))
        for d in reversed(shape):                 # the file stores the innermost dimension first
            head += struct.pack("<Q", d)
        head += struct.pack("<IQ", tid, off)
    pad = (len(head) + al - 1) // al * al - len(head)
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        for (_, _, _, data), off in zip(tensors, offsets):
            f.seek(len(head) + pad + off)
            f.write(data)
