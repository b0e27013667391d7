"""GGUF v3 reader: header, metadata, tensor table, and tensor loads into device buffers.

Mirror of the upstream loader's public surface (src/gguf/mod.rs:130-160 `TensorInfo` / `GgufFile`, :784-905 `open`,
:906-950 accessors, :990-1125 `load_tensor` / `load_tensor_f32`), on this library's device and buffer types:
quantized tensors are uploaded as the raw GGML blocks the matmul kernels consume (`DType.U8`), F32 / F16 tensors as
such; `load_tensor_f32` dequantizes on the host first (Q4_0, Q8_0, Q4_K, Q6_K; the block formulas of
src/gguf/mod.rs:440-452, 582-709).  Added for multi-GPU use: `load_tensor_rows` (the N-shard of a weight matrix: a
contiguous range of rows) and `load_tensor_experts` (the experts [lo, lo + count) of a stacked [E, n, k] tensor).

File layout (all little-endian): magic "GGUF", u32 version (3), u64 tensor count, u64 metadata count, the metadata
pairs (string key, u32 value type, value), the tensor table (string name, u32 n_dims, u64 dims innermost first,
u32 GGML type id, u64 offset into the data section), padding to `general.alignment` (default 32), tensor data.
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass

import numpy as np

from .api import DType, GgmlType, MlxBuffer, MlxDevice, MlxError

GGUF_MAGIC = 0x46554747
GGUF_VERSION = 3
DEFAULT_ALIGNMENT = 32
ALIGNMENT_KEY = "general.alignment"

# GGML type ids as stored in the file (src/gguf/mod.rs:67-74) -> GgmlType
_GGML_IDS = {0: GgmlType.F32, 1: GgmlType.F16, 2: GgmlType.Q4_0, 8: GgmlType.Q8_0, 12: GgmlType.Q4_K, 13: GgmlType.Q5_K,
             14: GgmlType.Q6_K, 17: GgmlType.I16}
# (values per block, bytes per block)
_BLOCK = {GgmlType.F32: (1, 4), GgmlType.F16: (1, 2), GgmlType.I16: (1, 2), GgmlType.Q4_0: (32, 18), GgmlType.Q8_0: (32, 34),
          GgmlType.Q4_K: (256, 144), GgmlType.Q5_K: (256, 176), GgmlType.Q6_K: (256, 210)}


class GgufParseError(MlxError):
    """src/error.rs `GgufParseError`."""
    status = 8


class IoError(MlxError):
    """src/error.rs `IoError`."""
    status = 7


@dataclass(frozen=True)
class TensorInfo:
    name: str
    shape: tuple          # outermost dimension first (the file stores innermost first; reversed on read, as upstream)
    ggml_type: GgmlType
    offset: int           # relative to the start of the tensor data section
    byte_len: int


class _Reader:
    def __init__(self, f):
        self.f = f

    def take(self, n: int) -> bytes:
        b = self.f.read(n)
        if len(b) != n:
            raise GgufParseError(f"GGUF parse error: unexpected end of file (wanted {n} bytes, got {len(b)})")
        return b

    def num(self, fmt: str):
        return struct.unpack("<" + fmt, self.take(struct.calcsize("<" + fmt)))[0]

    def string(self) -> str:
        n = self.num("Q")
        if n > 1 << 24:
            raise GgufParseError(f"GGUF parse error: string length {n} exceeds the 16 MiB safety limit")
        return self.take(n).decode("utf-8", "replace")


_SCALARS = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 10: "Q", 11: "q", 12: "d"}


def _read_value(r: _Reader, vtype: int, depth: int = 0):
    if vtype in _SCALARS:
        return r.num(_SCALARS[vtype])
    if vtype == 7:
        return r.num("B") != 0
    if vtype == 8:
        return r.string()
    if vtype == 9:
        if depth > 4:
            raise GgufParseError("GGUF parse error: metadata arrays nested too deeply")
        etype, count = r.num("I"), r.num("Q")
        if count > 1 << 26:
            raise GgufParseError(f"GGUF parse error: array length {count} exceeds the safety limit")
        return [_read_value(r, etype, depth + 1) for _ in range(count)]
    raise GgufParseError(f"GGUF parse error: unknown metadata value type {vtype}")


def compute_byte_len(shape, ggml_type: GgmlType) -> int:
    """Bytes of a tensor: the element count must be a whole number of blocks (src/gguf/mod.rs:320-338)."""
    qk, bb = _BLOCK[ggml_type]
    total = 1
    for d in shape:
        total *= int(d)
    if total == 0:
        return 0
    if total % qk:
        raise GgufParseError(f"GGUF parse error: total elements {total} not divisible by block size {qk} for type "
                             f"{ggml_type.name}")
    return total // qk * bb


def _align(pos: int, alignment: int) -> int:
    return (pos + alignment - 1) // alignment * alignment


class GgufFile:
    """A parsed GGUF file; tensor data is read on demand (the file stays open)."""

    def __init__(self, path, metadata, tensors, tensor_data_offset, fh):
        self.path = path
        self._metadata = metadata
        self._tensors = tensors
        self.tensor_data_offset = tensor_data_offset
        self._fh = fh

    # ---- src/gguf/mod.rs:784-905
    @classmethod
    def open(cls, path) -> "GgufFile":
        try:
            fh = open(path, "rb")
        except OSError as ex:
            raise IoError(f"IO error: cannot open GGUF file '{path}': {ex}") from None
        try:
            r = _Reader(fh)
            magic = r.num("I")
            if magic != GGUF_MAGIC:
                raise GgufParseError(f"GGUF parse error: bad magic: expected 0x{GGUF_MAGIC:08X}, got 0x{magic:08X}")
            version = r.num("I")
            if version != GGUF_VERSION:
                raise GgufParseError(f"GGUF parse error: unsupported GGUF version {version} (only v3 is supported)")
            tensor_count, kv_count = r.num("Q"), r.num("Q")
            if tensor_count > 100_000:
                raise GgufParseError(f"GGUF parse error: tensor_count {tensor_count} exceeds 100k safety limit")
            if kv_count > 1_000_000:
                raise GgufParseError(f"GGUF parse error: metadata_kv_count {kv_count} exceeds 1M safety limit")
            metadata = {}
            for _ in range(kv_count):
                key = r.string()
                vtype = r.num("I")
                metadata[key] = (vtype, _read_value(r, vtype))
            alignment = DEFAULT_ALIGNMENT
            if ALIGNMENT_KEY in metadata:
                v = _as_u32(metadata[ALIGNMENT_KEY])
                if v is not None:
                    alignment = v
            if alignment == 0 or alignment & (alignment - 1):
                raise GgufParseError(f"GGUF parse error: alignment {alignment} is not a power of two")
            tensors = {}
            for _ in range(tensor_count):
                name = r.string()
                n_dims = r.num("I")
                if n_dims > 8:
                    raise GgufParseError(f"GGUF parse error: tensor '{name}' has {n_dims} dimensions (max 8)")
                shape = tuple(reversed([r.num("Q") for _ in range(n_dims)]))
                type_id = r.num("I")
                if type_id not in _GGML_IDS:
                    raise GgufParseError(f"GGUF parse error: tensor '{name}': unsupported GGML type ID {type_id}")
                gt = _GGML_IDS[type_id]
                offset = r.num("Q")
                try:
                    blen = compute_byte_len(shape, gt)
                except GgufParseError as ex:
                    raise GgufParseError(f"GGUF parse error: tensor '{name}': {str(ex).replace('GGUF parse error: ', '')}") from None
                tensors[name] = TensorInfo(name, shape, gt, offset, blen)
            data_off = _align(fh.tell(), alignment)
        except Exception:
            fh.close()
            raise
        return cls(path, metadata, tensors, data_off, fh)

    def close(self) -> None:
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- accessors, src/gguf/mod.rs:906-950
    def metadata(self, key: str):
        """The value (Python int / float / bool / str / list) or None."""
        v = self._metadata.get(key)
        return None if v is None else v[1]

    def metadata_string(self, key: str):
        v = self._metadata.get(key)
        return v[1] if v is not None and v[0] == 8 else None

    def metadata_u32(self, key: str):
        v = self._metadata.get(key)
        return None if v is None else _as_u32(v)

    def metadata_f32(self, key: str):
        v = self._metadata.get(key)
        return float(np.float32(v[1])) if v is not None and v[0] in (6, 12) else None

    def tensor_names(self):
        return list(self._tensors)

    def tensor_info(self, name: str):
        return self._tensors.get(name)

    def tensor_count(self) -> int:
        return len(self._tensors)

    def metadata_count(self) -> int:
        return len(self._metadata)


def _as_u32(typed):
    """`MetadataValue::as_u32` (src/gguf/mod.rs:108-117): u32, u8, u16, or a non-negative i32."""
    vtype, v = typed
    if vtype in (4, 0, 2):
        return int(v)
    if vtype == 5 and v >= 0:
        return int(v)
    return None


# ---------------------------------------------------------------------------------------- host-side dequantizers
def _f16(b: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b).view(np.float16).astype(np.float32)


def dequantize_to_f32(data: np.ndarray, ggml_type: GgmlType) -> np.ndarray:
    """Raw tensor bytes -> f32 values (src/gguf/mod.rs:362-780).  Every product and difference is rounded in f32, in
    the order upstream evaluates them."""
    d8 = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    f32 = np.float32
    if ggml_type == GgmlType.F32:
        return d8.view(np.float32).copy()
    if ggml_type == GgmlType.F16:
        return d8.view(np.float16).astype(np.float32)
    if ggml_type == GgmlType.I16:
        return d8.view(np.int16).astype(np.float32)
    if ggml_type == GgmlType.Q4_0:
        b = d8.reshape(-1, 18)
        d = _f16(b[:, 0:2])                                            # [nb, 1]
        q = np.concatenate([b[:, 2:] & 0x0F, b[:, 2:] >> 4], axis=1).astype(np.int32) - 8
        return (d * q.astype(f32)).astype(f32).reshape(-1)
    if ggml_type == GgmlType.Q8_0:
        b = d8.reshape(-1, 34)
        return (_f16(b[:, 0:2]) * b[:, 2:].view(np.int8).astype(f32)).astype(f32).reshape(-1)
    if ggml_type == GgmlType.Q4_K:
        b = d8.reshape(-1, 144)
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])                     # [nb, 1]
        s = b[:, 4:16].astype(np.uint32)
        sc = np.concatenate([s[:, 0:4] & 63, (s[:, 8:12] & 0x0F) | ((s[:, 0:4] >> 6) << 4)], axis=1)     # [nb, 8]
        mn = np.concatenate([s[:, 4:8] & 63, (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)], axis=1)
        qs = b[:, 16:].reshape(-1, 4, 32)
        q = np.stack([qs & 0x0F, qs >> 4], axis=2).reshape(-1, 8, 32).astype(f32)                        # sub-block order
        dj = (d * sc.astype(f32)).astype(f32)[:, :, None]
        mj = (dmin * mn.astype(f32)).astype(f32)[:, :, None]
        return ((dj * q).astype(f32) - mj).astype(f32).reshape(-1)
    if ggml_type == GgmlType.Q5_K:
        b = d8.reshape(-1, 176)                                        # src/gguf/mod.rs:469-541
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        s = b[:, 4:16].astype(np.uint32)
        sc = np.concatenate([s[:, 0:4] & 63, (s[:, 8:12] & 0x0F) | ((s[:, 0:4] >> 6) << 4)], axis=1)     # [nb, 8]
        mn = np.concatenate([s[:, 4:8] & 63, (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)], axis=1)
        qh = b[:, 16:48]                                                                                 # [nb, 32]
        qs = b[:, 48:].reshape(-1, 4, 32)
        lo = np.stack([qs & 0x0F, qs >> 4], axis=2).reshape(-1, 8, 32)
        hi = (qh[:, None, :] >> np.arange(8, dtype=np.uint8)[None, :, None]) & 1                         # sub-block j: bit j
        q = (lo + 16 * hi).astype(f32)
        dj = (d * sc.astype(f32)).astype(f32)[:, :, None]
        mj = (dmin * mn.astype(f32)).astype(f32)[:, :, None]
        return ((dj * q).astype(f32) - mj).astype(f32).reshape(-1)
    if ggml_type == GgmlType.Q6_K:
        b = d8.reshape(-1, 210)
        nb = b.shape[0]
        ql = b[:, 0:128].reshape(nb, 2, 2, 32).astype(np.int32)        # [block, half, (l | l+32), l]
        qh = b[:, 128:192].reshape(nb, 2, 32).astype(np.int32)
        sc = b[:, 192:208].view(np.int8).reshape(nb, 2, 8).astype(f32)
        d = _f16(b[:, 208:210]).reshape(nb, 1, 1)
        q = np.empty((nb, 2, 4, 32), dtype=np.int32)
        q[:, :, 0] = (ql[:, :, 0] & 0x0F) | ((qh & 3) << 4)
        q[:, :, 1] = (ql[:, :, 1] & 0x0F) | (((qh >> 2) & 3) << 4)
        q[:, :, 2] = (ql[:, :, 0] >> 4) | (((qh >> 4) & 3) << 4)
        q[:, :, 3] = (ql[:, :, 1] >> 4) | (((qh >> 6) & 3) << 4)
        q -= 32
        # scale of element (half, quarter g, l): sc[half][2 g + l / 16]
        idx = (2 * np.arange(4)[:, None] + (np.arange(32)[None, :] >> 4))                               # [4, 32]
        scale = sc[:, :, idx]                                                                           # [nb, 2, 4, 32]
        ds = (d[:, :, :, None] * scale).astype(f32)
        return (ds * q.astype(f32)).astype(f32).reshape(-1)
    raise GgufParseError(f"GGUF parse error: no host dequantizer for {ggml_type.name}")


_DEVICE_DTYPE = {GgmlType.F32: DType.F32, GgmlType.F16: DType.F16}


def _read_bytes(self: GgufFile, info: TensorInfo, start: int = 0, length: int | None = None) -> np.ndarray:
    n = info.byte_len - start if length is None else length
    try:
        self._fh.seek(self.tensor_data_offset + info.offset + start)
        raw = self._fh.read(n)
    except OSError as ex:
        raise IoError(f"IO error: read tensor '{info.name}': {ex}") from None
    if len(raw) != n:
        raise IoError(f"IO error: read tensor '{info.name}' ({n} bytes at offset "
                      f"{self.tensor_data_offset + info.offset + start}): unexpected end of file")
    return np.frombuffer(raw, dtype=np.uint8)


def _info(self: GgufFile, name: str) -> TensorInfo:
    info = self._tensors.get(name)
    if info is None:
        raise GgufParseError(f"GGUF parse error: tensor '{name}' not found in GGUF file")
    return info


def _to_device(device: MlxDevice, raw: np.ndarray, ggml_type: GgmlType, shape) -> MlxBuffer:
    if raw.size == 0:
        raise GgufParseError("GGUF parse error: tensor has zero bytes")
    buf = device.alloc_buffer(raw.size, _DEVICE_DTYPE.get(ggml_type, DType.U8), list(shape))
    buf.upload(raw)
    return buf


def load_tensor(self: GgufFile, name: str, device: MlxDevice) -> MlxBuffer:
    """src/gguf/mod.rs:990-1060: the tensor's bytes in a device buffer (raw GGML blocks as U8; F32 / F16 typed)."""
    info = _info(self, name)
    return _to_device(device, _read_bytes(self, info), info.ggml_type, info.shape)


def load_tensor_f32(self: GgufFile, name: str, device: MlxDevice) -> MlxBuffer:
    """src/gguf/mod.rs:1066-1095: dequantized on the host, uploaded as F32."""
    info = _info(self, name)
    total = int(np.prod(info.shape)) if info.shape else 0
    if total == 0:
        raise GgufParseError(f"GGUF parse error: tensor '{name}' has zero elements")
    vals = dequantize_to_f32(_read_bytes(self, info), info.ggml_type)
    buf = device.alloc_buffer(total * 4, DType.F32, list(info.shape))
    buf.upload(vals)
    return buf


def load_tensor_rows(self: GgufFile, name: str, device: MlxDevice, rank: int, world: int) -> MlxBuffer:
    """The N-shard of a [n, k] weight matrix: rows [rank n / world, (rank + 1) n / world), one contiguous byte range of
    the file (rows are whole numbers of blocks).  No upstream counterpart (it runs on one GPU)."""
    info = _info(self, name)
    if len(info.shape) != 2:
        raise GgufParseError(f"GGUF parse error: tensor '{name}' is not a matrix (shape {info.shape})")
    n, k = info.shape
    qk, bb = _BLOCK[info.ggml_type]
    if k % qk or n % world:
        raise GgufParseError(f"GGUF parse error: tensor '{name}' [{n} x {k}] cannot be split into {world} row shards")
    row_bytes, per = k // qk * bb, n // world
    raw = _read_bytes(self, info, rank * per * row_bytes, per * row_bytes)
    return _to_device(device, raw, info.ggml_type, (per, k))


def load_tensor_experts(self: GgufFile, name: str, device: MlxDevice, rank: int, world: int) -> MlxBuffer:
    """The expert shard of a stacked [E, n, k] tensor: experts [rank E / world, (rank + 1) E / world)."""
    info = _info(self, name)
    if len(info.shape) != 3:
        raise GgufParseError(f"GGUF parse error: tensor '{name}' is not a stack of matrices (shape {info.shape})")
    e, n, k = info.shape
    qk, bb = _BLOCK[info.ggml_type]
    if k % qk or e % world:
        raise GgufParseError(f"GGUF parse error: tensor '{name}' [{e} x {n} x {k}] cannot be split into {world} expert shards")
    stride, per = n * (k // qk) * bb, e // world
    raw = _read_bytes(self, info, rank * per * stride, per * stride)
    return _to_device(device, raw, info.ggml_type, (per, n, k))


def load_tensor_into_pool(self: GgufFile, name: str, device: MlxDevice, pool) -> MlxBuffer:
    """src/gguf/mod.rs:1127-1137: `load_tensor`, then the buffer is registered with the pool so that the pool's residency
    accounting covers the weights (on this device every allocation is already resident: the registration only records
    it).  Errors: those of `load_tensor`, plus InvalidArgument from `register_existing`."""
    buf = load_tensor(self, name, device)
    pool.register_existing(device, buf)
    return buf


GgufFile.load_tensor = load_tensor
GgufFile.load_tensor_into_pool = load_tensor_into_pool
GgufFile.load_tensor_f32 = load_tensor_f32
GgufFile.load_tensor_rows = load_tensor_rows
GgufFile.load_tensor_experts = load_tensor_experts
GgufFile.read_tensor_bytes = lambda self, name: _read_bytes(self, _info(self, name))
