"""Host-side GGML block packers (numpy): f32 values -> Q4_0 / Q8_0 / Q6_K block bytes.

The kernels consume GGML blocks as they sit in a GGUF file; these helpers make such blocks from f32 data for
synthetic workloads and examples (upstream has no quantizer in its library either: its tests carry their own,
tests/test_quantized_matmul_ggml.rs:37-60, 99-116, 137-324).  Layouts (src/ops/quantized_matmul_ggml.rs:48-97):

  Q4_0  18 bytes / 32 values: f16 d, 16 bytes of nibbles (value i in the low nibble of byte i, value i+16 in the high one);
        w = d * (q - 8).  Rule: the element of largest magnitude maps to -8 (d = that element / -8), q = min(15, trunc(x/d + 8.5)).
  Q8_0  34 bytes / 32 values: f16 d, 32 int8; w = d * q, d = amax / 127, q = round(x / d).
  Q6_K  210 bytes / 256 values: ql[128] low nibbles, qh[64] high 2 bits, int8 scales[16], f16 d; w = d * sc * (q - 32);
        d = largest 16-group amax / (32 * 127), sc = round(amax_g / d / 32), q = round(x / (d sc) + 32) in [0, 63].
"""
from __future__ import annotations

import numpy as np

Q4_0, Q8_0, Q6_K = 2, 3, 6           # the values of `GgmlType` (src/ops/quantized_matmul_ggml.rs:48-63, declaration order)
BLOCK_VALUES = {Q4_0: 32, Q8_0: 32, Q6_K: 256}
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34, Q6_K: 210}


def _round_half_away(a: np.ndarray) -> np.ndarray:
    return np.copysign(np.floor(np.abs(a) + np.float32(0.5)), a)


def _inv(d: np.ndarray) -> np.ndarray:
    with np.errstate(divide="ignore"):
        return np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)


def _f16_bytes(d: np.ndarray) -> np.ndarray:
    return d.astype(np.float16).view(np.uint8).reshape(-1, 2)


def pack_q4_0(values: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(values, dtype=np.float32).reshape(-1, 32)
    idx = np.argmax(np.abs(x), axis=1)                       # first element of largest magnitude
    mx = x[np.arange(x.shape[0]), idx]
    d = (mx / np.float32(-8.0)).astype(np.float32)
    q = (x * _inv(d)[:, None] + np.float32(8.5)).astype(np.float32)
    q = np.clip(np.trunc(q), 0, 15).astype(np.uint8)
    out = np.empty((x.shape[0], 18), dtype=np.uint8)
    out[:, 0:2] = _f16_bytes(d)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def pack_q8_0(values: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(values, dtype=np.float32).reshape(-1, 32)
    d = (np.max(np.abs(x), axis=1) / np.float32(127.0)).astype(np.float32)
    q = np.clip(_round_half_away((x * _inv(d)[:, None]).astype(np.float32)), -128, 127).astype(np.int8)
    out = np.empty((x.shape[0], 34), dtype=np.uint8)
    out[:, 0:2] = _f16_bytes(d)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def pack_q6_k(values: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(values, dtype=np.float32).reshape(-1, 16, 16)     # [block, group, 16]
    nb = x.shape[0]
    amax = np.max(np.abs(x), axis=2)                                           # [block, 16]
    d = (np.max(amax, axis=1) / np.float32(32.0 * 127.0)).astype(np.float32)
    idd = _inv(d)
    sc = np.where(amax != 0, np.clip(_round_half_away((amax * idd[:, None] / np.float32(32.0)).astype(np.float32)), -128, 127), 0)
    sc = sc.astype(np.int8)
    sub_d = (d[:, None] * sc.astype(np.float32)).astype(np.float32)
    q = np.clip(_round_half_away((x * _inv(sub_d)[:, :, None] + np.float32(32.0)).astype(np.float32)), 0, 63).astype(np.uint8)
    q = q.reshape(nb, 2, 4, 32)                                                # [block, half, quarter v0..v3, l]
    out = np.empty((nb, 210), dtype=np.uint8)
    ql = out[:, :128].reshape(nb, 2, 2, 32)                                    # [block, half, (l | l+32), l]
    ql[:, :, 0, :] = (q[:, :, 0] & 0x0F) | ((q[:, :, 2] & 0x0F) << 4)
    ql[:, :, 1, :] = (q[:, :, 1] & 0x0F) | ((q[:, :, 3] & 0x0F) << 4)
    qh = out[:, 128:192].reshape(nb, 2, 32)
    qh[:] = ((q[:, :, 0] >> 4) & 3) | (((q[:, :, 1] >> 4) & 3) << 2) | (((q[:, :, 2] >> 4) & 3) << 4) | (((q[:, :, 3] >> 4) & 3) << 6)
    out[:, 192:208] = sc.view(np.uint8)
    out[:, 208:210] = _f16_bytes(d)
    return out.reshape(-1)


def pack(ggml_type: int, values: np.ndarray) -> np.ndarray:
    """Block bytes (uint8, 1-D) of `values` (f32, size a multiple of the type's block length)."""
    t = int(ggml_type)
    if t not in BLOCK_VALUES:
        raise ValueError(f"unsupported GGML type {ggml_type}")
    if values.size % BLOCK_VALUES[t] != 0:
        raise ValueError(f"{values.size} values is not a multiple of the block length {BLOCK_VALUES[t]}")
    return {Q4_0: pack_q4_0, Q8_0: pack_q8_0, Q6_K: pack_q6_k}[t](values)


# Block geometry by type name: (values per block, bytes per block, byte offset of the f16 scale d)
BLOCK_GEOMETRY = {"Q4_0": (32, 18, 0), "Q8_0": (32, 34, 0), "Q6_K": (256, 210, 208), "Q4_K": (256, 144, 0)}


def random_blocks(rng, type_name: str, n: int, k: int) -> np.ndarray:
    """n x k weights as random block bytes with finite f16 scales in a small range.  For timing and memory-traffic
    runs only: the kernels' speed does not depend on the values, and packing 600 MB of real weights takes minutes."""
    qk, bb, dpos = BLOCK_GEOMETRY[type_name]
    raw = rng.integers(0, 256, size=(n * (k // qk), bb), dtype=np.uint8)
    raw[:, dpos + 1] = (raw[:, dpos + 1] & 0x83) | 0x20   # f16 scale exponent in a small finite range
    if type_name == "Q4_K":
        raw[:, 3] = (raw[:, 3] & 0x83) | 0x20             # ... and the f16 dmin behind it
    return raw.reshape(-1)
