"""ctypes front end of the CPU oracle (oracle/oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this
module; it is the checker, never the product.  The shared library is built by
`make -C oracle` (the package's build step runs that too).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

# ggml_type codes (same numbering as include/mlxn_b200.h)
F32, F16, Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, I16 = range(8)
BLOCK_VALUES = {Q4_0: 32, Q8_0: 32, Q6_K: 256, Q4_K: 256, Q5_K: 256}
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34, Q6_K: 210, Q4_K: 144, Q5_K: 176}


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        vp, sz, i32, u64 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint64
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_lcg_f32.argtypes = [u64, sz, vp]
        L.orc_dequant.argtypes = [i32, vp, sz, vp]
        L.orc_dequant.restype = i32
        L.orc_quantize.argtypes = [i32, i32, vp, sz, vp]
        L.orc_quantize.restype = i32
        L.orc_qmatmul.argtypes = [i32, vp, vp, i32, sz, sz, sz, sz, vp, vp, i32, i32]
        L.orc_qmatmul.restype = i32
        L.orc_qmatmul_id.argtypes = [i32, vp, u64, vp, vp, sz, sz, sz, sz, sz, vp, vp, i32, i32]
        L.orc_qmatmul_id.restype = i32
        L.orc_moe_map0.argtypes = [vp, sz, sz, sz, vp, vp]
        L.orc_moe_softmax_topk.argtypes = [vp, sz, sz, sz, vp, vp]
        L.orc_silu_mul.argtypes = [vp, vp, sz, vp]
        L.orc_moe_weighted_reduce.argtypes = [vp, vp, sz, sz, sz, vp]
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def lcg_f32(seed: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().orc_lcg_f32(seed, n, _p(out))
    return out


def row_bytes(ggml_type: int, k: int) -> int:
    return k // BLOCK_VALUES[ggml_type] * BLOCK_BYTES[ggml_type]


def quantize(ggml_type: int, values: np.ndarray, rule: str = "test") -> np.ndarray:
    """values: f32 [..., k] -> uint8 raw GGML blocks, rows packed back to back."""
    v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
    qk = BLOCK_VALUES[ggml_type]
    assert v.size % qk == 0
    out = np.empty(v.size // qk * BLOCK_BYTES[ggml_type], dtype=np.uint8)
    rc = lib().orc_quantize(ggml_type, 1 if rule == "ggml" else 0, _p(v), v.size, _p(out))
    assert rc == 0
    return out


def dequantize(ggml_type: int, data: np.ndarray) -> np.ndarray:
    d = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    nb = d.size // BLOCK_BYTES[ggml_type]
    out = np.empty(nb * BLOCK_VALUES[ggml_type], dtype=np.float32)
    rc = lib().orc_dequant(ggml_type, _p(d), nb, _p(out))
    assert rc == 0
    return out


def qmatmul(ggml_type: int, w: np.ndarray, x: np.ndarray, n: int, k: int, *, f16_operands: bool = False,
            nthreads: int = 1, rows: tuple[int, int] | None = None, want_absdot: bool = True):
    """Returns (y[m,n] f32, absdot[m,n] f64 or None).  Rows outside `rows` are left at zero."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1)
    m = x.shape[0]
    y = np.zeros((m, n), dtype=np.float32)
    ad = np.zeros((m, n), dtype=np.float64) if want_absdot else None
    r0, r1 = rows if rows else (0, n)
    rc = lib().orc_qmatmul(ggml_type, _p(w), _p(x), m, n, k, r0, r1, _p(y), _p(ad) if want_absdot else None,
                           int(f16_operands), nthreads)
    assert rc == 0, rc
    return y, ad


def qmatmul_id(ggml_type: int, w: np.ndarray, expert_stride: int, x: np.ndarray, ids: np.ndarray, top_k: int,
               n: int, k: int, n_experts: int, *, f16_operands: bool = False, nthreads: int = 1):
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1)
    ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
    n_tokens = x.shape[0]
    assert ids.size == n_tokens * top_k
    y = np.zeros((n_tokens * top_k, n), dtype=np.float32)
    ad = np.zeros((n_tokens * top_k, n), dtype=np.float64)
    rc = lib().orc_qmatmul_id(ggml_type, _p(w), expert_stride, _p(x), _p(ids), n_tokens, top_k, n, k, n_experts,
                              _p(y), _p(ad), int(f16_operands), nthreads)
    assert rc == 0, rc
    return y, ad


def moe_map0(ids: np.ndarray, n_tokens: int, top_k: int, n_experts: int):
    ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
    htpe = np.zeros(n_experts, dtype=np.uint32)
    hids = np.full((n_experts, n_tokens), -1, dtype=np.int32)
    lib().orc_moe_map0(_p(ids), n_tokens, top_k, n_experts, _p(htpe), _p(hids))
    return htpe, hids


def moe_softmax_topk(logits: np.ndarray, top_k: int):
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    n_tokens, n_experts = lg.shape
    ids = np.zeros((n_tokens, top_k), dtype=np.uint32)
    w = np.zeros((n_tokens, top_k), dtype=np.float32)
    lib().orc_moe_softmax_topk(_p(lg), n_tokens, n_experts, top_k, _p(ids), _p(w))
    return ids, w


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    g = np.ascontiguousarray(gate, dtype=np.float32)
    u = np.ascontiguousarray(up, dtype=np.float32)
    out = np.empty_like(g)
    lib().orc_silu_mul(_p(g), _p(u), g.size, _p(out))
    return out


def moe_weighted_reduce(y: np.ndarray, w: np.ndarray, n_tokens: int, top_k: int, h: int) -> np.ndarray:
    y = np.ascontiguousarray(y, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty((n_tokens, h), dtype=np.float32)
    lib().orc_moe_weighted_reduce(_p(y), _p(w), n_tokens, top_k, h, _p(out))
    return out
