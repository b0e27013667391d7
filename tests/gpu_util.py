"""Helpers shared by the GPU parity tests: seeded inputs, calls through the C ABI, parity metrics."""
from __future__ import annotations

import numpy as np

import mlx_native_b200 as mx
from oracle import oracle as orc

TYPES = {"Q4_0": (mx.GgmlType.Q4_0, orc.Q4_0), "Q8_0": (mx.GgmlType.Q8_0, orc.Q8_0), "Q6_K": (mx.GgmlType.Q6_K, orc.Q6_K)}

MV_TOL = 1e-5   # mat-vec parity bound: max |y - y_ref| / sum |w*x|
MM_TOL = 2e-3   # f16 tensor-core mat-mat parity bound, same normalisation


def normal_weights(seed: int, n: int, k: int, otype: int, rule: str = "ggml") -> np.ndarray:
    """Seeded N(0, 0.02) weights quantized on the host (GGML rule for Q4_0/Q8_0, upstream test packer for Q6_K)."""
    rng = np.random.default_rng(seed)
    wf = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    return orc.quantize(otype, wf, rule=rule)


def normal_acts(seed: int, m: int, k: int) -> np.ndarray:
    return np.random.default_rng(seed + 7919).standard_normal((m, k)).astype(np.float32)


def lcg_weights(seed: int, n: int, k: int, otype: int) -> np.ndarray:
    return orc.quantize(otype, orc.lcg_f32(seed, n * k))


class Ctx:
    def __init__(self):
        self.device = mx.MlxDevice.new()
        self.registry = mx.KernelRegistry.new()

    def buf(self, data: np.ndarray, dtype: mx.DType) -> mx.MlxBuffer:
        a = np.ascontiguousarray(data)
        b = self.device.alloc_buffer(a.nbytes, dtype, list(a.shape))
        b.as_mut_slice(np.uint8)[:] = a.reshape(-1).view(np.uint8)
        return b

    def matmul(self, gtype, wq: np.ndarray, x: np.ndarray, n: int, k: int, force_mm: bool = False,
               weight_buf: mx.MlxBuffer | None = None) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
        m = x.shape[0]
        inp = self.buf(x, mx.DType.F32)
        w = weight_buf if weight_buf is not None else self.buf(wq, mx.DType.U8)
        out = self.device.alloc_buffer(m * n * 4, mx.DType.F32, [m, n])
        params = mx.GgmlQuantizedMatmulParams(m, n, k, gtype)
        enc = self.device.command_encoder()
        if force_mm:
            mx.dispatch_mm_for_test(enc, self.registry, self.device, inp, w, out, params)
        else:
            mx.quantized_matmul_ggml(enc, self.registry, self.device, inp, w, out, params)
        enc.commit_and_wait()
        return out.as_slice(np.float32).reshape(m, n).copy()

    def matmul_id(self, gtype, wq: np.ndarray, expert_stride: int, x: np.ndarray, ids: np.ndarray, top_k: int, n: int,
                  k: int, n_experts: int, mode: str = "auto", scratch=None):
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
        n_tokens = x.shape[0]
        inp = self.buf(x, mx.DType.F32)
        w = self.buf(wq, mx.DType.U8)
        idb = self.buf(np.ascontiguousarray(ids, dtype=np.uint32), mx.DType.U32)
        rows = n_tokens * top_k
        out = self.device.alloc_buffer(rows * n * 4, mx.DType.F32, [rows, n])
        enc = self.device.command_encoder()
        extra = None
        if mode == "auto":
            p = mx.GgmlQuantizedMatmulIdParams(n_tokens, top_k, n, k, n_experts, expert_stride, gtype)
            mx.quantized_matmul_id_ggml(enc, self.registry, self.device, inp, w, idb, out, p)
        elif mode == "pooled":
            p = mx.GgmlQuantizedMatmulIdParams(n_tokens, top_k, n, k, n_experts, expert_stride, gtype)
            scratch = scratch or mx.IdMmScratch.alloc(self.device, n_experts, n_tokens)
            mx.quantized_matmul_id_ggml_pooled(enc, self.registry, self.device, inp, w, idb, out, scratch, p)
            extra = scratch
        elif mode == "force_mm":
            p = mx.GgmlIdMmDispatchParams(n_tokens, top_k, n, k, n_experts, expert_stride, gtype)
            htpe = self.device.alloc_buffer(p.htpe_bytes(), mx.DType.U32, [n_experts])
            hids = self.device.alloc_buffer(p.hids_bytes(), mx.DType.U32, [n_experts, n_tokens])
            htpe.as_mut_slice(np.uint32)[:] = 0xDEADBEEF
            hids.as_mut_slice(np.uint32)[:] = 0xDEADBEEF
            mx.dispatch_id_mm_for_test(enc, self.registry, self.device, inp, w, idb, htpe, hids, out, p)
            extra = (htpe, hids)
        else:
            raise ValueError(mode)
        enc.commit_and_wait()
        return out.as_slice(np.float32).reshape(rows, n).copy(), extra


def norm_err(y: np.ndarray, y_ref: np.ndarray, absdot: np.ndarray) -> float:
    """max over outputs of |y - y_ref| / sum_k |w*x| (outputs whose normaliser is 0 must match exactly)."""
    d = np.abs(y.astype(np.float64) - y_ref.astype(np.float64))
    ok = absdot > 0
    assert np.all(d[~ok] == 0)
    return float(np.max(d[ok] / absdot[ok])) if ok.any() else 0.0
