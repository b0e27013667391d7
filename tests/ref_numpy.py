"""Second, independent restatement of the upstream dequantizers, in numpy.

It follows the upstream *production* CPU dequantizers (src/gguf/mod.rs:355-388 Q4_0,
:395-425 Q8_0, :656-709 Q6_K), whereas oracle/oracle.c follows the upstream *test-suite*
dequantizers.  The two must agree bit for bit; tests/test_oracle.py checks that.
"""
import numpy as np


def dequant_q4_0(data: np.ndarray) -> np.ndarray:
    blk = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1, 18)
    d = blk[:, 0:2].copy().view(np.float16).astype(np.float32)  # [nb,1]
    qs = blk[:, 2:18]
    x0 = (qs & 0x0F).astype(np.int16) - 8
    x1 = (qs >> 4).astype(np.int16) - 8
    out = np.concatenate([x0.astype(np.float32) * d, x1.astype(np.float32) * d], axis=1)
    return out.reshape(-1)


def dequant_q8_0(data: np.ndarray) -> np.ndarray:
    blk = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1, 34)
    d = blk[:, 0:2].copy().view(np.float16).astype(np.float32)
    qs = blk[:, 2:34].copy().view(np.int8).astype(np.float32)
    return (qs * d).reshape(-1)


def dequant_q6_k(data: np.ndarray) -> np.ndarray:
    blk = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1, 210)
    nb = blk.shape[0]
    ql = blk[:, 0:128]
    qh = blk[:, 128:192]
    sc = blk[:, 192:208].copy().view(np.int8).astype(np.float32)
    d = blk[:, 208:210].copy().view(np.float16).astype(np.float32)  # [nb,1]
    out = np.zeros((nb, 256), dtype=np.float32)
    for idx in range(2):
        l = ql[:, 64 * idx:64 * idx + 64]
        h = qh[:, 32 * idx:32 * idx + 32]
        s = sc[:, 8 * idx:8 * idx + 8]
        is_ = np.arange(32) // 16
        q1 = ((l[:, :32] & 0xF) | ((h & 3) << 4)).astype(np.int8) - np.int8(32)
        q2 = ((l[:, 32:] & 0xF) | (((h >> 2) & 3) << 4)).astype(np.int8) - np.int8(32)
        q3 = ((l[:, :32] >> 4) | (((h >> 4) & 3) << 4)).astype(np.int8) - np.int8(32)
        q4 = ((l[:, 32:] >> 4) | (((h >> 6) & 3) << 4)).astype(np.int8) - np.int8(32)
        base = 128 * idx
        out[:, base + 0:base + 32] = d * s[:, is_] * q1.astype(np.float32)
        out[:, base + 32:base + 64] = d * s[:, is_ + 2] * q2.astype(np.float32)
        out[:, base + 64:base + 96] = d * s[:, is_ + 4] * q3.astype(np.float32)
        out[:, base + 96:base + 128] = d * s[:, is_ + 6] * q4.astype(np.float32)
    return out.reshape(-1)


DEQUANT = {2: dequant_q4_0, 3: dequant_q8_0, 6: dequant_q6_k}


def lcg_f32(seed: int, n: int) -> np.ndarray:
    """tests/test_quantized_matmul_ggml.rs:17-28 with Python integers."""
    out = np.empty(n, dtype=np.float32)
    state = seed
    umax = np.float32(4294967295)
    for i in range(n):
        state = (state * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = np.float32(state >> 33) / umax - np.float32(0.5)
    return out


def bucket_scan_order(ids, n_tokens, top_k, n_experts):
    """tests/test_quantized_matmul_id_mm.rs:362-371: per-expert lists in (token, slot) scan order."""
    counts = [0] * n_experts
    lists = [[] for _ in range(n_experts)]
    for t in range(n_tokens):
        for s in range(top_k):
            e = int(ids[t * top_k + s])
            counts[e] += 1
            lists[e].append(t * top_k + s)
    return counts, lists
