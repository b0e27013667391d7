"""Small fixed workloads for profiler captures (a few hundred MB on the device, a handful of launches).

  python -m mlx_native_b200.profile_case mv  [Q8_0|Q6_K|Q4_0] [m]   decode mat-vec, n=12288 k=4096, 4 weight copies (> L2)
  python -m mlx_native_b200.profile_case mm  [Q4_0|Q6_K|Q8_0] [m]   prefill mat-mat, n=4096 k=4096, m=512 by default
  python -m mlx_native_b200.profile_case moe [m]                    expert-routed gate projection, 128 experts, top-8
  python -m mlx_native_b200.profile_case moe_layer [m] [reps]         whole MoE FFN layer (route, gate, up, SwiGLU, down, reduce),
                                                                     128 experts, top-8, hidden 2048, ffn 768
  python -m mlx_native_b200.profile_case cmp [types]                 tensor-core vs streaming mat-vec, microseconds per call
                                                                     (CUDA-graph replay over rotating weight copies > L2)

Weights are random bytes with finite f16 scales: the kernels' timing and memory traffic do not depend on the values.
"""
from __future__ import annotations

import sys

import numpy as np

import mlx_native_b200 as mx

BLOCK = {"Q4_0": (mx.GgmlType.Q4_0, 32, 18, 0), "Q8_0": (mx.GgmlType.Q8_0, 32, 34, 0), "Q6_K": (mx.GgmlType.Q6_K, 256, 210, 208)}


def random_blocks(rng, t: str, n: int, k: int) -> np.ndarray:
    _, qk, bb, dpos = BLOCK[t]
    raw = rng.integers(0, 256, size=(n * (k // qk), bb), dtype=np.uint8)
    raw[:, dpos + 1] = (raw[:, dpos + 1] & 0x83) | 0x20   # f16 scale exponent in a small finite range
    return raw.reshape(-1)


def compare_matvec_kernels(dev, reg, rng, types):
    """Event-timed microseconds per mat-vec for both kernels, every decode shape and m in {1, 2, 4, 8}; each call
    of a replayed graph has its own weight copy (more than L2 in total) and its own output buffer."""
    shapes = [(4096, 4096), (1024, 4096), (12288, 4096), (4096, 12288)]

    def timed(t, n, k, m, variant, reps=10):
        _, qk, bb, _ = BLOCK[t]
        wbytes = n * (k // qk) * bb
        ncopies = int(max(4, min(48, (300e6 // wbytes) + 1)))
        w = random_blocks(rng, t, n, k)
        ws = []
        for _ in range(ncopies):
            b = dev.alloc_buffer(wbytes, mx.DType.U8)
            b.upload(w)
            ws.append(b)
        x = rng.standard_normal((m, k)).astype(np.float32)
        xb = dev.alloc_buffer(x.nbytes, mx.DType.F32)
        xb.upload(x)
        ys = [dev.alloc_buffer(m * n * 4, mx.DType.F32) for _ in range(ncopies)]
        p = mx.GgmlQuantizedMatmulParams(m, n, k, BLOCK[t][0])
        mx.set_option("qmv", variant)
        enc = dev.command_encoder()
        for wb, yb in zip(ws[:2], ys[:2]):
            mx.quantized_matmul_ggml(enc, reg, dev, xb, wb, yb, p)
        enc.commit_and_wait()
        enc.begin_capture()
        for wb, yb in zip(ws, ys):
            mx.quantized_matmul_ggml(enc, reg, dev, xb, wb, yb, p)
        g = enc.end_capture()
        for _ in range(2):
            g.launch(enc)
        enc.commit_and_wait()
        for _ in range(reps):
            g.launch(enc)
        return enc.commit_wait_with_gpu_time() / (reps * ncopies) * 1e6

    for t in types:
        for (n, k) in shapes:
            cells = []
            for m in (1, 2, 4, 8):
                cells.append(f"m={m}: tc {timed(t, n, k, m, 'tc'):6.2f} st {timed(t, n, k, m, 'stream'):6.2f}")
            print(f"{t} {n:6d}x{k:<6d} " + " | ".join(cells), flush=True)
    mx.set_option("qmv", "auto")


def main(argv):
    mode = argv[0] if argv else "mv"
    dev = mx.MlxDevice.new(0)
    reg = mx.KernelRegistry.new()
    rng = np.random.default_rng(0)
    if mode == "cmp":
        compare_matvec_kernels(dev, reg, rng, (argv[1] if len(argv) > 1 else "Q8_0,Q6_K,Q4_0").split(","))
        return
    enc = dev.command_encoder()
    if mode == "moe_layer":
        T = int(argv[1]) if len(argv) > 1 else 512
        reps = int(argv[2]) if len(argv) > 2 else 3
        E, top_k, hidden, ffn = 128, 8, 2048, 768
        bufs = {}
        for name, t, rows, cols in (("gate", "Q4_0", E * ffn, hidden), ("up", "Q4_0", E * ffn, hidden), ("down", "Q6_K", E * hidden, ffn)):
            w = random_blocks(rng, t, rows, cols)
            bufs[name] = dev.alloc_buffer(w.size, mx.DType.U8)
            bufs[name].upload(w)
            bufs[name + "_stride"] = w.size // E
        logits = rng.standard_normal((T, E)).astype(np.float32)
        lg = dev.alloc_buffer(logits.nbytes, mx.DType.F32)
        lg.upload(logits)
        x = rng.standard_normal((T, hidden)).astype(np.float32)
        xb = dev.alloc_buffer(x.nbytes, mx.DType.F32)
        xb.upload(x)
        ids = dev.alloc_buffer(T * top_k * 4, mx.DType.U32)
        rw = dev.alloc_buffer(T * top_k * 4, mx.DType.F32)
        yg = dev.alloc_buffer(T * top_k * ffn * 4, mx.DType.F32)
        yu = dev.alloc_buffer(T * top_k * ffn * 4, mx.DType.F32)
        act = dev.alloc_buffer(T * top_k * ffn * 4, mx.DType.F32)
        yd = dev.alloc_buffer(T * top_k * hidden * 4, mx.DType.F32)
        outb = dev.alloc_buffer(T * hidden * 4, mx.DType.F32)
        pg = mx.GgmlQuantizedMatmulIdParams(T, top_k, ffn, hidden, E, bufs["gate_stride"], mx.GgmlType.Q4_0)
        pd = mx.GgmlQuantizedMatmulIdParams(T * top_k, 1, hidden, ffn, E, bufs["down_stride"], mx.GgmlType.Q6_K)
        for _ in range(reps):
            mx.moe_softmax_topk(enc, reg, dev, lg, ids, rw, T, E, top_k)
            mx.quantized_matmul_id_ggml(enc, reg, dev, xb, bufs["gate"], ids, yg, pg)
            mx.quantized_matmul_id_ggml(enc, reg, dev, xb, bufs["up"], ids, yu, pg)
            mx.silu_mul(enc, reg, dev, yg, yu, act, T * top_k * ffn)
            mx.quantized_matmul_id_ggml(enc, reg, dev, act, bufs["down"], ids, yd, pd)
            mx.moe_weighted_reduce(enc, reg, dev, rw, yd, outb, T, top_k, hidden)
            enc.commit_and_wait()
        print("ok", mx.last_kernel_name())
        return
    if mode == "moe":
        m = int(argv[1]) if len(argv) > 1 else 512
        E, top_k, hidden, ffn = 128, 8, 2048, 768
        w = random_blocks(rng, "Q4_0", E * ffn, hidden)
        wb = dev.alloc_buffer(w.size, mx.DType.U8)
        wb.upload(w)
        x = rng.standard_normal((m, hidden)).astype(np.float32)
        xb = dev.alloc_buffer(x.nbytes, mx.DType.F32)
        xb.upload(x)
        ids = np.stack([rng.permutation(E)[:top_k] for _ in range(m)]).astype(np.uint32)
        ib = dev.alloc_buffer(ids.nbytes, mx.DType.U32)
        ib.upload(ids)
        yb = dev.alloc_buffer(m * top_k * ffn * 4, mx.DType.F32)
        p = mx.GgmlQuantizedMatmulIdParams(m, top_k, ffn, hidden, E, w.size // E, mx.GgmlType.Q4_0)
        for _ in range(3):
            mx.quantized_matmul_id_ggml(enc, reg, dev, xb, wb, ib, yb, p)
        enc.commit_and_wait()
        print("ok", mx.last_kernel_name())
        return
    t = argv[1] if len(argv) > 1 else ("Q8_0" if mode == "mv" else "Q4_0")
    if mode == "mv":
        n, k, m, copies = 12288, 4096, int(argv[2]) if len(argv) > 2 else 1, 4
    else:
        n, k, m, copies = 4096, 4096, int(argv[2]) if len(argv) > 2 else 512, 1
    w = random_blocks(rng, t, n, k)
    ws = []
    for _ in range(copies):
        b = dev.alloc_buffer(w.size, mx.DType.U8)
        b.upload(w)
        ws.append(b)
    x = rng.standard_normal((m, k)).astype(np.float32)
    xb = dev.alloc_buffer(x.nbytes, mx.DType.F32)
    xb.upload(x)
    yb = dev.alloc_buffer(m * n * 4, mx.DType.F32)
    p = mx.GgmlQuantizedMatmulParams(m, n, k, BLOCK[t][0])
    for _ in range(2):
        for wbuf in ws:
            mx.quantized_matmul_ggml(enc, reg, dev, xb, wbuf, yb, p)
    enc.commit_and_wait()
    print("ok", mx.last_kernel_name())


if __name__ == "__main__":
    main(sys.argv[1:])
