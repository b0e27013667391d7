"""Writes tests/golden/matmul_vectors.npz: frozen inputs and outputs of the CPU oracle for small seeded problems.

    python tests/golden/make_golden.py

The upstream project ships no golden files for this path and cannot be run where this repository is built, so these
vectors are produced by the oracle itself (oracle/oracle.c, which restates the upstream scalar test path).  They do not
pin the oracle to upstream; they freeze its answers, so that a later change to the oracle or to the packers shows up
as a test failure, and they give the GPU tests inputs and expected outputs that do not depend on any host code at all.
Cases follow the upstream seeded tests (tests/test_quantized_matmul_ggml.rs:585-586, :694-695, :797-798: LCG seeds
42/123, 55/66, 99/100) plus one N(0, 0.02) case per type with four activation rows.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402

CASES = [("Q4_0", orc.Q4_0, 42, 123, 32, 256), ("Q8_0", orc.Q8_0, 55, 66, 32, 256), ("Q6_K", orc.Q6_K, 99, 100, 16, 256)]


def main():
    out = {}
    for name, ot, sw, sx, n, k in CASES:
        wq = orc.quantize(ot, orc.lcg_f32(sw, n * k))
        x = orc.lcg_f32(sx, k)[None]
        y, ad = orc.qmatmul(ot, wq, x, n, k)
        out[f"{name}_lcg_w"], out[f"{name}_lcg_x"], out[f"{name}_lcg_y"], out[f"{name}_lcg_absdot"] = wq, x, y, ad
        rng = np.random.default_rng(7)
        n2, k2, m2 = 48, 512, 4
        wq2 = orc.quantize(ot, (rng.standard_normal((n2, k2)) * 0.02).astype(np.float32), rule="ggml")
        x2 = rng.standard_normal((m2, k2)).astype(np.float32)
        y2, ad2 = orc.qmatmul(ot, wq2, x2, n2, k2)
        out[f"{name}_normal_w"], out[f"{name}_normal_x"], out[f"{name}_normal_y"], out[f"{name}_normal_absdot"] = wq2, x2, y2, ad2
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "matmul_vectors.npz"), **out)


if __name__ == "__main__":
    main()
