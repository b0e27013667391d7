"""The mat-mat entry point that allocates nothing, checked against the regular one through the C ABI.

Who needs it: code that holds device pointers but may not allocate device memory at call time — for example
a serving process whose own allocator has taken all of HBM, or a latency-critical loop that must never enter
the driver's allocation path.  The regular mat-mat keeps its packed f16 activations in a growable arena
(cudaMalloc on first use); this variant keeps them in a fixed 16 MiB array inside the library.

This file is collected last on purpose (run order is alphabetical), so a failure here cannot hide another test.
"""
import numpy as np
import pytest

import mlx_native_b200 as mx
from oracle import oracle as orc
from tests.gpu_util import MM_TOL, TYPES, Ctx, norm_err, normal_acts, normal_weights

pytestmark = pytest.mark.gpu


def run_both(ctx, tname, m, n, k, seed):
    gtype, otype = TYPES[tname]
    d = ctx.device
    wq = normal_weights(seed, n, k, otype)
    x = normal_acts(seed, m, k)
    p = mx.GgmlQuantizedMatmulParams(m, n, k, gtype)
    # regular entry point (arena-backed scratch)
    want = ctx.matmul(gtype, wq, x, n, k, force_mm=True)
    assert mx.last_kernel_name() == "qmm_tc"
    # allocation-free entry point on raw device pointers and the encoder's stream
    wb, xb = ctx.buf(wq, mx.DType.U8), ctx.buf(x, mx.DType.F32)
    yb = d.alloc_buffer(m * n * 4, mx.DType.F32)
    enc = d.command_encoder()
    # bind the buffers once through a regular call so that their host-written contents are uploaded
    mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, wb, yb, mx.GgmlQuantizedMatmulParams(1, n, k, gtype))
    enc.commit_and_wait()
    mx.quantized_matmul_ggml_mm_noalloc(enc.stream(), xb.contents_ptr(), wb.contents_ptr(), yb.contents_ptr(), p)
    enc.commit_and_wait()
    got = yb.download(np.float32).reshape(m, n)
    y_ref, ad = orc.qmatmul(otype, wq, x, n, k, nthreads=8)
    assert norm_err(got, y_ref, ad) <= MM_TOL            # parity with the oracle
    assert norm_err(got, want, ad) <= 2e-5               # same kernels, same tiles as the regular entry point
    return got, want


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    ctx = Ctx()
    assert mx.noalloc_scratch_limit() == 16 * 1024 * 1024
    # two calls in a row share the static array: a large one, then a smaller one of another type that must not
    # be disturbed by what the first left behind
    g1, w1 = run_both(ctx, "Q4_0", 300, 384, 1024, seed=1)
    g2, w2 = run_both(ctx, "Q6_K", 40, 130, 768, seed=2)
    assert np.array_equal(g1, w1) and np.array_equal(g2, w2)
    # and the first shape again gives the first result again
    g3, _ = run_both(ctx, "Q4_0", 300, 384, 1024, seed=1)
    assert np.array_equal(g3, g1)


def test_noalloc_rejects_what_does_not_fit():
    P = mx.GgmlQuantizedMatmulParams
    with pytest.raises(mx.InvalidArgument, match="static scratch holds 16777216"):
        mx.quantized_matmul_ggml_mm_noalloc(0, 256, 256, 256, P(4096, 128, 4096, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match="supports Q4_0, Q8_0 and Q6_K only"):
        mx.quantized_matmul_ggml_mm_noalloc(0, 256, 256, 256, P(16, 128, 256, mx.GgmlType.Q4_K))
    with pytest.raises(mx.InvalidArgument, match="must not be null"):
        mx.quantized_matmul_ggml_mm_noalloc(0, 0, 256, 256, P(16, 128, 256, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match="divisible"):
        mx.quantized_matmul_ggml_mm_noalloc(0, 256, 256, 256, P(16, 128, 48, mx.GgmlType.Q4_0))
