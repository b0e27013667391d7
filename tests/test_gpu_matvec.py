"""Parity of the mat-vec path (m <= 8) with the CPU oracle, through the C ABI.
Mirrors upstream tests/test_quantized_matmul_ggml.rs and adds the shapes and edge cases of the B200 kernels."""
import numpy as np
import pytest

import mlx_native_b200 as mx
from oracle import oracle as orc
from tests.gpu_util import MV_TOL, TYPES, Ctx, lcg_weights, norm_err, normal_acts, normal_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


@pytest.fixture(params=["mma", "tc", "stream", "simple"])
def variant(request):
    # shapes the tensor-core kernels ("mma", "tc") do not take fall through to "stream"
    mx.set_option("qmv", request.param)
    yield request.param
    mx.set_option("qmv", "auto")


KERNEL_OF = {"mma": "qmv_mma", "tc": "qmv_tc", "stream": "qmv_stream", "simple": "qmv_simple"}


def check(ctx, tname, wq, x, n, k, abs_tol=None, tol=MV_TOL):
    gtype, otype = TYPES[tname]
    y = ctx.matmul(gtype, wq, x, n, k)
    y_ref, ad = orc.qmatmul(otype, wq, x, n, k, nthreads=8)
    err = norm_err(y, y_ref, ad)
    assert err <= tol, f"{tname} n={n} k={k} m={x.shape[0]}: normalised error {err:.3e} > {tol}"
    if abs_tol is not None:
        assert np.max(np.abs(y - y_ref)) <= abs_tol
    return y


# ---- upstream known-value ramps (tests/test_quantized_matmul_ggml.rs:539-577, :651-686, :759-789)
@pytest.mark.parametrize("tname", ["Q4_0", "Q8_0", "Q6_K"])
def test_known_values(ctx, variant, tname):
    if tname == "Q4_0":
        n, k, tol = 8, 32, 1e-4
        wf = np.array([[(r * 0.1) * ((c - 16.0) / 16.0) for c in range(k)] for r in range(n)], np.float32)
    elif tname == "Q8_0":
        n, k, tol = 8, 32, 1e-4
        wf = np.array([[(r + 1.0) * (c - 16.0) / 32.0 for c in range(k)] for r in range(n)], np.float32)
    else:
        n, k, tol = 2, 256, 1e-3
        wf = np.array([[(r + 1.0) * (c - 128.0) / 256.0 for c in range(k)] for r in range(n)], np.float32)
    wq = orc.quantize(TYPES[tname][1], wf)
    check(ctx, tname, wq, np.ones((1, k), np.float32), n, k, abs_tol=tol)


# ---- upstream seeded random cases (:585-586, :694-695, :797-798)
@pytest.mark.parametrize("tname,sw,sx,n,k,tol", [("Q4_0", 42, 123, 32, 256, 1e-3), ("Q8_0", 55, 66, 32, 256, 1e-3),
                                                 ("Q6_K", 99, 100, 16, 256, 1e-2)])
def test_random(ctx, variant, tname, sw, sx, n, k, tol):
    wq = lcg_weights(sw, n, k, TYPES[tname][1])
    check(ctx, tname, wq, orc.lcg_f32(sx, k)[None], n, k, abs_tol=tol)


# ---- upstream production shape 4096 x 4096, m = 1 (:619-620, :727-728, :824-825)
@pytest.mark.parametrize("tname,sw,sx,tol", [("Q4_0", 1, 2, 0.5), ("Q8_0", 77, 88, 0.1), ("Q6_K", 200, 201, 1.0)])
def test_production_shape(ctx, variant, tname, sw, sx, tol):
    n = k = 4096
    wq = lcg_weights(sw, n, k, TYPES[tname][1])
    check(ctx, tname, wq, orc.lcg_f32(sx, k)[None], n, k, abs_tol=tol)
    assert mx.last_kernel_name() == KERNEL_OF[variant]


# ---- the benchmark's first configuration: Q4_0, m=1, 4096 x 4096, N(0,0.02) weights, GGML quantizer, seed 0
def test_config_q4_0_4096(ctx, variant):
    wq = normal_weights(0, 4096, 4096, orc.Q4_0)
    check(ctx, "Q4_0", wq, normal_acts(0, 1, 4096), 4096, 4096)


# ---- decode sweep shapes, every m in 1..8 on one shape and m in {1,2,4,8} on the others
@pytest.mark.parametrize("tname", ["Q4_0", "Q8_0", "Q6_K"])
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 6, 7, 8])
def test_all_m(ctx, variant, tname, m):
    n, k = 1024, 4096
    wq = normal_weights(3, n, k, TYPES[tname][1])
    check(ctx, tname, wq, normal_acts(m, m, k), n, k)


@pytest.mark.parametrize("tname", ["Q8_0", "Q6_K"])
@pytest.mark.parametrize("n,k", [(4096, 4096), (12288, 4096), (4096, 12288)])
@pytest.mark.parametrize("m", [1, 8])
@pytest.mark.parametrize("kernel", ["mma", "tc", "stream"])
def test_decode_sweep_shapes(ctx, tname, n, k, m, kernel):
    mx.set_option("qmv", kernel)
    wq = normal_weights(11, n, k, TYPES[tname][1])
    y = check(ctx, tname, wq, normal_acts(5, m, k), n, k)
    assert mx.last_kernel_name() == KERNEL_OF[kernel]
    # a row's result does not depend on how many rows share the weights (up to summation order)
    if m == 8:
        x3 = normal_acts(5, 8, k)[3:4]
        y1 = ctx.matmul(TYPES[tname][0], wq, x3, n, k)
        _, ad = orc.qmatmul(TYPES[tname][1], wq, x3, n, k, nthreads=8)
        assert norm_err(y1, y[3:4], ad) <= MV_TOL


# ---- edge cases: ragged n, short and odd k, k-slicing, misaligned weight views
@pytest.mark.parametrize("tname,n,k,m", [
    ("Q4_0", 5, 32, 1), ("Q4_0", 13, 96, 3), ("Q8_0", 1, 64, 8), ("Q8_0", 7, 256, 2), ("Q6_K", 3, 256, 1),
    ("Q6_K", 2049, 768, 1), ("Q6_K", 66, 5120, 2), ("Q4_0", 1027, 2048, 8), ("Q8_0", 130, 12288, 8),
    ("Q6_K", 37, 12288, 4), ("Q4_0", 4, 256, 1), ("Q8_0", 149, 512, 5),
])
def test_edge_shapes(ctx, variant, tname, n, k, m):
    wq = normal_weights(n * 31 + k, n, k, TYPES[tname][1])
    check(ctx, tname, wq, normal_acts(n, m, k), n, k)


@pytest.mark.parametrize("tname", ["Q4_0", "Q8_0", "Q6_K"])
@pytest.mark.parametrize("offset", [2, 6, 18])
def test_weight_view_offsets(ctx, variant, tname, offset):
    """Weights that start at a 2-byte-aligned (not 16-byte-aligned) address inside a larger buffer."""
    gtype, otype = TYPES[tname]
    n, k = 64, 1024
    wq = normal_weights(5, n, k, otype)
    big = np.zeros(wq.size + 64, np.uint8)
    big[offset:offset + wq.size] = wq
    base = ctx.buf(big, mx.DType.U8)
    view = base.slice_view(offset, wq.size)
    x = normal_acts(1, 2, k)
    y = ctx.matmul(gtype, wq, x, n, k, weight_buf=view)
    y_ref, ad = orc.qmatmul(otype, wq, x, n, k)
    assert norm_err(y, y_ref, ad) <= MV_TOL


def test_zero_weights_and_zero_scale(ctx, variant):
    n, k = 16, 512
    for tname in ("Q4_0", "Q8_0", "Q6_K"):
        gtype, otype = TYPES[tname]
        wq = orc.quantize(otype, np.zeros((n, k), np.float32))
        y = ctx.matmul(gtype, wq, normal_acts(0, 2, k), n, k)
        assert np.all(y == 0)


def test_kernels_agree_closely(ctx):
    """The four mat-vec kernels agree to within summation-order rounding."""
    n, k = 512, 4096
    for tname in ("Q4_0", "Q8_0", "Q6_K"):
        gtype, otype = TYPES[tname]
        wq = normal_weights(9, n, k, otype)
        x = normal_acts(9, 4, k)
        mx.set_option("qmv", "stream")
        a = ctx.matmul(gtype, wq, x, n, k)
        mx.set_option("qmv", "simple")
        b = ctx.matmul(gtype, wq, x, n, k)
        mx.set_option("qmv", "tc")
        c = ctx.matmul(gtype, wq, x, n, k)
        assert mx.last_kernel_name() == "qmv_tc"
        mx.set_option("qmv", "mma")
        e = ctx.matmul(gtype, wq, x, n, k)
        assert mx.last_kernel_name() == "qmv_mma"
        _, ad = orc.qmatmul(otype, wq, x, n, k, nthreads=8)
        mx.set_option("qmv", "auto")
        assert norm_err(a, b, ad) <= MV_TOL
        assert norm_err(a, c, ad) <= MV_TOL
        assert norm_err(a, e, ad) <= MV_TOL


# ---- error behaviour (src/ops/quantized_matmul_ggml.rs:283-334)
def test_errors(ctx):
    d = ctx.device
    enc = d.command_encoder()
    x = d.alloc_buffer(4 * 64, mx.DType.F32, [1, 64])
    w = d.alloc_buffer(18 * 2 * 8, mx.DType.U8)
    y = d.alloc_buffer(4 * 8, mx.DType.F32, [1, 8])
    P = mx.GgmlQuantizedMatmulParams
    with pytest.raises(mx.InvalidArgument, match="does not support F32"):
        mx.quantized_matmul_ggml(enc, ctx.registry, d, x, w, y, P(1, 8, 64, mx.GgmlType.F32))
    with pytest.raises(mx.InvalidArgument, match="M, K, and N must all be > 0"):
        mx.quantized_matmul_ggml(enc, ctx.registry, d, x, w, y, P(0, 8, 64, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match=r"K \(48\) must be divisible by block QK \(32\)"):
        mx.quantized_matmul_ggml(enc, ctx.registry, d, x, w, y, P(1, 8, 48, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match="Weight buffer too small: expected 576 bytes"):
        mx.quantized_matmul_ggml(enc, ctx.registry, d, x, w, y, P(1, 16, 64, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match="Input buffer too small"):
        mx.quantized_matmul_ggml(enc, ctx.registry, d, x, w, y, P(2, 8, 64, mx.GgmlType.Q4_0))
    small_y = d.alloc_buffer(4 * 4, mx.DType.F32)
    with pytest.raises(mx.InvalidArgument, match="Output buffer too small"):
        mx.quantized_matmul_ggml(enc, ctx.registry, d, x, w, small_y, P(1, 8, 64, mx.GgmlType.Q4_0))
    # over-sized buffers are accepted, as upstream
    mx.quantized_matmul_ggml(enc, ctx.registry, d, x, w, y, P(1, 4, 64, mx.GgmlType.Q4_0))
    enc.commit_and_wait()
    with pytest.raises(mx.InvalidArgument):
        d.alloc_buffer(0, mx.DType.F32)


# ---- Q6_K rows of 16 j + 8 bytes (k % 2048 == 1024, e.g. the 5120-wide lm_head): the tensor-core kernel reads pairs
# ---- of weight rows as one tensor-map row
@pytest.mark.parametrize("n,k,m", [(2, 1024, 1), (66, 5120, 2), (128, 1024, 8), (130, 3072, 3), (1000, 5120, 1), (4748, 5120, 4)])
def test_q6k_row_pairs(ctx, n, k, m):
    mx.set_option("qmv", "tc")
    try:
        wq = normal_weights(n + k, n, k, orc.Q6_K)
        check(ctx, "Q6_K", wq, normal_acts(m, m, k), n, k)
        assert mx.last_kernel_name() == "qmv_tc"
        # an odd row count cannot be paired: the streaming kernel takes it
        wq = normal_weights(7, 33, 1024, orc.Q6_K)
        check(ctx, "Q6_K", wq, normal_acts(m, m, 1024), 33, 1024)
        assert mx.last_kernel_name() != "qmv_tc"
    finally:
        mx.set_option("qmv", "auto")


@pytest.mark.parametrize("n,k,m", [(2, 1024, 1), (66, 5120, 2), (128, 1024, 8), (130, 3072, 3), (1000, 5120, 1), (4748, 5120, 4),
                                   (18992, 5120, 1)])
def test_q6k_row_pairs_register_kernel(ctx, n, k, m):
    """The same row geometry on the register-level kernel (its tensor map's rows are pairs of weight rows too)."""
    mx.set_option("qmv", "mma")
    try:
        wq = normal_weights(n + k, min(n, 1024), k, orc.Q6_K)
        if n > 1024:
            rb = orc.row_bytes(orc.Q6_K, k)
            wq = np.concatenate([np.roll(wq.reshape(1024, rb), 3 * i, axis=0) for i in range((n + 1023) // 1024)])[:n].reshape(-1)
        check(ctx, "Q6_K", wq, normal_acts(m, m, k), n, k)
        assert mx.last_kernel_name() == "qmv_mma"
    finally:
        mx.set_option("qmv", "auto")


# ---- the large-vocabulary lm_head at full size: Q6_K 151936 x 5120, m = 1 (638 MB of weights), a sample of rows
# ---- including the first and last tiles
@pytest.mark.parametrize("kernel", ["auto", "mma", "tc", "stream"])
def test_lm_head_q6k_full_size_sampled(ctx, kernel):
    mx.set_option("qmv", kernel)
    try:
        gtype, otype = TYPES["Q6_K"]
        n, k = 151936, 5120
        rb = orc.row_bytes(otype, k)
        base = normal_weights(51, 512, k, otype).reshape(512, rb)
        wq = np.concatenate([np.roll(base, 13 * i, axis=0) for i in range((n + 511) // 512)])[:n].reshape(-1)
        x = normal_acts(51, 1, k)
        y = ctx.matmul(gtype, wq, x, n, k)
        assert np.isfinite(y).all() and np.count_nonzero(y) > 0.99 * n
        rows = np.array(sorted({0, 1, 127, 128, n // 2, n - 129, n - 128, n - 2, n - 1} |
                               set(int(r) for r in np.random.default_rng(1).choice(n, size=55, replace=False))))
        wsub = np.concatenate([wq[r * rb:(r + 1) * rb] for r in rows])
        y_ref, ad = orc.qmatmul(otype, wsub, x, len(rows), k, nthreads=8)
        assert norm_err(y[:, rows], y_ref, ad) <= MV_TOL
    finally:
        mx.set_option("qmv", "auto")


# ---- several conflict-free mat-vecs in one encoder leave as one kernel (upstream: concurrent dispatch between
# ---- barriers, src/encoder.rs:837-853); see also test_chained_matvecs_in_one_launch below
@pytest.mark.parametrize("tname", ["Q4_0", "Q8_0", "Q6_K"])
def test_batched_launch_of_independent_matvecs(ctx, tname):
    gtype, otype = TYPES[tname]
    d = ctx.device
    k = 4096
    shapes = [(4096, 1), (1024, 1), (12288, 1), (512, 1), (4096, 2), (64, 1), (1030, 1), (2048, 1), (4096, 1), (256, 1)]
    ws, xs, wbs, xbs, ybs = [], [], [], [], []
    for i, (n, m) in enumerate(shapes):
        ws.append(normal_weights(60 + i, n, k, otype))
        xs.append(normal_acts(60 + i, m, k))
        wbs.append(ctx.buf(ws[-1], mx.DType.U8))
        xbs.append(ctx.buf(xs[-1], mx.DType.F32))
        ybs.append(d.alloc_buffer(m * n * 4, mx.DType.F32))
    mx.reset_counters()
    enc = d.command_encoder()
    for (n, m), wb, xb, yb in zip(shapes, wbs, xbs, ybs):
        mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, wb, yb, mx.GgmlQuantizedMatmulParams(m, n, k, gtype))
    assert mx.kernel_launch_count() <= 3          # nothing has been launched for the open batch yet
    enc.commit_and_wait()
    assert mx.dispatch_count() == len(shapes) and mx.kernel_launch_count() < len(shapes)
    for (n, m), w, x, yb in zip(shapes, ws, xs, ybs):
        y_ref, ad = orc.qmatmul(otype, w, x, n, k, nthreads=8)
        assert norm_err(yb.as_slice(np.float32).reshape(m, n), y_ref, ad) <= MV_TOL, (tname, n, m)
    # a dependent pair: the second reads the first one's result
    n1, n2 = 4096, 512
    w1, w2 = normal_weights(81, n1, k, otype), normal_weights(82, n2, n1, otype)
    x = normal_acts(81, 1, k)
    y1, y2 = d.alloc_buffer(n1 * 4, mx.DType.F32), d.alloc_buffer(n2 * 4, mx.DType.F32)
    enc = d.command_encoder()
    mx.quantized_matmul_ggml(enc, ctx.registry, d, ctx.buf(x, mx.DType.F32), ctx.buf(w1, mx.DType.U8), y1,
                             mx.GgmlQuantizedMatmulParams(1, n1, k, gtype))
    mx.quantized_matmul_ggml(enc, ctx.registry, d, y1, ctx.buf(w2, mx.DType.U8), y2, mx.GgmlQuantizedMatmulParams(1, n2, n1, gtype))
    enc.commit_and_wait()
    r1, ad1 = orc.qmatmul(otype, w1, x, n1, k, nthreads=8)
    got1 = y1.as_slice(np.float32).reshape(1, n1)
    assert norm_err(got1, r1, ad1) <= MV_TOL
    r2, ad2 = orc.qmatmul(otype, w2, got1.copy(), n2, n1, nthreads=8)
    assert norm_err(y2.as_slice(np.float32).reshape(1, n2), r2, ad2) <= MV_TOL


# ---- option qmv_chain=1: mat-vecs that depend on one another (each reads the result of the one before, or writes over
# ---- it) also leave as ONE kernel: its blocks meet at a barrier between them while the next one's weights keep streaming
@pytest.mark.parametrize("tname", ["Q4_0", "Q8_0", "Q6_K"])
@pytest.mark.parametrize("m", [1, 2, 4])
def test_chained_matvecs_in_one_launch(ctx, tname, m):
    gtype, otype = TYPES[tname]
    d = ctx.device
    # x0 [m, 2048] -> 4096 -> 2048 -> 6144 -> 2048 -> 4096 (every K a multiple of 2048: Q6_K rows on 16-byte boundaries)
    dims = [2048, 4096, 2048, 6144, 2048, 4096]
    ws = [normal_weights(300 + i, dims[i + 1], dims[i], otype) for i in range(len(dims) - 1)]
    wbs = [ctx.buf(w, mx.DType.U8) for w in ws]
    x0 = normal_acts(300, m, dims[0])
    results = {}
    for chain in ("1", "0"):
        mx.set_option("qmv_chain", chain)
        mx.set_option("qmv", "mma")            # the same kernel and tiling with and without chaining
        mx.set_option("qmv_mma_tpw", "1")
        try:
            bufs = [ctx.buf(x0, mx.DType.F32)] + [d.alloc_buffer(m * n * 4, mx.DType.F32) for n in dims[1:]]
            side = d.alloc_buffer(m * dims[3] * 4, mx.DType.F32)
            mx.reset_counters()
            enc = d.command_encoder()
            for i in range(len(ws)):
                mx.quantized_matmul_ggml(enc, ctx.registry, d, bufs[i], wbs[i], bufs[i + 1],
                                         mx.GgmlQuantizedMatmulParams(m, dims[i + 1], dims[i], gtype))
            # ... and one that overwrites the last result's neighbour twice (write after write)
            for i in (1, 1):
                mx.quantized_matmul_ggml(enc, ctx.registry, d, bufs[2], wbs[2], side, mx.GgmlQuantizedMatmulParams(m, dims[3], dims[2], gtype))
            enc.commit_and_wait()
            launches = mx.kernel_launch_count()
            results[chain] = ([b.as_slice(np.float32).copy() for b in bufs[1:]], side.as_slice(np.float32).copy(), launches)
        finally:
            mx.set_option("qmv_chain", "0")
            mx.set_option("qmv", "auto")
            mx.set_option("qmv_mma_tpw", "0")
    got, side1, launches1 = results["1"]
    ref, side0, launches0 = results["0"]
    assert launches1 == 1 and launches0 >= len(ws)    # (unchained, only conflict-free neighbours share a launch)
    x = x0
    for i, w in enumerate(ws):
        y_ref, ad = orc.qmatmul(otype, w, x, dims[i + 1], dims[i], nthreads=8)
        y = got[i].reshape(m, dims[i + 1])
        assert norm_err(y, y_ref, ad) <= MV_TOL, (tname, m, i)
        assert np.array_equal(got[i], ref[i])          # the same kernel either way: bit-identical to separate launches
        x = y.copy()
    assert np.array_equal(side1, side0) and np.array_equal(side1.reshape(m, dims[3]), got[2].reshape(m, dims[3]))
