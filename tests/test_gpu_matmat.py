"""Parity of the mat-mat path (m > 8; tcgen05 and CUDA-core kernels) with the CPU oracle.
Mirrors upstream tests/test_quantized_matmul_mm.rs (mm vs the scalar path, partial tiles, m = threshold + 1)."""
import numpy as np
import pytest

import mlx_native_b200 as mx
from oracle import oracle as orc
from tests.gpu_util import MM_TOL, TYPES, Ctx, lcg_weights, norm_err, normal_acts, normal_weights

pytestmark = pytest.mark.gpu

# the kernel's operands are the oracle's f16-rounded operands; only f32 summation order differs
F16_ORACLE_TOL = 2e-5


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


@pytest.fixture(params=["tc", "simt"])
def variant(request):
    mx.set_option("qmm", request.param)
    yield request.param
    mx.set_option("qmm", "tc")


def check(ctx, tname, wq, x, n, k, force=False, abs_tol=None):
    gtype, otype = TYPES[tname]
    y = ctx.matmul(gtype, wq, x, n, k, force_mm=force)
    y_ref, ad = orc.qmatmul(otype, wq, x, n, k, nthreads=8)
    err = norm_err(y, y_ref, ad)
    assert err <= MM_TOL, f"{tname} m={x.shape[0]} n={n} k={k}: normalised error {err:.3e} vs f32 oracle"
    if mx.last_kernel_name().startswith("qmm"):
        y16, _ = orc.qmatmul(otype, wq, x, n, k, f16_operands=True, nthreads=8)
        err16 = norm_err(y, y16, ad)
        assert err16 <= F16_ORACLE_TOL, f"{tname} m={x.shape[0]} n={n} k={k}: {err16:.3e} vs f16-operand oracle"
    if abs_tol is not None:
        assert np.max(np.abs(y - y_ref)) <= abs_tol
    return y


# upstream shapes and seeds (tests/test_quantized_matmul_mm.rs:372-547)
UPSTREAM = [
    ("Q4_0", 16, 64, 128, 0xA1B2, 0x1234, 5e-3), ("Q4_0", 64, 256, 2048, 0xC0FFEE, 0xDEADBEEF, 5e-2),
    ("Q4_0", 40, 96, 256, 0x13, 0x42, 1e-2), ("Q8_0", 16, 64, 128, 0xA1B3, 0x1235, 2e-3),
    ("Q8_0", 17, 72, 256, 0x14, 0x43, 5e-3), ("Q6_K", 16, 64, 256, 0xA1B4, 0x1236, 5e-3),
    ("Q6_K", 33, 100, 512, 0x15, 0x44, 1e-2),
]


@pytest.mark.parametrize("tname,m,n,k,sw,sx,tol", UPSTREAM)
def test_upstream_shapes(ctx, variant, tname, m, n, k, sw, sx, tol):
    wq = lcg_weights(sw, n, k, TYPES[tname][1])
    x = orc.lcg_f32(sx, m * k).reshape(m, k)
    check(ctx, tname, wq, x, n, k, force=True, abs_tol=tol * 4)
    assert mx.last_kernel_name() == ("qmm_tc" if variant == "tc" else "qmm_simt")


@pytest.mark.parametrize("tname", ["Q4_0", "Q8_0", "Q6_K"])
def test_threshold_plus_one_routes_to_mm(ctx, variant, tname):
    """m = MM_ROUTING_THRESHOLD + 1 takes the mat-mat route through the public entry point (:587-602)."""
    n, k, m = 128, 512, mx.MM_ROUTING_THRESHOLD + 1
    wq = normal_weights(1, n, k, TYPES[tname][1])
    check(ctx, tname, wq, normal_acts(1, m, k), n, k)
    assert mx.last_kernel_name().startswith("qmm")
    check(ctx, tname, wq, normal_acts(1, 8, k), n, k)
    assert mx.last_kernel_name().startswith("qmv")


@pytest.mark.parametrize("tname", ["Q4_0", "Q8_0", "Q6_K"])
@pytest.mark.parametrize("m,n,k", [(1, 8, 256), (3, 130, 256), (129, 257, 768), (64, 128, 4096), (300, 384, 1024),
                                   (512, 256, 2048), (65, 1000, 512)])
def test_tile_edges(ctx, variant, tname, m, n, k):
    wq = normal_weights(m + n, n, k, TYPES[tname][1])
    check(ctx, tname, wq, normal_acts(m, m, k), n, k, force=True)


@pytest.mark.parametrize("tname,k", [("Q4_0", 32), ("Q4_0", 96), ("Q8_0", 160), ("Q8_0", 64)])
def test_short_and_odd_k(ctx, variant, tname, k):
    n, m = 70, 20
    wq = normal_weights(k, n, k, TYPES[tname][1])
    check(ctx, tname, wq, normal_acts(k, m, k), n, k, force=True)


def sampled_rows(n, count, rng_seed=0):
    """A sample of weight rows that always includes the first and last rows of the first, a middle and the last
    128-row tile (the tensor-core kernel's work items)."""
    fixed = {0, 127, 128, n // 2, n - 129 if n > 129 else 0, n - 128 if n > 128 else 0, n - 1}
    rest = np.random.default_rng(rng_seed).choice(n, size=max(0, count - len(fixed)), replace=False)
    return np.array(sorted(fixed | set(int(r) for r in rest)))


# every prefill cell of the benchmark: m in {512, 2048} x {(4096, 4096), (12288, 4096), (4096, 12288)} x {Q4_0, Q6_K}
@pytest.mark.parametrize("tname", ["Q4_0", "Q6_K"])
@pytest.mark.parametrize("m,n,k", [(2048, 4096, 4096), (512, 12288, 4096), (2048, 12288, 4096), (512, 4096, 12288),
                                   (2048, 4096, 12288)])
def test_benchmark_prefill_cells_sampled(ctx, tname, m, n, k):
    """The benchmark's own prefill shapes at full size (256-wide activation tiles, no K split, 1.7 waves of the
    persistent walk) against the oracle on a sample of weight rows x a sample of activation rows."""
    mx.set_option("qmm", "tc")
    gtype, otype = TYPES[tname]
    rb = orc.row_bytes(otype, k)
    base = normal_weights(31, 512, k, otype).reshape(512, rb)
    # distinct rows everywhere, quick to build: the 512 seeded rows rolled by a different amount per block of 512
    wq = np.concatenate([np.roll(base, 7 * i, axis=0) for i in range(n // 512)]).reshape(-1)
    x = normal_acts(31, m, k)
    y = ctx.matmul(gtype, wq, x, n, k)
    assert mx.last_kernel_name() == "qmm_tc"
    assert np.isfinite(y).all()
    rows = sampled_rows(n, 40)
    xr = np.array(sorted({0, 1, 63, 64, 127, 128, 255, 256, m // 2, m - 257, m - 256, m - 65, m - 1}))
    wsub = np.concatenate([wq[r * rb:(r + 1) * rb] for r in rows])
    y_ref, ad = orc.qmatmul(otype, wsub, x[xr], len(rows), k, nthreads=8)
    assert norm_err(y[np.ix_(xr, rows)], y_ref, ad) <= MM_TOL
    y16, _ = orc.qmatmul(otype, wsub, x[xr], len(rows), k, f16_operands=True, nthreads=8)
    assert norm_err(y[np.ix_(xr, rows)], y16, ad) <= F16_ORACLE_TOL


# the large-vocabulary lm_head: Q6_K, k = 5120 (210-byte blocks x 20: rows start on 16-byte boundaries only every
# other row, so the mat-mat fetches them with the generic 16-byte copies), m = 256
@pytest.mark.parametrize("n", [16384 + 64, 151936])
def test_lm_head_q6k_m256_sampled(ctx, n):
    mx.set_option("qmm", "tc")
    gtype, otype = TYPES["Q6_K"]
    k, m = 5120, 256
    rb = orc.row_bytes(otype, k)
    base = normal_weights(41, 512, k, otype).reshape(512, rb)
    reps = (n + 511) // 512
    wq = np.concatenate([np.roll(base, 11 * i, axis=0) for i in range(reps)])[:n].reshape(-1)
    x = normal_acts(41, m, k)
    y = ctx.matmul(gtype, wq, x, n, k)
    assert mx.last_kernel_name() == "qmm_tc"
    assert np.isfinite(y).all()
    rows = sampled_rows(n, 48)
    xr = np.array([0, 1, 63, 64, 127, 128, 200, 255])
    wsub = np.concatenate([wq[r * rb:(r + 1) * rb] for r in rows])
    y_ref, ad = orc.qmatmul(otype, wsub, x[xr], len(rows), k, nthreads=8)
    assert norm_err(y[np.ix_(xr, rows)], y_ref, ad) <= MM_TOL
    y16, _ = orc.qmatmul(otype, wsub, x[xr], len(rows), k, f16_operands=True, nthreads=8)
    assert norm_err(y[np.ix_(xr, rows)], y16, ad) <= F16_ORACLE_TOL


@pytest.mark.parametrize("tname", ["Q4_0", "Q6_K"])
@pytest.mark.parametrize("m,n,k", [(512, 4096, 4096), (512, 1024, 12288)])
def test_prefill_shapes_sampled(ctx, tname, m, n, k):
    """Prefill-sized problems on the tcgen05 kernel, checked on a sample of weight rows and on the
    linearity of the product (size-independent properties at full size)."""
    mx.set_option("qmm", "tc")
    gtype, otype = TYPES[tname]
    wq = normal_weights(21, n, k, otype)
    x = normal_acts(21, m, k)
    y = ctx.matmul(gtype, wq, x, n, k)
    assert mx.last_kernel_name() == "qmm_tc"
    rows = np.random.default_rng(0).choice(n, size=48, replace=False)
    rb = orc.row_bytes(otype, k)
    wsub = np.concatenate([wq[r * rb:(r + 1) * rb] for r in rows])
    y_ref, ad = orc.qmatmul(otype, wsub, x, len(rows), k, nthreads=8)
    assert norm_err(y[:, rows], y_ref, ad) <= MM_TOL
    y16, _ = orc.qmatmul(otype, wsub, x, len(rows), k, f16_operands=True, nthreads=8)
    assert norm_err(y[:, rows], y16, ad) <= F16_ORACLE_TOL
    # linearity: doubling x doubles y (up to the few f16-subnormal activations that gain a bit)
    y2 = ctx.matmul(gtype, wq, x * np.float32(2.0), n, k)
    assert norm_err(y2[:, rows] * np.float32(0.5), y[:, rows], ad) <= 1e-5


def test_mm_matches_mv_by_row(ctx, variant):
    """Upstream's own check: mat-mat output row i equals the mat-vec result for input row i (:321-366)."""
    m, n, k = 24, 96, 512
    for tname, tol in (("Q4_0", 1e-2), ("Q8_0", 5e-3), ("Q6_K", 1e-2)):
        gtype, otype = TYPES[tname]
        wq = lcg_weights(0x77, n, k, otype)
        x = orc.lcg_f32(0x99, m * k).reshape(m, k)
        ymm = ctx.matmul(gtype, wq, x, n, k, force_mm=True)
        for i in range(0, m, 5):
            ymv = ctx.matmul(gtype, wq, x[i:i + 1], n, k)
            assert np.max(np.abs(ymm[i] - ymv[0])) <= tol


def test_dispatch_mm_for_test_errors(ctx):
    d = ctx.device
    enc = d.command_encoder()
    x = d.alloc_buffer(4 * 64 * 16, mx.DType.F32)
    w = d.alloc_buffer(144 * 16, mx.DType.U8)
    y = d.alloc_buffer(4 * 16 * 16, mx.DType.F32)
    with pytest.raises(mx.InvalidArgument, match="dispatch_mm_for_test does not support Q4_K"):
        mx.dispatch_mm_for_test(enc, ctx.registry, d, x, w, y, mx.GgmlQuantizedMatmulParams(16, 16, 256, mx.GgmlType.Q4_K))
    with pytest.raises(mx.InvalidArgument, match="must be divisible"):
        mx.dispatch_mm_for_test(enc, ctx.registry, d, x, w, y, mx.GgmlQuantizedMatmulParams(16, 16, 40, mx.GgmlType.Q4_0))
