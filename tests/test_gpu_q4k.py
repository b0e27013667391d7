"""Q4_K on the same entry points: dense mat-vec (any m: upstream has no dense Q4_K mat-mat and routes every m to the
mat-vec, src/ops/quantized_matmul_ggml.rs:350-360), expert-routed mat-vec and bucketed mat-mat.  Shapes follow the
upstream cases (tests/test_q4_k_kernels.rs:447-470, 619-663); seeded weights go through the oracle's restatement of
the upstream test packer."""
import numpy as np
import pytest

import mlx_native_b200 as mx
from oracle import oracle as orc
from tests.gpu_util import MM_TOL, MV_TOL, Ctx, lcg_weights, norm_err, normal_acts, normal_weights

pytestmark = pytest.mark.gpu
G, O = mx.GgmlType.Q4_K, orc.Q4_K


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


@pytest.mark.parametrize("n,k,m", [(2, 256, 1), (8, 256, 1), (4, 512, 1), (64, 1024, 1), (256, 4096, 1), (96, 2048, 3),
                                   (130, 1024, 8), (40, 768, 20)])
def test_dense_matvec(ctx, n, k, m):
    wq = normal_weights(n + k, n, k, O)
    x = normal_acts(m, m, k)
    y = ctx.matmul(G, wq, x, n, k)
    assert mx.last_kernel_name() == "qmv_mma"            # the register-level tensor-core kernel (144-byte blocks: rows always 16-byte aligned)
    y_ref, ad = orc.qmatmul(O, wq, x, n, k, nthreads=4)
    assert norm_err(y, y_ref, ad) <= MV_TOL
    mx.set_option("qmv", "simple")
    try:
        y2 = ctx.matmul(G, wq, x, n, k)
        assert mx.last_kernel_name() == "qmv_simple" and norm_err(y2, y_ref, ad) <= MV_TOL
    finally:
        mx.set_option("qmv", "auto")


@pytest.mark.parametrize("n,k,m", [(4096, 4096, 1), (1024, 4096, 4), (12288, 4096, 2), (4096, 12288, 1), (2048, 5120, 8), (777, 2304, 3)])
def test_dense_matvec_model_shapes(ctx, n, k, m):
    wq = normal_weights(n + k + m, n, k, O)
    x = normal_acts(m + 50, m, k)
    y = ctx.matmul(G, wq, x, n, k)
    assert mx.last_kernel_name() == "qmv_mma"
    y_ref, ad = orc.qmatmul(O, wq, x, n, k, nthreads=8)
    assert norm_err(y, y_ref, ad) <= MV_TOL


def test_dense_matvec_upstream_lcg_inputs(ctx):
    n, k = 64, 1024
    wq = lcg_weights(42, n, k, O)
    x = orc.lcg_f32(7, k).reshape(1, k)
    y = ctx.matmul(G, wq, x, n, k)
    y_ref, ad = orc.qmatmul(O, wq, x, n, k)
    assert norm_err(y, y_ref, ad) <= MV_TOL


@pytest.mark.parametrize("T,E,top_k,n,k", [(1, 4, 1, 64, 256), (1, 8, 8, 32, 512), (4, 8, 2, 64, 512), (8, 16, 4, 48, 1024)])
def test_routed_matvec(ctx, T, E, top_k, n, k):
    wq = normal_weights(T + E, E * n, k, O)
    x = normal_acts(T, T, k)
    rng = np.random.default_rng(T * 31 + E)
    ids = np.stack([rng.permutation(E)[:top_k] for _ in range(T)]).astype(np.uint32).reshape(-1)
    y, _ = ctx.matmul_id(G, wq, wq.size // E, x, ids, top_k, n, k, E)
    y_ref, ad = orc.qmatmul_id(O, wq, wq.size // E, x, ids, top_k, n, k, E)
    assert norm_err(y, y_ref, ad) <= MV_TOL


@pytest.mark.parametrize("T,E,top_k,n,k", [(16, 8, 8, 64, 512), (64, 4, 1, 96, 1024), (40, 16, 8, 128, 2048), (200, 32, 8, 768, 2048),
                                           (70, 6, 3, 130, 768)])
def test_routed_bucketed_matmat(ctx, T, E, top_k, n, k):
    wq = normal_weights(T + 3 * E, E * n, k, O)
    x = normal_acts(T + 1, T, k)
    rng = np.random.default_rng(T * 17 + E)
    ids = np.stack([rng.permutation(E)[:top_k] for _ in range(T)]).astype(np.uint32).reshape(-1)
    y, (htpe, hids) = ctx.matmul_id(G, wq, wq.size // E, x, ids, top_k, n, k, E, mode="force_mm")
    assert mx.last_kernel_name() == "qmm_tc_id"          # the tensor-core grouped mat-mat (weights dequantized into tensor memory)
    mx.set_option("qmm", "simt")
    try:
        y_simt, _ = ctx.matmul_id(G, wq, wq.size // E, x, ids, top_k, n, k, E, mode="force_mm")
        assert mx.last_kernel_name() == "qmm_simt_id"
    finally:
        mx.set_option("qmm", "tc")
    # bucketing: bit-exact against the oracle
    o_htpe, o_hids = orc.moe_map0(ids, T, top_k, E)
    assert np.array_equal(htpe.as_slice(np.uint32), o_htpe)
    y_ref, ad = orc.qmatmul_id(O, wq, wq.size // E, x, ids, top_k, n, k, E, f16_operands=True)
    assert norm_err(y, y_ref, ad) <= MM_TOL and norm_err(y_simt, y_ref, ad) <= MM_TOL
    y_f32, ad32 = orc.qmatmul_id(O, wq, wq.size // E, x, ids, top_k, n, k, E)
    assert norm_err(y, y_f32, ad32) <= MM_TOL


def test_dense_forced_matmat_is_refused(ctx):
    d = ctx.device
    wq = normal_weights(1, 16, 256, O)
    w, x = ctx.buf(wq, mx.DType.U8), ctx.buf(normal_acts(2, 16, 256), mx.DType.F32)
    out = d.alloc_buffer(16 * 16 * 4, mx.DType.F32)
    enc = d.command_encoder()
    with pytest.raises(mx.InvalidArgument):
        mx.dispatch_mm_for_test(enc, ctx.registry, d, x, w, out, mx.GgmlQuantizedMatmulParams(16, 16, 256, G))
