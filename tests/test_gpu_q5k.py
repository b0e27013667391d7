"""Q5_K on the expert-routed mat-vec (the one Q5_K kernel upstream has, src/shaders/quantized_matmul_id_ggml.metal:401-509;
src/ops/quantized_matmul_id_ggml.rs:265-273 sends Q5_K to mv_id at every token count), against the oracle."""
import numpy as np
import pytest

import mlx_native_b200 as mx
from oracle import oracle as orc
from tests.gpu_util import MV_TOL, Ctx, norm_err
from tests.test_oracle_q5k import random_q5k_blocks

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


@pytest.mark.parametrize("T,top_k,E,n,k", [(1, 8, 16, 768, 2048), (5, 2, 4, 96, 512), (40, 8, 16, 64, 256), (3, 1, 2, 7, 768), (2, 8, 8, 2048, 1024),
                                           (1, 4, 4, 33, 256)])
def test_q5k_routed_matvec(ctx, T, top_k, E, n, k):
    rng = np.random.default_rng(T * 131 + n)
    w = random_q5k_blocks(rng, E * n * (k // 256))
    x = rng.standard_normal((T, k)).astype(np.float32)
    ids = np.stack([rng.permutation(E)[:top_k] for _ in range(T)]).astype(np.uint32).reshape(-1)
    y, _ = ctx.matmul_id(mx.GgmlType.Q5_K, w, w.size // E, x, ids, top_k, n, k, E)
    # (also for T > 32: Q5_K has no grouped mat-mat) up to 16 rows: problems of the register-level tensor-core kernel
    assert mx.last_kernel_name() == ("qmv_mma" if T * top_k <= 16 and k % 256 == 0 else "qmv_simple")
    y_ref, ad = orc.qmatmul_id(orc.Q5_K, w, w.size // E, x, ids, top_k, n, k, E, nthreads=8)
    assert norm_err(y, y_ref, ad) <= MV_TOL


def test_q5k_dense_is_refused_like_upstream(ctx):
    d = ctx.device
    enc = d.command_encoder()
    x = d.alloc_buffer(256 * 4, mx.DType.F32)
    w = d.alloc_buffer(176 * 4, mx.DType.U8)
    y = d.alloc_buffer(4 * 4, mx.DType.F32)
    with pytest.raises(mx.InvalidArgument, match="does not support Q5_K"):
        mx.quantized_matmul_ggml(enc, ctx.registry, d, x, w, y, mx.GgmlQuantizedMatmulParams(1, 4, 256, mx.GgmlType.Q5_K))
