"""Row-sharded mat-vec (tensor parallelism along N) on one GPU: the ranks' kernels run one after the other and
store into a shared full-width result buffer and into a second buffer that stands in for a peer's memory; the
assembled result must equal the unsharded mat-vec.  (The multi-GPU path of bench.py uses the same entry point
with real peer addresses.)"""
import numpy as np
import pytest

import mlx_native_b200 as mx
from mlx_native_b200 import sharding
from oracle import oracle as orc
from tests.gpu_util import MV_TOL, TYPES, Ctx, norm_err, normal_acts, normal_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


@pytest.mark.parametrize("qmv", ["auto", "mma", "tc", "stream", "simple"])
@pytest.mark.parametrize("tname,n,k,m,world", [("Q8_0", 1024, 4096, 1, 2), ("Q8_0", 1024, 4096, 8, 4), ("Q6_K", 2048, 2048, 4, 2),
                                               ("Q4_0", 768, 1024, 3, 3), ("Q6_K", 512, 768, 2, 2), ("Q8_0", 1536, 12288, 2, 2)])
def test_sharded_equals_unsharded(ctx, qmv, tname, n, k, m, world):
    mx.set_option("qmv", qmv)
    try:
        d = ctx.device
        gtype, otype = TYPES[tname]
        wq = normal_weights(31, n, k, otype)
        x = normal_acts(31, m, k)
        xb = ctx.buf(x, mx.DType.F32)
        full = d.alloc_buffer(m * n * 4, mx.DType.F32)       # this "rank"'s result buffer
        peer = d.alloc_buffer(m * n * 4, mx.DType.F32)       # stands in for another rank's buffer
        full.upload(np.full(m * n, np.nan, np.float32))
        peer.upload(np.full(m * n, np.nan, np.float32))
        enc = d.command_encoder()
        n_loc = n // world
        for rank in range(world):
            w_loc = sharding.shard_weight_bytes(wq, int(gtype), n, k, rank, world)
            wb = ctx.buf(w_loc, mx.DType.U8)
            p = mx.GgmlQuantizedMatmulParams(m, n_loc, k, gtype)
            mx.quantized_matmul_ggml_sharded(enc, ctx.registry, d, xb, wb, full, p, n, rank * n_loc, [peer.contents_ptr()])
        enc.commit_and_wait()
        y_ref, ad = orc.qmatmul(otype, wq, x, n, k, nthreads=8)
        got = full.as_slice(np.float32).reshape(m, n)
        assert norm_err(got, y_ref, ad) <= MV_TOL
        # the peer copy is written by the same kernels; download it through a fresh host view
        got_peer = peer.download(np.float32).reshape(m, n)
        assert norm_err(got_peer, y_ref, ad) <= MV_TOL
        if mx.last_kernel_name() != "qmv_tc":     # every kernel but the one that adds split tiles up with atomics
            assert np.array_equal(got_peer.view(np.uint32), got.view(np.uint32))
    finally:
        mx.set_option("qmv", "auto")


@pytest.mark.parametrize("tname,n,k,m,world", [("Q6_K", 2048, 5120, 256, 2), ("Q4_0", 1536, 1024, 64, 4), ("Q8_0", 1024, 2048, 33, 2)])
def test_sharded_mat_mat_equals_oracle(ctx, tname, n, k, m, world):
    """The tensor-core mat-mat in the row-sharded form (prefill / lm_head with many rows): every rank's tiles land in
    the full-width result and in the buffer that stands in for a peer."""
    from tests.gpu_util import MM_TOL

    d = ctx.device
    gtype, otype = TYPES[tname]
    wq = normal_weights(33, n, k, otype)
    x = normal_acts(33, m, k)
    xb = ctx.buf(x, mx.DType.F32)
    full = d.alloc_buffer(m * n * 4, mx.DType.F32)
    peer = d.alloc_buffer(m * n * 4, mx.DType.F32)
    full.upload(np.full(m * n, np.nan, np.float32))
    peer.upload(np.full(m * n, np.nan, np.float32))
    enc = d.command_encoder()
    n_loc = n // world
    for rank in range(world):
        wb = ctx.buf(sharding.shard_weight_bytes(wq, int(gtype), n, k, rank, world), mx.DType.U8)
        mx.quantized_matmul_ggml_sharded(enc, ctx.registry, d, xb, wb, full, mx.GgmlQuantizedMatmulParams(m, n_loc, k, gtype),
                                         n, rank * n_loc, [peer.contents_ptr()])
        assert mx.last_kernel_name() == "qmm_tc"
    enc.commit_and_wait()
    got = full.as_slice(np.float32).reshape(m, n)
    got_peer = peer.download(np.float32).reshape(m, n)
    y_ref, ad = orc.qmatmul(otype, wq, x, n, k, nthreads=8)
    assert norm_err(got, y_ref, ad) <= MM_TOL
    y16, _ = orc.qmatmul(otype, wq, x, n, k, f16_operands=True, nthreads=8)
    assert norm_err(got, y16, ad) <= 2e-5
    assert np.array_equal(got_peer.view(np.uint32), got.view(np.uint32))


def test_sharded_argument_errors(ctx):
    d = ctx.device
    gtype, otype = TYPES["Q8_0"]
    n, k = 256, 256
    wq = normal_weights(1, n, k, otype)
    xb, wb = ctx.buf(normal_acts(1, 9, k), mx.DType.F32), ctx.buf(wq, mx.DType.U8)
    out = d.alloc_buffer(9 * 2 * n * 4, mx.DType.F32)
    enc = d.command_encoder()
    with pytest.raises(mx.InvalidArgument):   # m = 0
        mx.quantized_matmul_ggml_sharded(enc, ctx.registry, d, xb, wb, out, mx.GgmlQuantizedMatmulParams(0, n, k, gtype), 2 * n, 0)
    with pytest.raises(mx.InvalidArgument):   # columns outside the full width
        mx.quantized_matmul_ggml_sharded(enc, ctx.registry, d, xb, wb, out, mx.GgmlQuantizedMatmulParams(1, n, k, gtype), 2 * n, n + 1)
    small = d.alloc_buffer(n * 4, mx.DType.F32)
    with pytest.raises(mx.InvalidArgument):   # result buffer must hold the full width
        mx.quantized_matmul_ggml_sharded(enc, ctx.registry, d, xb, wb, small, mx.GgmlQuantizedMatmulParams(1, n, k, gtype), 2 * n, 0)
