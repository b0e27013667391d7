"""Expert-sharded MoE FFN layer: the g ranks' work run one after the other on one GPU (each rank's kernels see
only its experts' weights and its local ids), partial results added on the host the way the all-reduce adds them.
Against the unsharded layer on the same GPU and against the oracle."""
import numpy as np
import pytest

import mlx_native_b200 as mx
from mlx_native_b200 import sharding
from oracle import oracle as orc
from tests.gpu_util import TYPES, Ctx, normal_acts, normal_weights

pytestmark = pytest.mark.gpu

E, TOP_K, HIDDEN, FFN = 16, 8, 512, 256


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


def ffn_layer(ctx, x, ids_buf, rw_buf, wg, wu, wd, n_experts, T, local):
    """One (possibly partial) layer on device buffers; returns (down outputs [T*top_k, hidden], combined [T, hidden])."""
    d, reg = ctx.device, ctx.registry
    g4, g6 = TYPES["Q4_0"][0], TYPES["Q6_K"][0]
    pairs = T * TOP_K
    xb = ctx.buf(x, mx.DType.F32)
    yg = d.alloc_buffer(pairs * FFN * 4, mx.DType.F32)
    yu = d.alloc_buffer(pairs * FFN * 4, mx.DType.F32)
    act = d.alloc_buffer(pairs * FFN * 4, mx.DType.F32)
    yd = d.alloc_buffer(pairs * HIDDEN * 4, mx.DType.F32)
    yd.as_mut_slice(np.float32)[:] = np.nan      # rows of other ranks' pairs must never be read
    out = d.alloc_buffer(T * HIDDEN * 4, mx.DType.F32)
    pg = mx.GgmlQuantizedMatmulIdParams(T, TOP_K, FFN, HIDDEN, n_experts, wg.size // n_experts, g4)
    pd = mx.GgmlQuantizedMatmulIdParams(pairs, 1, HIDDEN, FFN, n_experts, wd.size // n_experts, g6)
    wgb, wub, wdb = ctx.buf(wg, mx.DType.U8), ctx.buf(wu, mx.DType.U8), ctx.buf(wd, mx.DType.U8)
    enc = d.command_encoder()
    mx.quantized_matmul_id_ggml(enc, reg, d, xb, wgb, ids_buf, yg, pg)
    mx.quantized_matmul_id_ggml(enc, reg, d, xb, wub, ids_buf, yu, pg)
    mx.silu_mul(enc, reg, d, yg, yu, act, pairs * FFN)
    mx.quantized_matmul_id_ggml(enc, reg, d, act, wdb, ids_buf, yd, pd)
    if local:
        mx.moe_weighted_reduce_local(enc, reg, d, rw_buf, yd, ids_buf, out, T, TOP_K, HIDDEN)
    else:
        mx.moe_weighted_reduce(enc, reg, d, rw_buf, yd, out, T, TOP_K, HIDDEN)
    enc.commit_and_wait()
    return yd.as_slice(np.float32).reshape(pairs, HIDDEN).copy(), out.as_slice(np.float32).reshape(T, HIDDEN).copy()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("T", [3, 40])     # mat-vec route and bucketed mat-mat route
def test_expert_sharded_layer_matches_unsharded(ctx, T, world):
    d, reg = ctx.device, ctx.registry
    o4, o6 = TYPES["Q4_0"][1], TYPES["Q6_K"][1]
    wg = normal_weights(11, E * FFN, HIDDEN, o4)
    wu = normal_weights(12, E * FFN, HIDDEN, o4)
    wd = normal_weights(13, E * HIDDEN, FFN, o6)
    x = normal_acts(14, T, HIDDEN)
    logits = np.random.default_rng(15).standard_normal((T, E)).astype(np.float32)
    lg = ctx.buf(logits, mx.DType.F32)
    ids = d.alloc_buffer(T * TOP_K * 4, mx.DType.U32, [T, TOP_K])
    rw = d.alloc_buffer(T * TOP_K * 4, mx.DType.F32, [T, TOP_K])
    enc = d.command_encoder()
    mx.moe_softmax_topk(enc, reg, d, lg, ids, rw, T, E, TOP_K)
    enc.commit_and_wait()
    ids_h = ids.as_slice(np.uint32).copy()

    yd_full, out_full = ffn_layer(ctx, x, ids, rw, wg, wu, wd, E, T, local=False)

    total = np.zeros_like(out_full)
    seen = np.zeros(T * TOP_K, dtype=bool)
    for r in range(world):
        lo, cnt = sharding.shard_experts(E, r, world)
        lids = d.alloc_buffer(T * TOP_K * 4, mx.DType.U32, [T, TOP_K])
        enc = d.command_encoder()
        mx.moe_expert_shard_route(enc, reg, d, ids, lids, T * TOP_K, lo, cnt)
        enc.commit_and_wait()
        lids_h = lids.as_slice(np.uint32).copy()
        assert np.array_equal(lids_h, sharding.local_expert_ids(ids_h, lo, cnt))     # ids: bit-exact
        yd_r, out_r = ffn_layer(ctx, x, lids, rw,
                                sharding.shard_expert_bytes(wg, wg.size // E, E, r, world),
                                sharding.shard_expert_bytes(wu, wu.size // E, E, r, world),
                                sharding.shard_expert_bytes(wd, wd.size // E, E, r, world), cnt, T, local=True)
        mine = lids_h != sharding.NOT_LOCAL
        assert not (seen & mine).any()
        seen |= mine
        # a pair's rows are computed by the same kernel from the same bytes as on one GPU: bit-identical
        assert np.array_equal(yd_r[mine], yd_full[mine])
        assert np.isfinite(out_r).all()
        total += out_r
    assert seen.all()
    # the combine adds the ranks' partial sums, so only the order of the top_k additions differs
    scale = np.abs(out_full).max()
    assert np.max(np.abs(total - out_full)) <= 1e-5 * scale

    # and the whole thing against the oracle
    flat = ids_h.reshape(-1)
    rg, _ = orc.qmatmul_id(o4, wg, wg.size // E, x, flat, TOP_K, FFN, HIDDEN, E, nthreads=8)
    ru, _ = orc.qmatmul_id(o4, wu, wu.size // E, x, flat, TOP_K, FFN, HIDDEN, E, nthreads=8)
    rd, _ = orc.qmatmul_id(o6, wd, wd.size // E, orc.silu_mul(rg, ru), flat, 1, HIDDEN, FFN, E, nthreads=8)
    want = orc.moe_weighted_reduce(rd, rw.as_slice(np.float32).reshape(T, TOP_K).copy(), T, TOP_K, HIDDEN)
    tol = 2e-3 if T > mx.mm_id_routing_threshold() else 2e-5
    assert np.max(np.abs(total - want)) <= tol * np.abs(want).max()


def test_shard_route_argument_errors(ctx):
    d, reg = ctx.device, ctx.registry
    ids = d.alloc_buffer(64, mx.DType.U32)
    small = d.alloc_buffer(16, mx.DType.U32)
    enc = d.command_encoder()
    with pytest.raises(mx.MlxError):
        mx.moe_expert_shard_route(enc, reg, d, ids, small, 16, 0, 4)
    with pytest.raises(mx.MlxError):
        mx.moe_expert_shard_route(enc, reg, d, ids, ids, 0, 0, 4)
