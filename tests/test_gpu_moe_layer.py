"""The expert half of a MoE FFN layer as one call (mlxn_moe_ffn_layer) against the chain of calls it stands for
(quantized_matmul_id_ggml for gate and up, silu_mul, quantized_matmul_id_ggml for down with n_tokens * top_k rows and
top_k = 1 -- what upstream's callers encode, benches/bench_mul_mm_id_qwen36_ffn.rs) and against the oracle."""
import numpy as np
import pytest

import mlx_native_b200 as mx
from oracle import oracle as orc
from tests.gpu_util import MM_TOL, MV_TOL, TYPES, Ctx, norm_err, normal_acts, normal_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


def make_layer(E, hidden, ffn, gname, dname, seed):
    (gt, go), (dt, do) = TYPES[gname], TYPES[dname]
    gate = np.concatenate([normal_weights(seed + e, ffn, hidden, go) for e in range(E)])
    up = np.concatenate([normal_weights(seed + 100 + e, ffn, hidden, go) for e in range(E)])
    down = np.concatenate([normal_weights(seed + 200 + e, hidden, ffn, do) for e in range(E)])
    return dict(gt=gt, go=go, dt=dt, do=do, gate=gate, up=up, down=down)


def route(T, E, top_k, seed):
    rng = np.random.default_rng(seed)
    return np.stack([rng.permutation(E)[:top_k] for _ in range(T)]).astype(np.uint32).reshape(-1)


def run_chain(ctx, L, x, ids, T, top_k, E, hidden, ffn):
    d, reg = ctx.device, ctx.registry
    pairs = T * top_k
    xb, ib = ctx.buf(x, mx.DType.F32), ctx.buf(ids, mx.DType.U32)
    wg, wu, wd = (ctx.buf(L[k], mx.DType.U8) for k in ("gate", "up", "down"))
    yg, yu, act = (d.alloc_buffer(pairs * ffn * 4, mx.DType.F32) for _ in range(3))
    yd = d.alloc_buffer(pairs * hidden * 4, mx.DType.F32)
    pg = mx.GgmlQuantizedMatmulIdParams(T, top_k, ffn, hidden, E, L["gate"].size // E, L["gt"])
    pd = mx.GgmlQuantizedMatmulIdParams(pairs, 1, hidden, ffn, E, L["down"].size // E, L["dt"])
    enc = d.command_encoder()
    mx.quantized_matmul_id_ggml(enc, reg, d, xb, wg, ib, yg, pg)
    mx.quantized_matmul_id_ggml(enc, reg, d, xb, wu, ib, yu, pg)
    mx.silu_mul(enc, reg, d, yg, yu, act, pairs * ffn)
    mx.quantized_matmul_id_ggml(enc, reg, d, act, wd, ib, yd, pd)
    enc.commit_and_wait()
    return (yg.as_slice(np.float32).reshape(pairs, ffn).copy(), yu.as_slice(np.float32).reshape(pairs, ffn).copy(),
            yd.as_slice(np.float32).reshape(pairs, hidden).copy())


def run_layer(ctx, L, x, ids, T, top_k, E, hidden, ffn):
    d, reg = ctx.device, ctx.registry
    pairs = T * top_k
    xb, ib = ctx.buf(x, mx.DType.F32), ctx.buf(ids, mx.DType.U32)
    wg, wu, wd = (ctx.buf(L[k], mx.DType.U8) for k in ("gate", "up", "down"))
    yg, yu = (d.alloc_buffer(pairs * ffn * 4, mx.DType.F32) for _ in range(2))
    yd = d.alloc_buffer(pairs * hidden * 4, mx.DType.F32)
    yd.as_mut_slice(np.float32)[:] = np.nan                          # every row must be written
    p = mx.MoeFfnLayerParams(T, top_k, hidden, ffn, E, L["gt"], L["gt"], L["dt"], L["gate"].size // E, L["up"].size // E,
                             L["down"].size // E)
    enc = d.command_encoder()
    mx.reset_counters()
    mx.moe_ffn_layer(enc, reg, d, xb, ib, wg, wu, wd, yg, yu, yd, p)
    enc.commit_and_wait()
    launches = mx.kernel_launch_count()
    return (yg.as_slice(np.float32).reshape(pairs, ffn).copy(), yu.as_slice(np.float32).reshape(pairs, ffn).copy(),
            yd.as_slice(np.float32).reshape(pairs, hidden).copy(), launches)


@pytest.mark.parametrize("T,E,top_k,hidden,ffn,gname,dname", [
    (96, 16, 4, 512, 256, "Q4_0", "Q6_K"),       # grouped route, the type mix of the benchmark layer
    (160, 8, 2, 256, 512, "Q8_0", "Q4_0"),       # ffn longer than hidden: the packed area is sized for the longer K
    (40, 32, 8, 1024, 256, "Q6_K", "Q8_0"),      # barely past the routing threshold, many empty experts
    (8, 16, 4, 512, 256, "Q4_0", "Q6_K"),        # decode: routed mat-vecs + fused SwiGLU mat-vec
    (1, 16, 8, 2048, 768, "Q4_0", "Q4_0"),
])
def test_layer_call_equals_the_chain(ctx, T, E, top_k, hidden, ffn, gname, dname):
    L = make_layer(E, hidden, ffn, gname, dname, seed=900 + T)
    x = normal_acts(T, T, hidden)
    ids = route(T, E, top_k, seed=T)
    g0, u0, d0 = run_chain(ctx, L, x, ids, T, top_k, E, hidden, ffn)
    g1, u1, d1, launches = run_layer(ctx, L, x, ids, T, top_k, E, hidden, ffn)
    assert np.array_equal(g0.view(np.uint32), g1.view(np.uint32))
    assert np.array_equal(u0.view(np.uint32), u1.view(np.uint32))
    if T > mx.MM_ID_ROUTING_THRESHOLD:
        assert np.array_equal(d0.view(np.uint32), d1.view(np.uint32))
        assert launches == 7 and mx.last_kernel_name() == "qmm_tc_id"    # map0, tile list, pack, 3 mat-mats, SwiGLU pack
    else:
        # (the chain above forms the SwiGLU in a kernel of its own, the layer call in the mat-vec's activation load: the
        #  same f32 values, but more than 16 rows take the streaming kernel in one form and not the other)
        assert float(np.max(np.abs(d0 - d1))) <= 2e-5 * float(np.max(np.abs(d0)))
        assert launches <= 3


def test_layer_call_against_the_oracle_and_bad_ids(ctx):
    T, E, top_k, hidden, ffn = 64, 8, 2, 256, 256
    L = make_layer(E, hidden, ffn, "Q4_0", "Q6_K", seed=77)
    x = normal_acts(5, T, hidden)
    ids = route(T, E, top_k, seed=3)
    ids[7] = 200                                                       # no such expert: a zero row in down_out
    g1, u1, d1, _ = run_layer(ctx, L, x, ids, T, top_k, E, hidden, ffn)
    good = ids < E
    safe = np.where(good, ids, 0).astype(np.uint32)
    xh = x.astype(np.float16).astype(np.float32)
    g_ref, gad = orc.qmatmul_id(L["go"], L["gate"], L["gate"].size // E, xh, safe, top_k, ffn, hidden, E, f16_operands=True, nthreads=8)
    u_ref, uad = orc.qmatmul_id(L["go"], L["up"], L["up"].size // E, xh, safe, top_k, ffn, hidden, E, f16_operands=True, nthreads=8)
    assert norm_err(g1[good], g_ref[good], gad[good]) <= MM_TOL and norm_err(u1[good], u_ref[good], uad[good]) <= MM_TOL
    act = orc.silu_mul(g1, u1).reshape(T * top_k, ffn)
    d_ref, dad = orc.qmatmul_id(L["do"], L["down"], L["down"].size // E, act, safe, 1, hidden, ffn, E, f16_operands=True, nthreads=8)
    assert norm_err(d1[good], d_ref[good], dad[good]) <= MM_TOL
    assert np.all(d1[~good] == 0.0) and np.all(np.isfinite(d1))


def test_layer_call_argument_errors(ctx):
    d, reg = ctx.device, ctx.registry
    T, E, top_k, hidden, ffn = 40, 4, 2, 256, 256
    L = make_layer(E, hidden, ffn, "Q4_0", "Q4_0", seed=5)
    bufs = [ctx.buf(normal_acts(1, T, hidden), mx.DType.F32), ctx.buf(route(T, E, top_k, 1), mx.DType.U32)]
    bufs += [ctx.buf(L[k], mx.DType.U8) for k in ("gate", "up", "down")]
    outs = [d.alloc_buffer(T * top_k * ffn * 4, mx.DType.F32), d.alloc_buffer(T * top_k * ffn * 4, mx.DType.F32),
            d.alloc_buffer(T * top_k * hidden * 4, mx.DType.F32)]
    ok = mx.MoeFfnLayerParams(T, top_k, hidden, ffn, E, L["gt"], L["gt"], L["dt"], L["gate"].size // E, L["up"].size // E, L["down"].size // E)
    small = d.alloc_buffer(64, mx.DType.F32)
    with pytest.raises(mx.InvalidArgument, match=r"moe_ffn_layer \(down\): output buffer too small"):
        mx.moe_ffn_layer(d.command_encoder(), reg, d, *bufs, outs[0], outs[1], small, ok)
    with pytest.raises(mx.InvalidArgument, match=r"moe_ffn_layer \(up\): output buffer too small"):
        mx.moe_ffn_layer(d.command_encoder(), reg, d, *bufs, outs[0], small, outs[2], ok)
    bad = mx.MoeFfnLayerParams(T, 0, hidden, ffn, E, L["gt"], L["gt"], L["dt"], L["gate"].size // E, L["up"].size // E, L["down"].size // E)
    with pytest.raises(mx.InvalidArgument, match="n_tokens \\* top_k"):
        mx.moe_ffn_layer(d.command_encoder(), reg, d, *bufs, *outs, bad)
