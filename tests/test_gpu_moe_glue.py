"""Router softmax/top-k, SwiGLU and weighted combine against the oracle, and one whole MoE FFN layer
chained the way the upstream engine chains it (gate/up with top_k = 8, down with n_tokens = T*8, top_k = 1)."""
import numpy as np
import pytest

import mlx_native_b200 as mx
from oracle import oracle as orc
from tests.gpu_util import TYPES, Ctx, norm_err, normal_acts, normal_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


def route(ctx, logits, top_k):
    T, E = logits.shape
    d = ctx.device
    lg = ctx.buf(logits, mx.DType.F32)
    ids = d.alloc_buffer(T * top_k * 4, mx.DType.U32, [T, top_k])
    w = d.alloc_buffer(T * top_k * 4, mx.DType.F32, [T, top_k])
    enc = d.command_encoder()
    mx.moe_softmax_topk(enc, ctx.registry, d, lg, ids, w, T, E, top_k)
    enc.commit_and_wait()
    return ids.as_slice(np.uint32).reshape(T, top_k).copy(), w.as_slice(np.float32).reshape(T, top_k).copy()


@pytest.mark.parametrize("T,E,top_k", [(1, 128, 8), (512, 128, 8), (7, 8, 2), (3, 96, 4), (5, 256, 8)])
def test_softmax_topk(ctx, T, E, top_k):
    logits = np.random.default_rng(T * 1000 + E).standard_normal((T, E)).astype(np.float32)
    o_ids, o_w = orc.moe_softmax_topk(logits, top_k)
    # the seeded inputs have no near-tie at the selection boundary, so expf differences cannot flip an id
    p = np.exp(logits.astype(np.float64) - logits.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    srt = -np.sort(-p, axis=1)
    gaps = (srt[:, :top_k] - srt[:, 1:top_k + 1]) / srt[:, :top_k]
    assert gaps.min() > 1e-5
    ids, w = route(ctx, logits, top_k)
    assert np.array_equal(ids, o_ids)          # expert ids and their order: bit-exact
    assert np.allclose(w, o_w, rtol=2e-6, atol=1e-9)


def test_softmax_topk_ties_keep_lower_index(ctx):
    ids, w = route(ctx, np.zeros((2, 16), np.float32), 4)
    assert ids.tolist() == [[0, 1, 2, 3]] * 2 and np.allclose(w, 0.25)


def test_silu_mul_and_weighted_reduce(ctx):
    d = ctx.device
    rng = np.random.default_rng(2)
    g = rng.standard_normal(5000).astype(np.float32) * 3
    u = rng.standard_normal(5000).astype(np.float32)
    gb, ub = ctx.buf(g, mx.DType.F32), ctx.buf(u, mx.DType.F32)
    ob = d.alloc_buffer(g.nbytes, mx.DType.F32)
    enc = d.command_encoder()
    mx.silu_mul(enc, ctx.registry, d, gb, ub, ob, g.size)
    enc.commit_and_wait()
    assert np.allclose(ob.as_slice(np.float32), orc.silu_mul(g, u), rtol=2e-6, atol=1e-7)

    T, top_k, h = 9, 8, 300
    y = rng.standard_normal((T * top_k, h)).astype(np.float32)
    w = rng.random((T, top_k)).astype(np.float32)
    yb, wb = ctx.buf(y, mx.DType.F32), ctx.buf(w, mx.DType.F32)
    out = d.alloc_buffer(T * h * 4, mx.DType.F32)
    enc = d.command_encoder()
    mx.moe_weighted_reduce(enc, ctx.registry, d, wb, yb, out, T, top_k, h)
    enc.commit_and_wait()
    want = orc.moe_weighted_reduce(y, w, T, top_k, h)
    assert np.allclose(out.as_slice(np.float32).reshape(T, h), want, rtol=1e-5, atol=1e-6)
    # with shared expert and residual terms
    ys = rng.standard_normal((T, h)).astype(np.float32)
    sl = rng.standard_normal(T).astype(np.float32)
    res = rng.standard_normal((T, h)).astype(np.float32)
    enc = d.command_encoder()
    mx.moe_weighted_reduce(enc, ctx.registry, d, wb, yb, out, T, top_k, h, sh_logit=ctx.buf(sl, mx.DType.F32),
                           y_shared=ctx.buf(ys, mx.DType.F32), residual=ctx.buf(res, mx.DType.F32))
    enc.commit_and_wait()
    want2 = want + (1.0 / (1.0 + np.exp(-sl)))[:, None] * ys + res
    assert np.allclose(out.as_slice(np.float32).reshape(T, h), want2, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("T", [1, 40])
def test_moe_ffn_layer(ctx, T):
    """Router -> gate/up (Q4_0) -> SwiGLU -> down (Q6_K) -> combine, scaled-down expert shapes, vs the oracle."""
    d = ctx.device
    E, top_k, hidden, ffn = 16, 8, 512, 256
    g4, o4 = TYPES["Q4_0"]
    g6, o6 = TYPES["Q6_K"]
    wg = normal_weights(1, E * ffn, hidden, o4)
    wu = normal_weights(2, E * ffn, hidden, o4)
    wd = normal_weights(3, E * hidden, ffn, o6)
    x = normal_acts(4, T, hidden)
    logits = np.random.default_rng(5).standard_normal((T, E)).astype(np.float32)

    ids, rw = route(ctx, logits, top_k)
    o_ids, o_rw = orc.moe_softmax_topk(logits, top_k)
    assert np.array_equal(ids, o_ids)
    flat = ids.reshape(-1)
    yg, _ = ctx.matmul_id(g4, wg, wg.size // E, x, flat, top_k, ffn, hidden, E)
    yu, _ = ctx.matmul_id(g4, wu, wu.size // E, x, flat, top_k, ffn, hidden, E)
    gb, ub = ctx.buf(yg, mx.DType.F32), ctx.buf(yu, mx.DType.F32)
    act = d.alloc_buffer(yg.nbytes, mx.DType.F32)
    enc = d.command_encoder()
    mx.silu_mul(enc, ctx.registry, d, gb, ub, act, yg.size)
    enc.commit_and_wait()
    a = act.as_slice(np.float32).reshape(T * top_k, ffn).copy()
    yd, _ = ctx.matmul_id(g6, wd, wd.size // E, a, flat, 1, hidden, ffn, E)
    out = d.alloc_buffer(T * hidden * 4, mx.DType.F32)
    enc = d.command_encoder()
    mx.moe_weighted_reduce(enc, ctx.registry, d, ctx.buf(rw, mx.DType.F32), ctx.buf(yd, mx.DType.F32), out, T, top_k,
                           hidden)
    enc.commit_and_wait()
    got = out.as_slice(np.float32).reshape(T, hidden)

    rg, _ = orc.qmatmul_id(o4, wg, wg.size // E, x, flat, top_k, ffn, hidden, E, nthreads=8)
    ru, _ = orc.qmatmul_id(o4, wu, wu.size // E, x, flat, top_k, ffn, hidden, E, nthreads=8)
    ra = orc.silu_mul(rg, ru)
    rd, _ = orc.qmatmul_id(o6, wd, wd.size // E, ra, flat, 1, hidden, ffn, E, nthreads=8)
    want = orc.moe_weighted_reduce(rd, o_rw, T, top_k, hidden)
    scale = np.abs(want).max()
    tol = 2e-3 if T > mx.mm_id_routing_threshold() else 2e-5
    assert np.max(np.abs(got - want)) <= tol * scale


def test_moe_ffn_layer_full_size_sampled(ctx):
    """The MoE configuration at its full size (128 experts, top-8, hidden 2048, ffn 768, T = 512: the persistent grouped
    mat-mat with 768 / 2048 work items), checked on a sample of (token, slot) pairs against the oracle, stage by stage."""
    d = ctx.device
    E, top_k, hidden, ffn, T = 128, 8, 2048, 768, 512
    g4, o4 = TYPES["Q4_0"]
    g6, o6 = TYPES["Q6_K"]
    # one seeded expert, rolled by a different amount per expert (distinct weights everywhere, quick to build)
    base_g = normal_weights(21, ffn, hidden, o4).reshape(ffn, -1)
    base_u = normal_weights(22, ffn, hidden, o4).reshape(ffn, -1)
    base_d = normal_weights(23, hidden, ffn, o6).reshape(hidden, -1)
    wg = np.concatenate([np.roll(base_g, e, axis=0) for e in range(E)]).reshape(-1)
    wu = np.concatenate([np.roll(base_u, 3 * e, axis=0) for e in range(E)]).reshape(-1)
    wd = np.concatenate([np.roll(base_d, 5 * e, axis=0) for e in range(E)]).reshape(-1)
    x = normal_acts(24, T, hidden)
    logits = np.random.default_rng(25).standard_normal((T, E)).astype(np.float32)
    ids, rw = route(ctx, logits, top_k)
    o_ids, o_rw = orc.moe_softmax_topk(logits, top_k)
    assert np.array_equal(ids, o_ids)
    flat = ids.reshape(-1)

    yg, _ = ctx.matmul_id(g4, wg, wg.size // E, x, flat, top_k, ffn, hidden, E)
    assert mx.last_kernel_name() == "qmm_tc_id"
    yu, _ = ctx.matmul_id(g4, wu, wu.size // E, x, flat, top_k, ffn, hidden, E)
    gb, ub = ctx.buf(yg, mx.DType.F32), ctx.buf(yu, mx.DType.F32)
    act = d.alloc_buffer(yg.nbytes, mx.DType.F32)
    enc = d.command_encoder()
    mx.silu_mul(enc, ctx.registry, d, gb, ub, act, yg.size)
    enc.commit_and_wait()
    a = act.as_slice(np.float32).reshape(T * top_k, ffn).copy()
    yd, _ = ctx.matmul_id(g6, wd, wd.size // E, a, flat, 1, hidden, ffn, E)
    out = d.alloc_buffer(T * hidden * 4, mx.DType.F32)
    enc = d.command_encoder()
    mx.moe_weighted_reduce(enc, ctx.registry, d, ctx.buf(rw, mx.DType.F32), ctx.buf(yd, mx.DType.F32), out, T, top_k, hidden)
    enc.commit_and_wait()
    got = out.as_slice(np.float32).reshape(T, hidden)

    # every output row was written (no NaN left from an unvisited tile) and a sample matches the oracle
    assert np.isfinite(yg).all() and np.isfinite(yd).all() and np.isfinite(got).all()
    pairs = np.random.default_rng(26).choice(T * top_k, size=96, replace=False)
    sel_ids = flat[pairs]
    rg, adg = orc.qmatmul_id(o4, wg, wg.size // E, x[pairs // top_k], sel_ids, 1, ffn, hidden, E, f16_operands=True, nthreads=8)
    assert norm_err(yg[pairs], rg, adg) <= 2e-5          # against the f16-operand oracle
    rd, add = orc.qmatmul_id(o6, wd, wd.size // E, a[pairs], sel_ids, 1, hidden, ffn, E, f16_operands=True, nthreads=8)
    assert norm_err(yd[pairs], rd, add) <= 2e-5
    toks = np.unique(pairs // top_k)[:16]
    want = orc.moe_weighted_reduce(yd.reshape(T, top_k, hidden)[toks].reshape(-1, hidden), rw[toks], len(toks), top_k, hidden)
    assert np.allclose(got[toks], want, rtol=1e-5, atol=1e-6)


def test_moe_ffn_layer_full_size_decode(ctx):
    """The MoE configuration at its full size for one token (128 experts, top-8, hidden 2048, ffn 768; the routed
    mat-vec form, n_tokens = 1 for gate / up and n_tokens = 8, top_k = 1 for down): every output against the oracle."""
    d = ctx.device
    E, top_k, hidden, ffn, T = 128, 8, 2048, 768, 1
    g4, o4 = TYPES["Q4_0"]
    g6, o6 = TYPES["Q6_K"]
    base_g = normal_weights(71, ffn, hidden, o4).reshape(ffn, -1)
    base_u = normal_weights(72, ffn, hidden, o4).reshape(ffn, -1)
    base_d = normal_weights(73, hidden, ffn, o6).reshape(hidden, -1)
    wg = np.concatenate([np.roll(base_g, e, axis=0) for e in range(E)]).reshape(-1)
    wu = np.concatenate([np.roll(base_u, 3 * e, axis=0) for e in range(E)]).reshape(-1)
    wd = np.concatenate([np.roll(base_d, 5 * e, axis=0) for e in range(E)]).reshape(-1)
    x = normal_acts(74, T, hidden)
    logits = np.random.default_rng(75).standard_normal((T, E)).astype(np.float32)
    ids, rw = route(ctx, logits, top_k)
    o_ids, o_rw = orc.moe_softmax_topk(logits, top_k)
    assert np.array_equal(ids, o_ids)
    flat = ids.reshape(-1)
    yg, _ = ctx.matmul_id(g4, wg, wg.size // E, x, flat, top_k, ffn, hidden, E)
    assert mx.last_kernel_name().startswith("qmv")
    yu, _ = ctx.matmul_id(g4, wu, wu.size // E, x, flat, top_k, ffn, hidden, E)
    rg, adg = orc.qmatmul_id(o4, wg, wg.size // E, x, flat, top_k, ffn, hidden, E, nthreads=8)
    ru, adu = orc.qmatmul_id(o4, wu, wu.size // E, x, flat, top_k, ffn, hidden, E, nthreads=8)
    assert norm_err(yg, rg, adg) <= 1e-5 and norm_err(yu, ru, adu) <= 1e-5
    act = d.alloc_buffer(yg.nbytes, mx.DType.F32)
    enc = d.command_encoder()
    mx.silu_mul(enc, ctx.registry, d, ctx.buf(yg, mx.DType.F32), ctx.buf(yu, mx.DType.F32), act, yg.size)
    enc.commit_and_wait()
    a = act.as_slice(np.float32).reshape(T * top_k, ffn).copy()
    yd, _ = ctx.matmul_id(g6, wd, wd.size // E, a, flat, 1, hidden, ffn, E)
    rd, add = orc.qmatmul_id(o6, wd, wd.size // E, a, flat, 1, hidden, ffn, E, nthreads=8)
    assert norm_err(yd, rd, add) <= 1e-5
    out = d.alloc_buffer(T * hidden * 4, mx.DType.F32)
    enc = d.command_encoder()
    mx.moe_weighted_reduce(enc, ctx.registry, d, ctx.buf(rw, mx.DType.F32), ctx.buf(yd, mx.DType.F32), out, T, top_k, hidden)
    enc.commit_and_wait()
    want = orc.moe_weighted_reduce(yd, o_rw, T, top_k, hidden)
    assert np.allclose(out.as_slice(np.float32).reshape(T, hidden), want, rtol=1e-5, atol=1e-6)
