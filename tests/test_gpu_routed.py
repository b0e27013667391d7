"""Parity of the expert-routed path: mv_id, bucketing (map0) and grouped mat-mat, through the C ABI.
Mirrors upstream tests/test_quantized_matmul_id_ggml.rs and tests/test_quantized_matmul_id_mm.rs."""
import numpy as np
import pytest

import mlx_native_b200 as mx
from oracle import oracle as orc
from tests import ref_numpy as rn
from tests.gpu_util import MM_TOL, MV_TOL, TYPES, Ctx, norm_err, normal_acts, normal_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


def stacked_lcg(otype, n_experts, n, k, seed0=100):
    ws = [orc.quantize(otype, orc.lcg_f32(seed0 + e, n * k)) for e in range(n_experts)]
    return np.concatenate(ws), ws[0].size, ws


# ---- mv_id equals the per-expert mat-vec bit for bit (tests/test_quantized_matmul_id_ggml.rs:328-573)
@pytest.mark.parametrize("qmv", ["stream", "simple"])
@pytest.mark.parametrize("tname,n_tokens,n,k", [("Q4_0", 1, 64, 128), ("Q8_0", 1, 64, 128), ("Q4_0", 4, 64, 128),
                                                ("Q8_0", 4, 64, 128), ("Q8_0", 1, 256, 256), ("Q4_0", 1, 256, 256),
                                                ("Q6_K", 4, 64, 256), ("Q6_K", 2, 96, 768), ("Q4_0", 3, 768, 2048)])
def test_id_vs_nonid_bit_exact(ctx, qmv, tname, n_tokens, n, k):
    mx.set_option("qmv", qmv)
    try:
        gtype, otype = TYPES[tname]
        n_experts, top_k = 8, 2
        stacked, stride, ws = stacked_lcg(otype, n_experts, n, k)
        x = orc.lcg_f32(42, n_tokens * k).reshape(n_tokens, k)
        ids = np.array([(t * 3 + s * 7 + 1) % n_experts for t in range(n_tokens) for s in range(top_k)], np.uint32)
        y, _ = ctx.matmul_id(gtype, stacked, stride, x, ids, top_k, n, k, n_experts)
        assert mx.last_kernel_name().startswith("qmv")
        for r in range(n_tokens * top_k):
            yr = ctx.matmul(gtype, ws[ids[r]], x[r // top_k][None], n, k)
            assert np.array_equal(y[r].view(np.uint32), yr[0].view(np.uint32)), f"row {r}"
        y_ref, ad = orc.qmatmul_id(otype, stacked, stride, x, ids, top_k, n, k, n_experts)
        assert norm_err(y, y_ref, ad) <= MV_TOL
    finally:
        mx.set_option("qmv", "auto")


def test_id_expert_stride_with_padding(ctx):
    gtype, otype = TYPES["Q8_0"]
    n_experts, top_k, n, k, n_tokens = 4, 2, 32, 256, 3
    ws = [orc.quantize(otype, orc.lcg_f32(7 + e, n * k)) for e in range(n_experts)]
    stride = ws[0].size + 34 * 3  # padding between experts, still 2-byte aligned
    stacked = np.zeros(stride * n_experts, np.uint8)
    for e in range(n_experts):
        stacked[e * stride:e * stride + ws[e].size] = ws[e]
    x = normal_acts(2, n_tokens, k)
    ids = np.array([[0, 3], [2, 1], [3, 3]], np.uint32).reshape(-1)
    y, _ = ctx.matmul_id(gtype, stacked, stride, x, ids, top_k, n, k, n_experts)
    y_ref, ad = orc.qmatmul_id(otype, stacked, stride, x, ids, top_k, n, k, n_experts)
    assert norm_err(y, y_ref, ad) <= MV_TOL


# ---- bucketing: htpe / hids equal the scan-order reference exactly (tests/test_quantized_matmul_id_mm.rs:340-449)
@pytest.mark.parametrize("n_tokens,n_experts,top_k", [(16, 8, 8), (64, 32, 8), (17, 16, 8), (16, 64, 8), (40, 128, 1),
                                                      (513, 128, 8), (33, 7, 3)])
def test_map0_exact(ctx, n_tokens, n_experts, top_k):
    gtype, otype = TYPES["Q4_0"]
    n, k = 64, 128
    w1 = orc.quantize(otype, np.zeros(n * k, np.float32))
    stacked = np.tile(w1, n_experts)
    if top_k == 8:
        ids = np.array([(t * 17 + s * 13 + 7) % n_experts for t in range(n_tokens) for s in range(top_k)], np.uint32)
    else:
        rng = np.random.default_rng(n_tokens)
        ids = np.stack([rng.permutation(n_experts)[:top_k] for _ in range(n_tokens)]).astype(np.uint32).reshape(-1)
    x = np.zeros((n_tokens, k), np.float32)
    _, (htpe, hids) = ctx.matmul_id(gtype, stacked, w1.size, x, ids, top_k, n, k, n_experts, mode="force_mm")
    counts, lists = rn.bucket_scan_order(ids, n_tokens, top_k, n_experts)
    got_counts = htpe.as_slice(np.uint32)[:n_experts]
    got = hids.as_slice(np.int32).reshape(n_experts, n_tokens)
    assert got_counts.tolist() == counts
    for e in range(n_experts):
        assert got[e, :counts[e]].tolist() == lists[e]
    o_htpe, o_hids = orc.moe_map0(ids, n_tokens, top_k, n_experts)
    assert np.array_equal(got_counts, o_htpe)
    for e in range(n_experts):
        assert np.array_equal(got[e, :counts[e]], o_hids[e, :counts[e]])


# ---- grouped mat-mat equals mv_id (and the oracle) (tests/test_quantized_matmul_id_mm.rs:180-319, 456-563)
MMID = [("Q4_0", 16, 8, 64, 128, 5e-3), ("Q4_0", 64, 32, 128, 512, 5e-2), ("Q8_0", 16, 8, 64, 128, 2e-3),
        ("Q8_0", 64, 32, 128, 512, 2e-2), ("Q6_K", 16, 8, 32, 256, 5e-3), ("Q6_K", 64, 32, 128, 512, 5e-2),
        ("Q4_0", 17, 16, 72, 256, 5e-3), ("Q4_0", 16, 64, 64, 128, 5e-3)]


@pytest.mark.parametrize("qmm", ["tc", "simt"])
@pytest.mark.parametrize("tname,n_tokens,n_experts,n,k,tol", MMID)
def test_mm_id_matches_mv_id(ctx, qmm, tname, n_tokens, n_experts, n, k, tol):
    mx.set_option("qmm", qmm)
    try:
        gtype, otype = TYPES[tname]
        top_k = 8
        stacked, stride, _ = stacked_lcg(otype, n_experts, n, k, seed0=1000)
        x = orc.lcg_f32(0xBEEF, n_tokens * k).reshape(n_tokens, k)
        ids = np.array([(t * 17 + s * 13 + 7) % n_experts for t in range(n_tokens) for s in range(top_k)], np.uint32)
        y_mm, _ = ctx.matmul_id(gtype, stacked, stride, x, ids, top_k, n, k, n_experts, mode="force_mm")
        assert mx.last_kernel_name() == ("qmm_tc_id" if qmm == "tc" else "qmm_simt_id")
        y_mv, _ = ctx.matmul_id(gtype, stacked, stride, x, ids, top_k, n, k, n_experts)  # n_tokens <= 32 -> mv_id
        if n_tokens <= mx.mm_id_routing_threshold():
            assert mx.last_kernel_name().startswith("qmv")
            assert np.max(np.abs(y_mm - y_mv)) <= tol
        y_ref, ad = orc.qmatmul_id(otype, stacked, stride, x, ids, top_k, n, k, n_experts, nthreads=8)
        assert norm_err(y_mm, y_ref, ad) <= MM_TOL
        y16, _ = orc.qmatmul_id(otype, stacked, stride, x, ids, top_k, n, k, n_experts, f16_operands=True, nthreads=8)
        assert norm_err(y_mm, y16, ad) <= 2e-5
    finally:
        mx.set_option("qmm", "tc")


@pytest.mark.parametrize("mode", ["auto", "pooled"])
def test_routing_threshold_and_pooled(ctx, mode):
    """n_tokens > 32 takes the grouped mat-mat (any top_k); the pooled form leaves the bucketing
    in the caller's scratch; top_k = 1 is the down-projection convention (n_tokens = T*top_k rows, flat ids)."""
    gtype, otype = TYPES["Q6_K"]
    n_experts, n, k = 16, 96, 768
    stacked = normal_weights(4, n_experts * n, k, otype)
    stride = stacked.size // n_experts
    T, top_k = 48, 8
    rng = np.random.default_rng(5)
    ids = np.stack([rng.permutation(n_experts)[:top_k] for _ in range(T)]).astype(np.uint32).reshape(-1)
    x = normal_acts(8, T, k)
    y, scratch = ctx.matmul_id(gtype, stacked, stride, x, ids, top_k, n, k, n_experts, mode=mode)
    assert mx.last_kernel_name() == "qmm_tc_id"
    y_ref, ad = orc.qmatmul_id(otype, stacked, stride, x, ids, top_k, n, k, n_experts, nthreads=8)
    assert norm_err(y, y_ref, ad) <= MM_TOL
    if mode == "pooled":
        counts, _ = rn.bucket_scan_order(ids, T, top_k, n_experts)
        assert scratch.htpe.as_slice(np.uint32)[:n_experts].tolist() == counts
    # down projection: one row per (token, slot), top_k = 1
    xd = normal_acts(9, T * top_k, k)
    yd, _ = ctx.matmul_id(gtype, stacked, stride, xd, ids, 1, n, k, n_experts, mode=mode)
    assert mx.last_kernel_name() == "qmm_tc_id"
    yd_ref, add = orc.qmatmul_id(otype, stacked, stride, xd, ids, 1, n, k, n_experts, nthreads=8)
    assert norm_err(yd, yd_ref, add) <= MM_TOL
    # other top_k values (upstream falls back to mv_id for them and lists that as a gap,
    # docs/moe-q-perf-audit-2026-04-27.md:79-84): the bucketing takes any top_k, so they take the grouped route too
    for tk in (2, 3, 5):
        idsk = ids.reshape(T, top_k)[:, :tk].reshape(-1)
        yk, _ = ctx.matmul_id(gtype, stacked, stride, x, idsk, tk, n, k, n_experts, mode=mode)
        assert mx.last_kernel_name() == "qmm_tc_id"
        yk_ref, adk = orc.qmatmul_id(otype, stacked, stride, x, idsk, tk, n, k, n_experts, nthreads=8)
        assert norm_err(yk, yk_ref, adk) <= MM_TOL
        yk16, _ = orc.qmatmul_id(otype, stacked, stride, x, idsk, tk, n, k, n_experts, f16_operands=True, nthreads=8)
        assert norm_err(yk, yk16, adk) <= 2e-5
    # an id past n_experts gives a zero row on the grouped route, as on the mat-vec route
    bad = ids.copy()
    bad[5] = n_experts + 3
    bad[77] = 0x10005                        # its low 16 bits name a real expert: must not be mistaken for it
    yb, _ = ctx.matmul_id(gtype, stacked, stride, x, bad, top_k, n, k, n_experts, mode=mode)
    assert np.all(yb[5] == 0) and np.all(yb[77] == 0)
    keep = np.ones(T * top_k, bool)
    keep[[5, 77]] = False
    assert norm_err(yb[keep], y_ref[keep], ad[keep]) <= MM_TOL


def test_pooled_capacity_errors(ctx):
    d = ctx.device
    gtype = mx.GgmlType.Q4_0
    n_experts, n, k, T = 8, 64, 128, 40
    enc = d.command_encoder()
    x = d.alloc_buffer(T * k * 4, mx.DType.F32)
    w = d.alloc_buffer(n_experts * n * (k // 32) * 18, mx.DType.U8)
    ids = d.alloc_buffer(T * 8 * 4, mx.DType.U32)
    y = d.alloc_buffer(T * 8 * n * 4, mx.DType.F32)
    p = mx.GgmlQuantizedMatmulIdParams(T, 8, n, k, n_experts, n * (k // 32) * 18, gtype)
    small = mx.IdMmScratch.alloc(d, n_experts, 16)
    with pytest.raises(mx.InvalidArgument, match=r"IdMmScratch: n_tokens \(40\) > cap \(16\)"):
        mx.quantized_matmul_id_ggml_pooled(enc, ctx.registry, d, x, w, ids, y, small, p)
    few = mx.IdMmScratch.alloc(d, 4, 64)
    with pytest.raises(mx.InvalidArgument, match=r"IdMmScratch: n_experts \(8\) > cap \(4\)"):
        mx.quantized_matmul_id_ggml_pooled(enc, ctx.registry, d, x, w, ids, y, few, p)


def test_id_errors(ctx):
    d = ctx.device
    enc = d.command_encoder()
    x = d.alloc_buffer(2 * 128 * 4, mx.DType.F32)
    w = d.alloc_buffer(4 * 64 * 4 * 18, mx.DType.U8)
    ids = d.alloc_buffer(4 * 4, mx.DType.U32)
    y = d.alloc_buffer(4 * 64 * 4, mx.DType.F32)
    P = mx.GgmlQuantizedMatmulIdParams
    pe = 64 * 4 * 18
    with pytest.raises(mx.InvalidArgument, match="n_tokens, K, and N must all be > 0"):
        mx.quantized_matmul_id_ggml(enc, ctx.registry, d, x, w, ids, y, P(0, 2, 64, 128, 4, pe, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match="top_k must be > 0"):
        mx.quantized_matmul_id_ggml(enc, ctx.registry, d, x, w, ids, y, P(2, 0, 64, 128, 4, pe, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match="n_experts must be > 0"):
        mx.quantized_matmul_id_ggml(enc, ctx.registry, d, x, w, ids, y, P(2, 2, 64, 128, 0, pe, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match=r"expert_stride \(100\) < per_expert_bytes \(4608\)"):
        mx.quantized_matmul_id_ggml(enc, ctx.registry, d, x, w, ids, y, P(2, 2, 64, 128, 4, 100, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match="weight buffer too small: expected 36864 bytes for 8 experts"):
        mx.quantized_matmul_id_ggml(enc, ctx.registry, d, x, w, ids, y, P(2, 2, 64, 128, 8, pe, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match="ids buffer too small"):
        mx.quantized_matmul_id_ggml(enc, ctx.registry, d, x, w, ids, y, P(2, 4, 64, 128, 4, pe, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match="input buffer too small"):
        mx.quantized_matmul_id_ggml(enc, ctx.registry, d, x, w, ids, y, P(3, 1, 64, 128, 4, pe, mx.GgmlType.Q4_0))
    small_y = d.alloc_buffer(64 * 4, mx.DType.F32)
    with pytest.raises(mx.InvalidArgument, match="output buffer too small"):
        mx.quantized_matmul_id_ggml(enc, ctx.registry, d, x, w, ids, small_y, P(2, 2, 64, 128, 4, pe, mx.GgmlType.Q4_0))


def test_out_of_range_expert_id_writes_zeros(ctx):
    gtype, otype = TYPES["Q8_0"]
    n_experts, n, k = 4, 32, 256
    stacked = normal_weights(1, n_experts * n, k, otype)
    ids = np.array([1, 9, 3, 2], np.uint32)  # 9 is out of range
    x = normal_acts(1, 2, k)
    y, _ = ctx.matmul_id(gtype, stacked, stacked.size // n_experts, x, ids, 2, n, k, n_experts)
    assert np.all(y[1] == 0) and np.any(y[0] != 0)
