"""Fused SwiGLU + expert-routed mat-vec (upstream quantized_matmul_id_swiglu_q4_0, src/ops/quantized_matmul_id_ggml.rs:551-670,
tests/test_quantized_matmul_id_swiglu.rs) and the few-row routed mat-vec on the register-level kernel, against the oracle."""
import numpy as np
import pytest

import mlx_native_b200 as mx
from oracle import oracle as orc
from tests.gpu_util import MM_TOL, MV_TOL, TYPES, Ctx, norm_err, normal_acts, normal_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


def stacked(otype, n_experts, n, k, seed=500):
    ws = [normal_weights(seed + e, n, k, otype) for e in range(n_experts)]
    return np.concatenate(ws), ws[0].size


def run_fused(ctx, gtype, w, stride, gate, up, ids, n, k, n_experts, fn=None):
    rows = gate.shape[0]
    d = ctx.device
    out = d.alloc_buffer(rows * n * 4, mx.DType.F32, [rows, n])
    enc = d.command_encoder()
    # the calling convention of the MoE down projection: n_tokens = rows, top_k = 1
    p = mx.GgmlQuantizedMatmulIdParams(rows, 1, n, k, n_experts, stride, gtype)
    (fn or mx.quantized_matmul_id_swiglu)(enc, ctx.registry, d, ctx.buf(gate, mx.DType.F32), ctx.buf(up, mx.DType.F32),
                                          ctx.buf(w, mx.DType.U8), ctx.buf(ids, mx.DType.U32), out, p)
    enc.commit_and_wait()
    return out.as_slice(np.float32).reshape(rows, n).copy()


# rows <= 16 take the register-level kernel where the weight rows start on 16-byte boundaries (not Q6_K with k = 768:
# 630-byte rows), the others the streaming kernel; both form silu(gate) * up while loading the activations
@pytest.mark.parametrize("tname,rows,n,k", [("Q4_0", 8, 2048, 768), ("Q4_0", 40, 2048, 768), ("Q8_0", 8, 512, 1024), ("Q8_0", 33, 96, 256),
                                            ("Q6_K", 8, 2048, 768), ("Q6_K", 8, 256, 1024), ("Q6_K", 24, 2048, 768), ("Q4_0", 1, 64, 256)])
def test_fused_swiglu_matches_the_oracle_chain(ctx, tname, rows, n, k):
    gtype, otype = TYPES[tname]
    n_experts = 8
    w, stride = stacked(otype, n_experts, n, k)
    gate, up = normal_acts(70, rows, k) * 2.0, normal_acts(71, rows, k)
    ids = np.array([(5 * r + 3) % n_experts for r in range(rows)], np.uint32)
    mx.reset_counters()
    y = run_fused(ctx, gtype, w, stride, gate, up, ids, n, k, n_experts)
    assert mx.kernel_launch_count() == 1                           # no separate SwiGLU launch
    h = orc.silu_mul(gate, up).reshape(rows, k)
    y_ref, ad = orc.qmatmul_id(otype, w, stride, h, ids, 1, n, k, n_experts, nthreads=8)
    assert norm_err(y, y_ref, ad) <= MV_TOL
    # ... and the unfused chain of this library gives the same rows (the same activations, computed by silu_mul)
    d = ctx.device
    act = d.alloc_buffer(rows * k * 4, mx.DType.F32)
    enc = d.command_encoder()
    mx.silu_mul(enc, ctx.registry, d, ctx.buf(gate, mx.DType.F32), ctx.buf(up, mx.DType.F32), act, rows * k)
    enc.commit_and_wait()
    assert np.allclose(act.as_slice(np.float32).reshape(rows, k), h, rtol=2e-6, atol=1e-7)
    y2, _ = ctx.matmul_id(gtype, w, stride, h, ids, 1, n, k, n_experts)
    # (more than 32 rows: the unfused call takes the grouped f16 mat-mat, the fused one stays a mat-vec as upstream's does)
    assert norm_err(y, y2, ad) <= (MV_TOL if rows <= mx.MM_ID_ROUTING_THRESHOLD else MM_TOL)


def test_q4_0_wrapper_and_errors(ctx):
    gtype, otype = TYPES["Q4_0"]
    w, stride = stacked(otype, 4, 64, 256)
    gate, up = normal_acts(1, 4, 256), normal_acts(2, 4, 256)
    ids = np.array([0, 3, 1, 2], np.uint32)
    y = run_fused(ctx, gtype, w, stride, gate, up, ids, 64, 256, 4, fn=mx.quantized_matmul_id_swiglu_q4_0)
    y_ref, ad = orc.qmatmul_id(otype, w, stride, orc.silu_mul(gate, up).reshape(4, 256), ids, 1, 64, 256, 4)
    assert norm_err(y, y_ref, ad) <= MV_TOL
    w8, stride8 = stacked(TYPES["Q8_0"][1], 4, 64, 256)
    with pytest.raises(mx.InvalidArgument, match="expected Q4_0"):
        run_fused(ctx, TYPES["Q8_0"][0], w8, stride8, gate, up, ids, 64, 256, 4, fn=mx.quantized_matmul_id_swiglu_q4_0)
    d = ctx.device
    small = d.alloc_buffer(16, mx.DType.F32)
    p = mx.GgmlQuantizedMatmulIdParams(4, 1, 64, 256, 4, stride, gtype)
    with pytest.raises(mx.InvalidArgument, match="up buffer too small"):
        mx.quantized_matmul_id_swiglu(d.command_encoder(), ctx.registry, d, ctx.buf(gate, mx.DType.F32), small, ctx.buf(w, mx.DType.U8),
                                      ctx.buf(ids, mx.DType.U32), d.alloc_buffer(4 * 64 * 4, mx.DType.F32), p)
    with pytest.raises(mx.InvalidArgument, match="expected Q4_0, Q8_0 or Q6_K"):
        mx.quantized_matmul_id_swiglu(d.command_encoder(), ctx.registry, d, ctx.buf(gate, mx.DType.F32), ctx.buf(up, mx.DType.F32),
                                      ctx.buf(w, mx.DType.U8), ctx.buf(ids, mx.DType.U32), d.alloc_buffer(4 * 64 * 4, mx.DType.F32),
                                      mx.GgmlQuantizedMatmulIdParams(4, 1, 64, 256, 4, stride, mx.GgmlType.Q4_K))


# ---- decode-sized routed mat-vecs: every (token, slot) row is one problem of the batched register-level kernel, and gate and
# ---- up of one layer (same activations and ids, different weights) leave as ONE launch
def test_gate_and_up_share_a_launch_and_bad_ids_give_zeros(ctx):
    gtype, otype = TYPES["Q4_0"]
    n_experts, top_k, n, k = 16, 8, 768, 2048
    wg, stride = stacked(otype, n_experts, n, k, seed=600)
    wu, _ = stacked(otype, n_experts, n, k, seed=700)
    x = normal_acts(9, 1, k)
    ids = np.array([3, 15, 0, 7, 99, 8, 2, 11], np.uint32)          # 99: no such expert
    d = ctx.device
    xb, ib = ctx.buf(x, mx.DType.F32), ctx.buf(ids, mx.DType.U32)
    yg, yu = d.alloc_buffer(top_k * n * 4, mx.DType.F32), d.alloc_buffer(top_k * n * 4, mx.DType.F32)
    p = mx.GgmlQuantizedMatmulIdParams(1, top_k, n, k, n_experts, stride, gtype)
    mx.reset_counters()
    enc = d.command_encoder()
    mx.quantized_matmul_id_ggml(enc, ctx.registry, d, xb, ctx.buf(wg, mx.DType.U8), ib, yg, p)
    mx.quantized_matmul_id_ggml(enc, ctx.registry, d, xb, ctx.buf(wu, mx.DType.U8), ib, yu, p)
    enc.commit_and_wait()
    assert mx.last_kernel_name() == "qmv_mma" and mx.kernel_launch_count() == 1 and mx.dispatch_count() == 2
    good = ids < n_experts
    for w, yb in ((wg, yg), (wu, yu)):
        y = yb.as_slice(np.float32).reshape(top_k, n)
        y_ref, ad = orc.qmatmul_id(otype, w, stride, x, np.where(good, ids, 0).astype(np.uint32), top_k, n, k, n_experts, nthreads=8)
        assert norm_err(y[good], y_ref[good], ad[good]) <= MV_TOL
        assert np.all(y[~good] == 0.0)


# ---- a (token, slot) pair's row does not depend on how many pairs share its launch: the all-to-all MoE layer sends
# ---- each rank a different subset of the pairs and is still bit-identical to the one-GPU layer
@pytest.mark.parametrize("tname,n,k", [("Q4_0", 768, 2048), ("Q8_0", 768, 2048), ("Q6_K", 512, 2048), ("Q4_K", 512, 2048)])
def test_routed_rows_do_not_depend_on_the_launch_composition(ctx, tname, n, k):
    gtype, otype = TYPES[tname] if tname in TYPES else (mx.GgmlType.Q4_K, orc.Q4_K)
    n_experts = 8
    w, stride = stacked(otype, n_experts, n, k, seed=800)
    rows = normal_acts(21, 8, k)                                       # eight pairs, one activation row each (top_k = 1)
    ids = np.array([5, 1, 7, 2, 2, 0, 6, 3], np.uint32)
    whole, _ = ctx.matmul_id(gtype, w, stride, rows, ids, 1, n, k, n_experts)
    assert mx.last_kernel_name() == "qmv_mma"
    for parts in ((3, 5), (1, 7), (2, 2, 4)):
        lo = 0
        for cnt in parts:
            part, _ = ctx.matmul_id(gtype, w, stride, rows[lo:lo + cnt], ids[lo:lo + cnt], 1, n, k, n_experts)
            assert np.array_equal(part.view(np.uint32), whole[lo:lo + cnt].view(np.uint32)), (tname, parts, lo)
            lo += cnt
    # ... nor on whether the eight pairs belong to one token (top_k = 8, the row shared) or to eight
    one_tok, _ = ctx.matmul_id(gtype, w, stride, rows[:1], ids, 8, n, k, n_experts)
    eight, _ = ctx.matmul_id(gtype, w, stride, np.repeat(rows[:1], 8, axis=0), ids, 1, n, k, n_experts)
    assert np.array_equal(one_tok.view(np.uint32), eight.view(np.uint32))
