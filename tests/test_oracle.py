"""Pins the CPU oracle (oracle/oracle.c): hand-derived known answers with literal expected
values, an independent numpy restatement of the upstream production dequantizers, and the
upstream test suite's seeded cases.  CPU only."""
import struct

import numpy as np
import pytest

from oracle import oracle as orc
from tests import ref_numpy as rn

Q4_0, Q8_0, Q6_K = orc.Q4_0, orc.Q8_0, orc.Q6_K


def f16_bytes(v: float) -> bytes:
    return struct.pack("<e", v)


# ---------------------------------------------------------------- f16 conversion and LCG

def test_f16_to_f32_all_65536_values():
    L = orc.lib()
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([L.orc_f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])
    assert np.all(np.isnan(got[np.isnan(want)]))


def test_f32_to_f16_round_to_nearest_even():
    L = orc.lib()
    rng = np.random.default_rng(7)
    vals = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(0.02),
        rng.standard_normal(5000).astype(np.float32) * np.float32(1e-6),   # subnormal halves
        rng.standard_normal(5000).astype(np.float32) * np.float32(3e4),    # near overflow
        np.array([0.0, -0.0, 65504.0, 65520.0, 1e9, 5.9604645e-8, 2.9802322e-8, 1.0009766, 1.0004883],
                 dtype=np.float32),
    ])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([L.orc_f32_to_f16(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("seed", [0, 1, 2, 42, 123, 55, 66, 99, 100, 77, 88, 200, 201])
def test_lcg_matches_integer_restatement(seed):
    assert np.array_equal(orc.lcg_f32(seed, 257), rn.lcg_f32(seed, 257))


def test_lcg_known_first_value():
    # one LCG step from seed 42 with arbitrary-precision integers; value = (state >> 33) / 2^32 - 0.5
    state1 = (42 * 6364136223846793005 + 1442695040888963407) % (1 << 64)
    want = np.float32(np.float32(state1 >> 33) / np.float32(4294967296.0) - np.float32(0.5))
    assert orc.lcg_f32(42, 1)[0] == want
    assert -0.5 <= float(want) < 0.5


# ---------------------------------------------------------------- hand-built known-answer blocks

def test_q4_0_known_block():
    # d = 0.5; qs[i] = i | (15-i)<<4  ->  element i = 0.5*(i-8), element 16+i = 0.5*(7-i)
    blk = f16_bytes(0.5) + bytes([(i | ((15 - i) << 4)) for i in range(16)])
    vals = orc.dequantize(Q4_0, np.frombuffer(blk, dtype=np.uint8))
    want = [0.5 * (i - 8) for i in range(16)] + [0.5 * (7 - i) for i in range(16)]
    assert vals.tolist() == want
    y, ad = orc.qmatmul(Q4_0, np.frombuffer(blk, dtype=np.uint8), np.ones((1, 32), np.float32), 1, 32)
    assert y[0, 0] == -8.0          # 0.5 * (sum(i-8) + sum(7-i)) = 0.5 * (-8 - 8)
    assert ad[0, 0] == 64.0         # 0.5 * (2 * (8+7+6+5+4+3+2+1+0+1+2+3+4+5+6+7))


def test_q8_0_known_block():
    # d = 0.25; qs[i] = i-16
    blk = f16_bytes(0.25) + bytes([(i - 16) & 0xFF for i in range(32)])
    w = np.frombuffer(blk, dtype=np.uint8)
    assert orc.dequantize(Q8_0, w).tolist() == [0.25 * (i - 16) for i in range(32)]
    y, _ = orc.qmatmul(Q8_0, w, np.ones((1, 32), np.float32), 1, 32)
    assert y[0, 0] == -4.0          # 0.25 * (496 - 512)
    y, _ = orc.qmatmul(Q8_0, w, np.arange(32, dtype=np.float32)[None], 1, 32)
    assert y[0, 0] == 620.0         # 0.25 * (sum i^2 - 16 sum i) = 0.25 * (10416 - 7936)


def test_q6_k_known_block():
    # d = 1; scales[s] = s+1; every ql byte 0x21; every qh byte 0xE4 (2-bit fields 0,1,2,3)
    # -> q1 = 1+0-32 = -31, q2 = 1+16-32 = -15, q3 = 2+32-32 = 2, q4 = 2+48-32 = 18
    blk = bytes([0x21] * 128) + bytes([0xE4] * 64) + bytes(range(1, 17)) + f16_bytes(1.0)
    assert len(blk) == 210
    w = np.frombuffer(blk, dtype=np.uint8)
    v = orc.dequantize(Q6_K, w)
    assert v[0] == -31.0 and v[16] == -62.0 and v[32] == -45.0 and v[64] == 10.0 and v[96] == 126.0
    assert v[128] == -279.0 and v[255] == 288.0
    y, _ = orc.qmatmul(Q6_K, w, np.ones((1, 256), np.float32), 1, 256)
    assert y[0, 0] == -3648.0       # 16*(60+34) + 16*(-148-174)


# ---------------------------------------------------------------- the two upstream formulations agree

@pytest.mark.parametrize("t", [Q4_0, Q8_0, Q6_K])
def test_random_bytes_dequant_matches_production_restatement(t):
    rng = np.random.default_rng(t)
    nb = 64
    raw = rng.integers(0, 256, size=nb * orc.BLOCK_BYTES[t], dtype=np.uint8)
    # keep the f16 scales finite
    blk = raw.reshape(nb, -1)
    dpos = 208 if t == Q6_K else 0
    blk[:, dpos + 1] &= 0x3B
    a = orc.dequantize(t, raw)
    b = rn.DEQUANT[t](raw)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("t,seed_w,seed_x,n,k", [
    (Q4_0, 42, 123, 32, 256), (Q8_0, 55, 66, 32, 256), (Q6_K, 99, 100, 16, 256),
])
def test_upstream_seeded_cases_against_numpy(t, seed_w, seed_x, n, k):
    """tests/test_quantized_matmul_ggml.rs:585-586, :694-695, :797-798 (random cases)."""
    wf = orc.lcg_f32(seed_w, n * k)
    x = orc.lcg_f32(seed_x, k)
    wq = orc.quantize(t, wf)
    deq = rn.DEQUANT[t](wq).reshape(n, k)
    # sequential f32 accumulation, as cpu_matvec does
    want = np.zeros(n, dtype=np.float32)
    for ki in range(k):
        want = (want + x[ki] * deq[:, ki]).astype(np.float32)
    y, ad = orc.qmatmul(t, wq, x[None], n, k)
    assert np.array_equal(y[0].view(np.uint32), want.view(np.uint32))
    assert np.allclose(ad[0], np.abs(deq.astype(np.float64) * x.astype(np.float64)).sum(1), rtol=1e-6)
    # quantisation error is bounded by half a step per element
    err = np.abs(deq.reshape(-1) - wf)
    step = {Q4_0: 1 / 7, Q8_0: 1 / 127, Q6_K: 1 / 31}[t]
    assert err.max() <= 0.5 * step * 0.5 * 1.02 + 1e-3


@pytest.mark.parametrize("t", [Q4_0, Q8_0, Q6_K])
def test_known_value_ramps(t):
    """tests/test_quantized_matmul_ggml.rs:539-577, :651-686, :759-789: ramp weights, x = 1."""
    if t == Q4_0:
        n, k = 8, 32
        wf = np.array([[(r * 0.1) * ((c - 16.0) / 16.0) for c in range(k)] for r in range(n)], np.float32)
    elif t == Q8_0:
        n, k = 8, 32
        wf = np.array([[(r + 1.0) * (c - 16.0) / 32.0 for c in range(k)] for r in range(n)], np.float32)
    else:
        n, k = 2, 256
        wf = np.array([[(r + 1.0) * (c - 128.0) / 256.0 for c in range(k)] for r in range(n)], np.float32)
    wq = orc.quantize(t, wf)
    y, _ = orc.qmatmul(t, wq, np.ones((1, k), np.float32), n, k)
    deq = orc.dequantize(t, wq).reshape(n, k)
    # the ramp sums to -(row scale)/2 * (one step); quantisation keeps it within a few steps
    exact = wf.astype(np.float64).sum(1)
    assert np.all(np.abs(y[0] - exact) <= np.abs(wf).max(1) * 0.6 + 1e-6)
    assert np.allclose(y[0], deq.sum(1), atol=1e-4)


def test_q4_0_ggml_rule():
    rng = np.random.default_rng(0)
    v = (rng.standard_normal(32 * 50) * 0.02).astype(np.float32)
    q = orc.quantize(Q4_0, v, rule="ggml").reshape(-1, 18)
    d = q[:, :2].copy().view(np.float16).astype(np.float32)[:, 0]
    vb = v.reshape(-1, 32)
    imax = np.abs(vb).argmax(1)
    mx = vb[np.arange(vb.shape[0]), imax]
    assert np.array_equal(d, (mx / np.float32(-8.0)).astype(np.float16).astype(np.float32))
    # the extreme element quantises to nibble 0 (value -8)
    deq = orc.dequantize(Q4_0, q).reshape(-1, 32)
    assert np.allclose(deq[np.arange(vb.shape[0]), imax], mx, rtol=2e-3)
    assert np.abs(deq - vb).max() <= np.abs(d).max() * 0.5 * 1.01 + np.abs(d).max()  # clamp at +7 costs one step


# ---------------------------------------------------------------- f16-operand variant and threading

def test_f16_operand_variant_and_threads():
    rng = np.random.default_rng(3)
    n, k, m = 24, 512, 3
    wq = orc.quantize(Q6_K, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    x = rng.standard_normal((m, k)).astype(np.float32)
    y1, ad1 = orc.qmatmul(Q6_K, wq, x, n, k)
    y8, ad8 = orc.qmatmul(Q6_K, wq, x, n, k, nthreads=8)
    assert np.array_equal(y1, y8) and np.array_equal(ad1, ad8)
    yh, _ = orc.qmatmul(Q6_K, wq, x, n, k, f16_operands=True)
    deq = orc.dequantize(Q6_K, wq).reshape(n, k).astype(np.float16).astype(np.float32)
    xh = x.astype(np.float16).astype(np.float32)
    want = np.zeros((m, n), np.float32)
    for ki in range(k):
        want = (want + xh[:, ki:ki + 1] * deq[None, :, ki]).astype(np.float32)
    assert np.array_equal(yh, want)
    assert np.max(np.abs(yh - y1) / ad1) < 2e-3


# ---------------------------------------------------------------- routing

def test_map0_matches_scan_order_reference():
    """tests/test_quantized_matmul_id_mm.rs:340-449 (ids = (t*17 + s*13 + 7) % E)."""
    n_tokens, n_experts, top_k = 16, 8, 8
    ids = np.array([(t * 17 + s * 13 + 7) % n_experts for t in range(n_tokens) for s in range(top_k)], np.uint32)
    htpe, hids = orc.moe_map0(ids, n_tokens, top_k, n_experts)
    counts, lists = rn.bucket_scan_order(ids, n_tokens, top_k, n_experts)
    assert htpe.tolist() == counts
    for e in range(n_experts):
        assert hids[e, :counts[e]].tolist() == lists[e]


def test_map0_sparse_and_top1():
    n_tokens, n_experts = 37, 128
    ids = np.array([(t * 5 + 3) % 7 for t in range(n_tokens)], np.uint32)  # only experts 0..6 are used
    htpe, hids = orc.moe_map0(ids, n_tokens, 1, n_experts)
    counts, lists = rn.bucket_scan_order(ids, n_tokens, 1, n_experts)
    assert htpe.tolist() == counts and sum(counts) == n_tokens and all(c == 0 for c in counts[7:])
    for e in range(7):
        assert hids[e, :counts[e]].tolist() == lists[e]


def test_softmax_topk_properties():
    rng = np.random.default_rng(0)
    lg = rng.standard_normal((33, 128)).astype(np.float32)
    ids, w = orc.moe_softmax_topk(lg, 8)
    order = np.argsort(-lg, axis=1, kind="stable")[:, :8]
    assert np.array_equal(ids, order.astype(np.uint32))
    assert np.allclose(w.sum(1), 1.0, atol=1e-6)
    p = np.exp(lg - lg.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    sel = np.take_along_axis(p, order, 1)
    assert np.allclose(w, sel / sel.sum(1, keepdims=True), rtol=1e-5)
    # ties keep the lower expert index first
    tie = np.zeros((1, 16), np.float32)
    ids, w = orc.moe_softmax_topk(tie, 4)
    assert ids.tolist() == [[0, 1, 2, 3]] and np.allclose(w, 0.25)


def test_qmatmul_id_equals_per_expert_matvec():
    """tests/test_quantized_matmul_id_ggml.rs:328-495 (ids = (t*3 + s*7 + 1) % E)."""
    n_tokens, n_experts, top_k, n, k = 4, 8, 2, 64, 128
    x = orc.lcg_f32(42, n_tokens * k).reshape(n_tokens, k)
    ws = [orc.quantize(Q8_0, orc.lcg_f32(100 + e, n * k)) for e in range(n_experts)]
    stacked = np.concatenate(ws)
    ids = np.array([(t * 3 + s * 7 + 1) % n_experts for t in range(n_tokens) for s in range(top_k)], np.uint32)
    y, _ = orc.qmatmul_id(Q8_0, stacked, ws[0].size, x, ids, top_k, n, k, n_experts)
    for r in range(n_tokens * top_k):
        yr, _ = orc.qmatmul(Q8_0, ws[ids[r]], x[r // top_k][None], n, k)
        assert np.array_equal(y[r], yr[0])


def test_silu_and_weighted_reduce():
    rng = np.random.default_rng(1)
    g = rng.standard_normal(100).astype(np.float32)
    u = rng.standard_normal(100).astype(np.float32)
    assert np.allclose(orc.silu_mul(g, u), g / (1 + np.exp(-g)) * u, rtol=1e-6)
    y = rng.standard_normal((6, 10)).astype(np.float32)
    w = rng.random((3, 2)).astype(np.float32)
    out = orc.moe_weighted_reduce(y, w, 3, 2, 10)
    assert np.allclose(out, (y.reshape(3, 2, 10) * w[:, :, None]).sum(1), rtol=1e-6)
