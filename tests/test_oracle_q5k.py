"""Pins the oracle's Q5_K restatement on the upstream known answers (tests/test_q5_k_dequant.rs:121-262: all-zero
block, zero quants under unit scales, first value with its high bit -> 31, second sub-block sc=2 -> 62, third pair with
the shifted bit selector -> 63, d=2 / dmin=3 -> 59) and on an independent numpy restatement of src/gguf/mod.rs:469-540."""
import numpy as np

from oracle import oracle as orc


def block(d, dmin, scales, qh, qs):
    b = np.zeros(176, np.uint8)
    b[0:2] = np.array([d], np.float16).view(np.uint8)
    b[2:4] = np.array([dmin], np.float16).view(np.uint8)
    b[4:16], b[16:48], b[48:176] = scales, qh, qs
    return b


def numpy_dequant_q5_k(data):
    blocks = np.asarray(data, np.uint8).reshape(-1, 176)
    out = np.zeros((blocks.shape[0], 256), np.float32)
    for bi, blk in enumerate(blocks):
        d = np.float32(blk[0:2].view(np.float16)[0])
        dmin = np.float32(blk[2:4].view(np.float16)[0])
        scales, qh, qs = blk[4:16], blk[16:48], blk[48:176]
        for j in range(8):
            if j < 4:
                sc, mn = scales[j] & 63, scales[j + 4] & 63
            else:
                sc = (scales[j + 4] & 0xF) | ((scales[j - 4] >> 6) << 4)
                mn = (scales[j + 4] >> 4) | ((scales[j] >> 6) << 4)
            ql = qs[32 * (j // 2):32 * (j // 2) + 32]
            low = (ql & 0xF) if j % 2 == 0 else (ql >> 4)
            high = ((qh >> j) & 1).astype(np.uint32) * 16        # pair p = j // 2 uses bits 2p (even j) and 2p + 1 (odd j)
            q = low.astype(np.uint32) + high
            dj = np.float32(d * np.float32(sc))
            mj = np.float32(dmin * np.float32(mn))
            out[bi, 32 * j:32 * j + 32] = (dj * q.astype(np.float32)).astype(np.float32) - mj
    return out.reshape(-1)


def test_upstream_known_answers():
    z12, z32, z128 = np.zeros(12, np.uint8), np.zeros(32, np.uint8), np.zeros(128, np.uint8)
    assert np.all(orc.dequantize(orc.Q5_K, block(0.0, 0.0, z12, z32, z128)) == 0)
    sc = z12.copy()
    sc[0:4] = 1
    assert np.all(orc.dequantize(orc.Q5_K, block(1.0, 0.0, sc, z32, z128)) == 0)
    sc, qs, qh = z12.copy(), z128.copy(), z32.copy()
    sc[0], qs[0], qh[0] = 1, 0x0F, 0x01
    out = orc.dequantize(orc.Q5_K, block(1.0, 0.0, sc, qh, qs))
    assert out[0] == 31.0 and out[1] == 0.0
    sc, qs, qh = z12.copy(), z128.copy(), z32.copy()
    sc[0], sc[1], qs[0], qh[0] = 1, 2, 0xF0, 0x02
    out = orc.dequantize(orc.Q5_K, block(1.0, 0.0, sc, qh, qs))
    assert out[0] == 0.0 and out[32] == 62.0
    sc, qs, qh = z12.copy(), z128.copy(), z32.copy()
    sc[8], qs[64], qh[0] = 3, 0x05, 0x10
    assert orc.dequantize(orc.Q5_K, block(1.0, 0.0, sc, qh, qs))[128] == 63.0
    sc, qs, qh = z12.copy(), z128.copy(), z32.copy()
    sc[0], sc[4], qs[0], qh[0] = 1, 1, 0x0F, 0x01
    assert orc.dequantize(orc.Q5_K, block(2.0, 3.0, sc, qh, qs))[0] == 59.0


def random_q5k_blocks(rng, nblocks):
    raw = rng.integers(0, 256, size=(nblocks, 176), dtype=np.uint8)
    raw[:, 1] = (raw[:, 1] & 0x83) | 0x20        # finite f16 d and dmin in a small range
    raw[:, 3] = (raw[:, 3] & 0x83) | 0x20
    return raw.reshape(-1)


def test_matches_numpy_restatement_of_the_production_dequantizer():
    data = random_q5k_blocks(np.random.default_rng(3), 40)
    assert np.array_equal(orc.dequantize(orc.Q5_K, data), numpy_dequant_q5_k(data))


def test_routed_matvec_uses_the_q5k_blocks():
    rng = np.random.default_rng(4)
    E, n, k, T, top_k = 4, 8, 512, 3, 2
    w = random_q5k_blocks(rng, E * n * (k // 256))
    x = rng.standard_normal((T, k)).astype(np.float32)
    ids = rng.integers(0, E, T * top_k).astype(np.uint32)
    y, ad = orc.qmatmul_id(orc.Q5_K, w, w.size // E, x, ids, top_k, n, k, E)
    wf = numpy_dequant_q5_k(w).reshape(E, n, k)
    for r in range(T * top_k):
        want = np.zeros(n, np.float32)
        for c in range(n):
            acc = np.float32(0.0)
            for kk in range(k):
                acc = np.float32(acc + np.float32(x[r // top_k, kk] * wf[ids[r], c, kk]))
            want[c] = acc
        assert np.array_equal(y[r], want)
