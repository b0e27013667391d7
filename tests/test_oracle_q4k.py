"""Pins the oracle's Q4_K restatement on the upstream known-answer cases
(tests/test_q4_k_kernels.rs:262-343: scale round trip over all 6-bit pairs, all-zero block, first low nibble,
the dmin offset) and on an independent numpy restatement of src/gguf/mod.rs:582-644."""
import ctypes as C

import numpy as np

from oracle import oracle as orc


def _scale_min(j, scales):
    sc, mn = C.c_uint8(), C.c_uint8()
    s = np.ascontiguousarray(scales, dtype=np.uint8)
    orc.lib().orc_q4k_scale_min(j, s.ctypes.data_as(C.c_void_p), C.byref(sc), C.byref(mn))
    return sc.value, mn.value


def _encode(sc, mn):
    out = np.zeros(12, dtype=np.uint8)
    a, b = np.asarray(sc, np.uint8), np.asarray(mn, np.uint8)
    orc.lib().orc_q4k_encode_scales(a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p))
    return out


def f16_bytes(v):
    return np.array([v], dtype=np.float16).view(np.uint8)


def numpy_dequant_q4_k(data):
    blocks = np.asarray(data, np.uint8).reshape(-1, 144)
    out = np.zeros((blocks.shape[0], 256), dtype=np.float32)
    for bi, blk in enumerate(blocks):
        d = np.float32(blk[0:2].view(np.float16)[0])
        dmin = np.float32(blk[2:4].view(np.float16)[0])
        scales, qs = blk[4:16], blk[16:144]
        for j in range(8):
            if j < 4:
                sc, mn = scales[j] & 63, scales[j + 4] & 63
            else:
                sc = (scales[j + 4] & 0xF) | ((scales[j - 4] >> 6) << 4)
                mn = (scales[j + 4] >> 4) | ((scales[j] >> 6) << 4)
            q = qs[32 * (j // 2):32 * (j // 2) + 32]
            nib = (q & 0xF) if j % 2 == 0 else (q >> 4)
            dj = np.float32(d * np.float32(sc))
            mj = np.float32(dmin * np.float32(mn))
            out[bi, 32 * j:32 * j + 32] = (dj * nib.astype(np.float32)).astype(np.float32) - mj
    return out.reshape(-1)


def test_scale_round_trip_all_6bit_pairs():
    for scp in range(64):
        for mp in range(0, 64, 7):
            enc = _encode([scp] * 8, [mp] * 8)
            for j in range(8):
                assert _scale_min(j, enc) == (scp, mp)
    rng = np.random.default_rng(0)
    for _ in range(200):      # mixed values per sub-block
        sc, mn = rng.integers(0, 64, 8), rng.integers(0, 64, 8)
        enc = _encode(sc, mn)
        assert [_scale_min(j, enc) for j in range(8)] == list(zip(sc.tolist(), mn.tolist()))


def test_known_answer_blocks():
    assert np.all(orc.dequantize(orc.Q4_K, np.zeros(144, np.uint8)) == 0.0)
    blk = np.zeros(144, np.uint8)
    blk[0:2] = f16_bytes(1.0)
    blk[4] = 1
    blk[16] = 0x0F
    out = orc.dequantize(orc.Q4_K, blk)
    assert out[0] == 15.0 and out[32] == 0.0
    blk = np.zeros(144, np.uint8)
    blk[0:2] = f16_bytes(2.0)
    blk[2:4] = f16_bytes(3.0)
    blk[4] = 1
    blk[8] = 1
    blk[16] = 0x0F
    assert orc.dequantize(orc.Q4_K, blk)[0] == 27.0


def test_dequant_matches_numpy_restatement_on_random_blocks():
    rng = np.random.default_rng(3)
    raw = rng.integers(0, 256, size=(64, 144), dtype=np.uint8)
    raw[:, 1] = (raw[:, 1] & 0x83) | 0x20      # finite f16 d and dmin
    raw[:, 3] = (raw[:, 3] & 0x83) | 0x20
    assert np.array_equal(orc.dequantize(orc.Q4_K, raw.reshape(-1)), numpy_dequant_q4_k(raw))


def test_pack_round_trip_and_matvec():
    rng = np.random.default_rng(4)
    v = (rng.standard_normal((8, 512)) * 0.02).astype(np.float32)
    w = orc.quantize(orc.Q4_K, v)
    assert w.size == 8 * 2 * 144
    back = orc.dequantize(orc.Q4_K, w).reshape(v.shape)
    span = v.max() - v.min()
    assert np.max(np.abs(back - v)) <= span / 15.0           # a 4-bit grid over at most the block's range
    x = rng.standard_normal((2, 512)).astype(np.float32)
    y, ad = orc.qmatmul(orc.Q4_K, w, x, 8, 512)
    want = x.astype(np.float64) @ back.astype(np.float64).T
    assert np.max(np.abs(y - want) / ad) < 1e-5
