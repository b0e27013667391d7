/*
 * CPU oracle for the GGML block-quantized matmul path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the scalar reference the upstream project uses
 * to judge its GPU kernels: dequantize the GGML blocks to f32, then take a
 * sequential f32 dot product.  It is compiled by oracle/Makefile into
 * oracle/liboracle.so and loaded by the tests, by the smoke check and by the
 * benchmark's CPU-baseline leg.  Nothing in the product path may call it.
 *
 * Parity pin: the upstream repository ships no golden vectors and no
 * known-answer files for this path (its tests compare a GPU run with this same
 * scalar path), and its Rust sources cannot be compiled where this oracle is
 * built.  The oracle is therefore pinned by (1) hand-derived known-answer blocks
 * whose expected values are literal numbers in tests/test_oracle.py, (2) an
 * independent numpy restatement of the upstream production dequantizers
 * (src/gguf/mod.rs) that must agree bit for bit with this file, which follows
 * the upstream test-suite dequantizers, and (3) the vectors under tests/golden/,
 * which this oracle produced itself (tests/golden/make_golden.py): they freeze
 * its answers against later edits, they do not tie it to upstream.  Against
 * outputs of the upstream code itself parity is unpinned.
 *
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared (no FMA contraction, so the
 * f32 accumulation order and rounding are those of the upstream scalar loop).
 *
 * Upstream sources followed (paths inside the upstream repository):
 *   tests/test_quantized_matmul_ggml.rs:17-28    pseudo_random_f32 (LCG)
 *   tests/test_quantized_matmul_ggml.rs:37-60    pack_q4_0 (test quantizer)
 *   tests/test_quantized_matmul_ggml.rs:63-94    dequant_q4_0
 *   tests/test_quantized_matmul_ggml.rs:99-116   pack_q8_0
 *   tests/test_quantized_matmul_ggml.rs:119-132  dequant_q8_0
 *   tests/test_quantized_matmul_ggml.rs:137-324  pack_q6_k
 *   tests/test_quantized_matmul_ggml.rs:327-407  dequant_q6_k
 *   tests/test_quantized_matmul_ggml.rs:414-426  cpu_matvec
 *   src/gguf/mod.rs:355-388, 395-425, 656-709    production dequantizers
 *   src/shaders/quantized_matmul_id_mm.metal:242-283  map0 bucketing
 *   src/shaders/moe_softmax_topk.metal:27-148    router softmax + top-k
 *   src/gguf/mod.rs:440-452, 582-644             Q4_K scale/min unpacking and dequantize
 *   src/gguf/mod.rs:469-540                      Q5_K dequantize (known answers: tests/test_q5_k_dequant.rs:121-262)
 *   tests/test_q4_k_kernels.rs:58-76, 108-180    Q4_K scale packing and the test packer
 *   src/shaders/moe_weighted_reduce.metal:33-66  weighted combine
 *   src/shaders/silu_mul.metal:17-30             SwiGLU
 *   src/shaders/quantized_matmul_mm_tensor.metal:92-158, 280-287  f16 operand rounding
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK4_0 32
#define QK8_0 32
#define QK_K 256
#define BYTES_Q4_0 18
#define BYTES_Q8_0 34
#define BYTES_Q6_K 210
#define BYTES_Q4_K 144
#define BYTES_Q5_K 176

/* ggml_type codes shared with include/mlxn_b200.h */
enum { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q8_0 = 3, T_Q4_K = 4, T_Q5_K = 5, T_Q6_K = 6, T_I16 = 7 };

/* ------------------------------------------------------------------ f16 <-> f32 */

/* IEEE binary16 -> binary32, exact (what half::f16::to_f32 does). */
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* binary32 -> binary16, round to nearest even (what half::f16::from_f32 does). */
uint16_t orc_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 255) return (uint16_t)(sign | 0x7C00u | (man ? (0x200u | (man >> 13)) : 0));
    int e = (int)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        int shift = 14 - e; /* 14..24 */
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half_man = man >> 13;
    uint32_t rem = man & 0x1FFFu;
    uint16_t out = (uint16_t)(sign | ((uint32_t)e << 10) | half_man);
    if (rem > 0x1000u || (rem == 0x1000u && (half_man & 1))) out++; /* carry may roll into exponent: correct */
    return out;
}

static inline uint16_t rd_u16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ------------------------------------------------------------------ LCG */

/* tests/test_quantized_matmul_ggml.rs:17-28 */
void orc_lcg_f32(uint64_t seed, size_t n, float *out) {
    uint64_t state = seed;
    for (size_t i = 0; i < n; i++) {
        state = state * 6364136223846793005ULL + 1442695040888963407ULL;
        out[i] = ((float)(state >> 33)) / ((float)UINT32_MAX) - 0.5f;
    }
}

/* ------------------------------------------------------------------ dequantizers */

/* tests/test_quantized_matmul_ggml.rs:63-94 (net effect after its reordering pass);
 * element-for-element equal to src/gguf/mod.rs:355-388. */
void orc_dequant_q4_0(const uint8_t *data, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = data + b * BYTES_Q4_0;
        float d = orc_f16_to_f32(rd_u16(blk));
        const uint8_t *qs = blk + 2;
        float *o = out + b * QK4_0;
        for (int i = 0; i < 16; i++) {
            float lo = (float)(qs[i] & 0x0F);
            float hi = (float)(qs[i] >> 4);
            o[i] = d * (lo - 8.0f);
            o[i + 16] = d * (hi - 8.0f);
        }
    }
}

/* tests/test_quantized_matmul_ggml.rs:119-132; src/gguf/mod.rs:395-425 */
void orc_dequant_q8_0(const uint8_t *data, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = data + b * BYTES_Q8_0;
        float d = orc_f16_to_f32(rd_u16(blk));
        float *o = out + b * QK8_0;
        for (int i = 0; i < 32; i++) o[i] = d * (float)(int8_t)blk[2 + i];
    }
}

/* tests/test_quantized_matmul_ggml.rs:327-407; src/gguf/mod.rs:656-709.
 * Value = (d * scale) * q, evaluated left to right in f32. */
void orc_dequant_q6_k(const uint8_t *data, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = data + b * BYTES_Q6_K;
        const uint8_t *ql = blk;
        const uint8_t *qh = blk + 128;
        const int8_t *sc = (const int8_t *)(blk + 192);
        float d = orc_f16_to_f32(rd_u16(blk + 208));
        float *o = out + b * QK_K;
        for (int half = 0; half < 2; half++) {
            const uint8_t *l = ql + 64 * half;
            const uint8_t *h = qh + 32 * half;
            const int8_t *s = sc + 8 * half;
            float *y = o + 128 * half;
            for (int i = 0; i < 32; i++) {
                int is = i / 16;
                int q1 = (int)((l[i] & 0x0F) | ((h[i] & 0x03) << 4)) - 32;
                int q2 = (int)((l[i + 32] & 0x0F) | (((h[i] >> 2) & 0x03) << 4)) - 32;
                int q3 = (int)((l[i] >> 4) | (((h[i] >> 4) & 0x03) << 4)) - 32;
                int q4 = (int)((l[i + 32] >> 4) | (((h[i] >> 6) & 0x03) << 4)) - 32;
                y[i] = d * (float)s[is] * (float)q1;
                y[i + 32] = d * (float)s[is + 2] * (float)q2;
                y[i + 64] = d * (float)s[is + 4] * (float)q3;
                y[i + 96] = d * (float)s[is + 6] * (float)q4;
            }
        }
    }
}

/* src/gguf/mod.rs:440-452: the 6-bit (scale, min) pair of sub-block j from the 12 packed bytes. */
void orc_q4k_scale_min(int j, const uint8_t *scales, uint8_t *sc, uint8_t *mn) {
    if (j < 4) {
        *sc = scales[j] & 63;
        *mn = scales[j + 4] & 63;
    } else {
        *sc = (uint8_t)((scales[j + 4] & 0x0F) | ((scales[j - 4] >> 6) << 4));
        *mn = (uint8_t)((scales[j + 4] >> 4) | ((scales[j] >> 6) << 4));
    }
}

/* src/gguf/mod.rs:582-644; tests/test_q4_k_kernels.rs:206-233.  Block: f16 d, f16 dmin, scales[12], qs[128].
 * Eight sub-blocks of 32; bytes [32p, 32p+32) of qs hold sub-block 2p in the low nibbles and 2p+1 in the
 * high ones.  Value = (d * sc) * q - (dmin * m), each product and the difference rounded in f32. */
void orc_dequant_q4_k(const uint8_t *data, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = data + b * BYTES_Q4_K;
        const float d = orc_f16_to_f32(rd_u16(blk));
        const float dmin = orc_f16_to_f32(rd_u16(blk + 2));
        const uint8_t *scales = blk + 4, *qs = blk + 16;
        float *o = out + b * QK_K;
        for (int p = 0; p < 4; p++) {
            uint8_t sc1, m1, sc2, m2;
            orc_q4k_scale_min(2 * p, scales, &sc1, &m1);
            orc_q4k_scale_min(2 * p + 1, scales, &sc2, &m2);
            const float d1 = d * (float)sc1, min1 = dmin * (float)m1;
            const float d2 = d * (float)sc2, min2 = dmin * (float)m2;
            for (int l = 0; l < 32; l++) {
                volatile float a = d1 * (float)(qs[32 * p + l] & 0x0F);   /* no fused multiply-subtract */
                volatile float c = d2 * (float)(qs[32 * p + l] >> 4);
                o[64 * p + l] = a - min1;
                o[64 * p + 32 + l] = c - min2;
            }
        }
    }
}

/* src/gguf/mod.rs:469-540 (tests/test_q5_k_dequant.rs:55-98 holds the same formula as the specification).
 * Block: f16 d, f16 dmin, scales[12] (as Q4_K), qh[32], qs[128].  Pair p of sub-blocks: bytes [32p, 32p+32) of qs,
 * low nibbles + bit 2p of qh[l] -> sub-block 2p, high nibbles + bit 2p+1 -> sub-block 2p+1;
 * value = (d * sc) * q - (dmin * m), q = nibble + 16 * bit, each product and the difference rounded in f32. */
void orc_dequant_q5_k(const uint8_t *data, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = data + b * BYTES_Q5_K;
        const float d = orc_f16_to_f32(rd_u16(blk));
        const float dmin = orc_f16_to_f32(rd_u16(blk + 2));
        const uint8_t *scales = blk + 4, *qh = blk + 16, *qs = blk + 48;
        float *o = out + b * QK_K;
        for (int p = 0; p < 4; p++) {
            uint8_t sc1, m1, sc2, m2;
            orc_q4k_scale_min(2 * p, scales, &sc1, &m1);
            orc_q4k_scale_min(2 * p + 1, scales, &sc2, &m2);
            const float d1 = d * (float)sc1, min1 = dmin * (float)m1;
            const float d2 = d * (float)sc2, min2 = dmin * (float)m2;
            for (int l = 0; l < 32; l++) {
                const unsigned q1 = (qs[32 * p + l] & 0x0Fu) + (((qh[l] >> (2 * p)) & 1u) ? 16u : 0u);
                const unsigned q2 = (qs[32 * p + l] >> 4) + (((qh[l] >> (2 * p + 1)) & 1u) ? 16u : 0u);
                volatile float a = d1 * (float)q1;   /* no fused multiply-subtract */
                volatile float c = d2 * (float)q2;
                o[64 * p + l] = a - min1;
                o[64 * p + 32 + l] = c - min2;
            }
        }
    }
}

static int type_qk(int t) { return (t == T_Q6_K || t == T_Q4_K || t == T_Q5_K) ? QK_K : 32; }
static int type_bytes(int t) {
    return t == T_Q4_0 ? BYTES_Q4_0 : t == T_Q8_0 ? BYTES_Q8_0 : t == T_Q4_K ? BYTES_Q4_K : t == T_Q5_K ? BYTES_Q5_K : BYTES_Q6_K;
}

int orc_dequant(int ggml_type, const uint8_t *data, size_t nblocks, float *out) {
    switch (ggml_type) {
    case T_Q4_0: orc_dequant_q4_0(data, nblocks, out); return 0;
    case T_Q8_0: orc_dequant_q8_0(data, nblocks, out); return 0;
    case T_Q6_K: orc_dequant_q6_k(data, nblocks, out); return 0;
    case T_Q4_K: orc_dequant_q4_k(data, nblocks, out); return 0;
    case T_Q5_K: orc_dequant_q5_k(data, nblocks, out); return 0;
    default: return -1;
    }
}

/* ------------------------------------------------------------------ quantizers (test data only) */

/* tests/test_quantized_matmul_ggml.rs:37-60: d = amax/7, q = round(x/d + 8) in [0,15]. */
void orc_pack_q4_0_test(const float *v, size_t n, uint8_t *out) {
    for (size_t b = 0; b < n / 32; b++) {
        const float *x = v + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));
        float d = amax / 7.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        uint16_t dh = orc_f32_to_f16(d);
        uint8_t *o = out + b * BYTES_Q4_0;
        o[0] = (uint8_t)(dh & 0xFF);
        o[1] = (uint8_t)(dh >> 8);
        for (int i = 0; i < 16; i++) {
            float a = fminf(fmaxf(roundf(x[i] * id + 8.0f), 0.0f), 15.0f);
            float c = fminf(fmaxf(roundf(x[i + 16] * id + 8.0f), 0.0f), 15.0f);
            o[2 + i] = (uint8_t)((uint8_t)a | ((uint8_t)c << 4));
        }
    }
}

/* The GGML Q4_0 rule: the element of largest magnitude, with its sign, maps to -8:
 * d = that element / -8; q = min(15, trunc(x/d + 8.5)). */
void orc_pack_q4_0_ggml(const float *v, size_t n, uint8_t *out) {
    for (size_t b = 0; b < n / 32; b++) {
        const float *x = v + b * 32;
        float amax = 0.0f, mx = 0.0f;
        for (int i = 0; i < 32; i++) {
            if (fabsf(x[i]) > amax) {
                amax = fabsf(x[i]);
                mx = x[i];
            }
        }
        float d = mx / -8.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        uint16_t dh = orc_f32_to_f16(d);
        uint8_t *o = out + b * BYTES_Q4_0;
        o[0] = (uint8_t)(dh & 0xFF);
        o[1] = (uint8_t)(dh >> 8);
        for (int i = 0; i < 16; i++) {
            int a = (int)(x[i] * id + 8.5f);
            int c = (int)(x[i + 16] * id + 8.5f);
            if (a > 15) a = 15;
            if (c > 15) c = 15;
            if (a < 0) a = 0;
            if (c < 0) c = 0;
            o[2 + i] = (uint8_t)(a | (c << 4));
        }
    }
}

/* tests/test_quantized_matmul_ggml.rs:99-116: d = amax/127, q = round(x/d).  GGML's Q8_0 rule is the same. */
void orc_pack_q8_0(const float *v, size_t n, uint8_t *out) {
    for (size_t b = 0; b < n / 32; b++) {
        const float *x = v + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));
        float d = amax / 127.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        uint16_t dh = orc_f32_to_f16(d);
        uint8_t *o = out + b * BYTES_Q8_0;
        o[0] = (uint8_t)(dh & 0xFF);
        o[1] = (uint8_t)(dh >> 8);
        for (int i = 0; i < 32; i++) {
            float q = fminf(fmaxf(roundf(x[i] * id), -128.0f), 127.0f);
            o[2 + i] = (uint8_t)(int8_t)q;
        }
    }
}

/* tests/test_quantized_matmul_ggml.rs:137-324: 16 sub-blocks of 16, int8 sub-scales,
 * d = max sub-block amax / (32*127), 6-bit quants with zero point 32. */
void orc_pack_q6_k(const float *v, size_t n, uint8_t *out) {
    for (size_t b = 0; b < n / 256; b++) {
        const float *x = v + b * 256;
        float sub_amax[16];
        float max_scale = 0.0f;
        for (int s = 0; s < 16; s++) {
            float a = 0.0f;
            for (int i = 0; i < 16; i++) a = fmaxf(a, fabsf(x[s * 16 + i]));
            sub_amax[s] = a;
            if (a > max_scale) max_scale = a;
        }
        float d = max_scale / (32.0f * 127.0f);
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        int8_t isc[16];
        for (int s = 0; s < 16; s++) {
            if (sub_amax[s] != 0.0f) {
                float r = roundf(sub_amax[s] * id / 32.0f);
                isc[s] = (int8_t)fminf(fmaxf(r, -128.0f), 127.0f);
            } else {
                isc[s] = 0;
            }
        }
        uint8_t q6[256];
        for (int s = 0; s < 16; s++) {
            float sub_d = d * (float)isc[s];
            float sub_id = sub_d != 0.0f ? 1.0f / sub_d : 0.0f;
            for (int i = 0; i < 16; i++) {
                float q = fminf(fmaxf(roundf(x[s * 16 + i] * sub_id + 32.0f), 0.0f), 63.0f);
                q6[s * 16 + i] = (uint8_t)q;
            }
        }
        uint8_t *o = out + b * BYTES_Q6_K;
        uint8_t *ql = o, *qh = o + 128;
        for (int half = 0; half < 2; half++) {
            for (int l = 0; l < 32; l++) {
                uint8_t v0 = q6[128 * half + l], v1 = q6[128 * half + l + 32];
                uint8_t v2 = q6[128 * half + l + 64], v3 = q6[128 * half + l + 96];
                ql[64 * half + l] = (uint8_t)((v0 & 0x0F) | ((v2 & 0x0F) << 4));
                ql[64 * half + l + 32] = (uint8_t)((v1 & 0x0F) | ((v3 & 0x0F) << 4));
                qh[32 * half + l] = (uint8_t)(((v0 >> 4) & 3) | (((v1 >> 4) & 3) << 2) |
                                              (((v2 >> 4) & 3) << 4) | (((v3 >> 4) & 3) << 6));
            }
        }
        for (int s = 0; s < 16; s++) o[192 + s] = (uint8_t)isc[s];
        uint16_t dh = orc_f32_to_f16(d);
        o[208] = (uint8_t)(dh & 0xFF);
        o[209] = (uint8_t)(dh >> 8);
    }
}

/* tests/test_q4_k_kernels.rs:58-76: packs eight 6-bit scales and mins into 12 bytes. */
void orc_q4k_encode_scales(const uint8_t *sc, const uint8_t *mn, uint8_t *s) {
    memset(s, 0, 12);
    for (int j = 0; j < 4; j++) {
        s[j] = sc[j] & 63;
        s[j + 4] = mn[j] & 63;
    }
    for (int j = 4; j < 8; j++) {
        s[j + 4] = (uint8_t)((sc[j] & 0x0F) | ((mn[j] & 0x0F) << 4));
        s[j - 4] |= (uint8_t)((sc[j] >> 4) << 6);
        s[j] |= (uint8_t)((mn[j] >> 4) << 6);
    }
}

static float clampf(float v, float lo, float hi) { return v < lo ? lo : v > hi ? hi : v; }

/* tests/test_q4_k_kernels.rs:108-180 (the upstream test packer, a uniform per-sub-block quantizer):
 * shift = -min(values) if negative; d = max(values + shift) / (15*63) (1 if that max is 0); dmin = shift / 63
 * (1 if shift is 0); per sub-block sc = round(max(sub + shift) / 15 / d), m = round(shift / dmin), both
 * clamped to 0..63; q = round((v + dmin*m) / (d*sc)) clamped to 0..15. */
void orc_pack_q4_k(const float *v, size_t n, uint8_t *out) {
    for (size_t b = 0; b < n / 256; b++) {
        const float *x = v + b * 256;
        float gmin = 3.402823466e+38f;
        for (int i = 0; i < 256; i++) gmin = fminf(gmin, x[i]);
        const float shift = gmin < 0.0f ? -gmin : 0.0f;
        float gmax = 0.0f;
        for (int i = 0; i < 256; i++) gmax = fmaxf(gmax, x[i] + shift);
        const float d = gmax > 0.0f ? gmax / (15.0f * 63.0f) : 1.0f;
        const float dmin = shift > 0.0f ? shift / 63.0f : 1.0f;
        const float id_d = 1.0f / d, id_dmin = 1.0f / dmin;
        uint8_t sc[8], mn[8];
        for (int s = 0; s < 8; s++) {
            float smax = 0.0f;
            for (int i = 0; i < 32; i++) smax = fmaxf(smax, x[32 * s + i] + shift);
            sc[s] = (uint8_t)clampf(roundf((smax / 15.0f) * id_d), 0.0f, 63.0f);
            mn[s] = (uint8_t)clampf(roundf(shift * id_dmin), 0.0f, 63.0f);
        }
        uint8_t q4[256];
        for (int s = 0; s < 8; s++) {
            const float sub_scale = d * (float)sc[s], sub_min = dmin * (float)mn[s];
            const float inv = sub_scale != 0.0f ? 1.0f / sub_scale : 0.0f;
            for (int i = 0; i < 32; i++)
                q4[32 * s + i] = (uint8_t)clampf(roundf((x[32 * s + i] + sub_min) * inv), 0.0f, 15.0f);
        }
        uint8_t *o = out + b * BYTES_Q4_K;
        const uint16_t dh = orc_f32_to_f16(d), mh = orc_f32_to_f16(dmin);
        o[0] = (uint8_t)(dh & 0xFF);
        o[1] = (uint8_t)(dh >> 8);
        o[2] = (uint8_t)(mh & 0xFF);
        o[3] = (uint8_t)(mh >> 8);
        orc_q4k_encode_scales(sc, mn, o + 4);
        for (int p = 0; p < 4; p++)
            for (int l = 0; l < 32; l++)
                o[16 + 32 * p + l] = (uint8_t)((q4[64 * p + l] & 0x0F) | ((q4[64 * p + 32 + l] & 0x0F) << 4));
    }
}

/* quantizer: 0 = upstream test quantizer, 1 = GGML rule (differs for Q4_0 only). */
int orc_quantize(int ggml_type, int rule, const float *v, size_t n, uint8_t *out) {
    switch (ggml_type) {
    case T_Q4_0:
        if (rule) orc_pack_q4_0_ggml(v, n, out); else orc_pack_q4_0_test(v, n, out);
        return 0;
    case T_Q8_0: orc_pack_q8_0(v, n, out); return 0;
    case T_Q6_K: orc_pack_q6_k(v, n, out); return 0;
    case T_Q4_K: orc_pack_q4_k(v, n, out); return 0;
    default: return -1;
    }
}

/* ------------------------------------------------------------------ matmul */

/* tests/test_quantized_matmul_ggml.rs:414-426 applied to one dequantized weight row:
 * acc += x[ki] * w[ki], ki ascending, f32.  absdot (may be NULL) receives sum |w*x| in f64,
 * the normaliser of the parity bound. */
static void row_dots(const float *wrow, const float *x, int m, size_t k, size_t n, size_t col,
                     float *y, double *absdot, int f16_operands) {
    for (int r = 0; r < m; r++) {
        const float *xr = x + (size_t)r * k;
        float acc = 0.0f;
        double a = 0.0;
        if (!f16_operands) {
            for (size_t ki = 0; ki < k; ki++) {
                float p = xr[ki] * wrow[ki];
                acc += p;
                a += fabs((double)p);
            }
        } else {
            for (size_t ki = 0; ki < k; ki++) {
                float p = orc_f16_to_f32(orc_f32_to_f16(xr[ki])) * wrow[ki];
                acc += p;
                a += fabs((double)p);
            }
        }
        y[(size_t)r * n + col] = acc;
        if (absdot) absdot[(size_t)r * n + col] = a;
    }
}

typedef struct {
    int ggml_type;
    const uint8_t *w;
    const float *x;
    int m;
    size_t n, k;
    size_t row0, row1;
    float *y;
    double *absdot;
    int f16_operands;
} mm_job;

static void *mm_worker(void *arg) {
    mm_job *j = (mm_job *)arg;
    size_t nb = j->k / (size_t)type_qk(j->ggml_type);
    size_t row_bytes = nb * (size_t)type_bytes(j->ggml_type);
    float *wrow = (float *)malloc(j->k * sizeof(float));
    for (size_t col = j->row0; col < j->row1; col++) {
        orc_dequant(j->ggml_type, j->w + col * row_bytes, nb, wrow);
        if (j->f16_operands)
            for (size_t ki = 0; ki < j->k; ki++) wrow[ki] = orc_f16_to_f32(orc_f32_to_f16(wrow[ki]));
        row_dots(wrow, j->x, j->m, j->k, j->n, col, j->y, j->absdot, j->f16_operands);
    }
    free(wrow);
    return NULL;
}

/* y[m,n] = x[m,k] * dequant(W[n,k])^T over weight rows [row0,row1), nthreads host threads.
 * f16_operands = 1 rounds both operands to binary16 first (the upstream tensor mat-mat
 * staging, quantized_matmul_mm_tensor.metal:92-158 and :280-287) and still accumulates in f32. */
int orc_qmatmul(int ggml_type, const uint8_t *w, const float *x, int m, size_t n, size_t k,
                size_t row0, size_t row1, float *y, double *absdot, int f16_operands, int nthreads) {
    if (ggml_type != T_Q4_0 && ggml_type != T_Q8_0 && ggml_type != T_Q6_K && ggml_type != T_Q4_K && ggml_type != T_Q5_K) return -1;
    if (k % (size_t)type_qk(ggml_type)) return -2;
    if (nthreads < 1) nthreads = 1;
    if (nthreads > 256) nthreads = 256;
    size_t rows = row1 - row0;
    if ((size_t)nthreads > rows) nthreads = rows ? (int)rows : 1;
    pthread_t th[256];
    mm_job jobs[256];
    for (int t = 0; t < nthreads; t++) {
        mm_job j = {ggml_type, w, x, m, n, k, row0 + rows * (size_t)t / (size_t)nthreads,
                    row0 + rows * (size_t)(t + 1) / (size_t)nthreads, y, absdot, f16_operands};
        jobs[t] = j;
    }
    if (nthreads == 1) {
        mm_worker(&jobs[0]);
        return 0;
    }
    for (int t = 0; t < nthreads; t++) pthread_create(&th[t], NULL, mm_worker, &jobs[t]);
    for (int t = 0; t < nthreads; t++) pthread_join(th[t], NULL);
    return 0;
}

/* Expert-routed form: out[t*top_k+s, :] = dequant(W[ids[t*top_k+s]]) * x[t]
 * (src/ops/quantized_matmul_id_ggml.rs:163-276). */
int orc_qmatmul_id(int ggml_type, const uint8_t *w, uint64_t expert_stride, const float *x,
                   const uint32_t *ids, size_t n_tokens, size_t top_k, size_t n, size_t k,
                   size_t n_experts, float *y, double *absdot, int f16_operands, int nthreads) {
    for (size_t r = 0; r < n_tokens * top_k; r++) {
        if (ids[r] >= n_experts) return -3;
        int rc = orc_qmatmul(ggml_type, w + (size_t)ids[r] * expert_stride, x + (r / top_k) * k, 1, n, k,
                             0, n, y + r * n, absdot ? absdot + r * n : NULL, f16_operands, nthreads);
        if (rc) return rc;
    }
    return 0;
}

/* ------------------------------------------------------------------ MoE routing */

/* src/shaders/quantized_matmul_id_mm.metal:242-283.  One scan per expert over the tokens in
 * ascending order; entry = token*top_k + (sum of (slot+1) over matching slots) - 1; ids are
 * compared after truncation to 16 bits, as the shader stages them as uint16. */
void orc_moe_map0(const uint32_t *ids, size_t n_tokens, size_t top_k, size_t n_experts,
                  uint32_t *htpe, int32_t *hids) {
    for (size_t e = 0; e < n_experts; e++) {
        uint32_t n_all = 0;
        int32_t *row = hids + e * n_tokens;
        for (size_t t = 0; t < n_tokens; t++) {
            int sel = 0;
            for (size_t s = 0; s < top_k; s++)
                sel += ((uint16_t)ids[t * top_k + s] == (uint16_t)e) ? (int)(s + 1) : 0;
            if (sel > 0) row[n_all++] = (int32_t)(t * top_k) + sel - 1;
        }
        htpe[e] = n_all;
    }
}

/* src/shaders/moe_softmax_topk.metal:58-147: max, exp, halving-stride tree sum over
 * min(E,128) lanes, divide, insertion top-k with strict '>' (ties keep the lower index),
 * renormalise with the 1e-9 guard. */
void orc_moe_softmax_topk(const float *logits, size_t n_tokens, size_t n_experts, size_t top_k,
                          uint32_t *out_ids, float *out_w) {
    size_t tg = n_experts < 128 ? n_experts : 128;
    float *lane = (float *)malloc(tg * sizeof(float));
    float *prob = (float *)malloc(n_experts * sizeof(float));
    float vals[64];
    uint32_t idxs[64];
    for (size_t t = 0; t < n_tokens; t++) {
        const float *lg = logits + t * n_experts;
        for (size_t i = 0; i < tg; i++) {
            float mx = -INFINITY;
            for (size_t e = i; e < n_experts; e += tg)
                if (lg[e] > mx) mx = lg[e];
            lane[i] = mx;
        }
        for (size_t stride = tg / 2; stride > 0; stride >>= 1)
            for (size_t i = 0; i < stride; i++)
                if (lane[i + stride] > lane[i]) lane[i] = lane[i + stride];
        float gmax = lane[0];
        for (size_t i = 0; i < tg; i++) {
            float s = 0.0f;
            for (size_t e = i; e < n_experts; e += tg) {
                float ev = expf(lg[e] - gmax);
                prob[e] = ev;
                s += ev;
            }
            lane[i] = s;
        }
        for (size_t stride = tg / 2; stride > 0; stride >>= 1)
            for (size_t i = 0; i < stride; i++) lane[i] += lane[i + stride];
        float gsum = lane[0];
        for (size_t e = 0; e < n_experts; e++) prob[e] /= gsum;
        for (size_t k = 0; k < top_k; k++) {
            vals[k] = -INFINITY;
            idxs[k] = 0;
        }
        for (size_t e = 0; e < n_experts; e++) {
            float p = prob[e];
            if (p <= vals[top_k - 1]) continue;
            size_t ins = top_k - 1;
            while (ins > 0 && p > vals[ins - 1]) ins--;
            for (size_t k = top_k - 1; k > ins; k--) {
                vals[k] = vals[k - 1];
                idxs[k] = idxs[k - 1];
            }
            vals[ins] = p;
            idxs[ins] = (uint32_t)e;
        }
        float ts = 0.0f;
        for (size_t k = 0; k < top_k; k++) ts += vals[k];
        float inv = ts > 1e-9f ? 1.0f / ts : 1.0f;
        for (size_t k = 0; k < top_k; k++) {
            out_ids[t * top_k + k] = idxs[k];
            out_w[t * top_k + k] = vals[k] * inv;
        }
    }
    free(lane);
    free(prob);
}

/* src/shaders/silu_mul.metal:17-30 */
void orc_silu_mul(const float *gate, const float *up, size_t n, float *out) {
    for (size_t i = 0; i < n; i++) out[i] = gate[i] / (1.0f + expf(-gate[i])) * up[i];
}

/* src/shaders/moe_weighted_reduce.metal:33-66 without the optional shared-expert and
 * residual terms: out[t,h] = sum_k w[t,k] * y[t*top_k+k, h], k ascending, f32. */
void orc_moe_weighted_reduce(const float *y, const float *w, size_t n_tokens, size_t top_k, size_t h,
                             float *out) {
    for (size_t t = 0; t < n_tokens; t++)
        for (size_t c = 0; c < h; c++) {
            float acc = 0.0f;
            for (size_t k = 0; k < top_k; k++) acc += w[t * top_k + k] * y[(t * top_k + k) * h + c];
            out[t * h + c] = acc;
        }
}
