// Fused dequantise-and-dot mat-vec kernels for GGML Q4_0 / Q8_0 / Q6_K weights (decode path, m <= 8).
//
// Replaces upstream kernel_mul_mv_{q4_0,q8_0,q6_K}_f32 (src/shaders/quantized_matmul_ggml.metal:104-330)
// and kernel_mul_mv_id_* (src/shaders/quantized_matmul_id_ggml.metal:136-201, 327-386, 515-598).
//
// Two kernels:
//   qmv_simple  one warp per weight row, blocks read straight from global memory.  Used for shapes
//               the streaming kernel does not take (k not a multiple of 256, tiny matrices).
//   qmv_stream  persistent CTAs, one per SM.  A producer warp streams weight-row segments into a
//               shared-memory ring with bulk async copies (TMA) signalled through mbarriers; eight
//               consumer warps unpack the blocks from shared memory with conflict-free 32-bit loads,
//               multiply with activations staged (swizzled) in shared memory, and hand per-row
//               partial sums to the producer warp, which finishes the reduction and writes y.
//               The weights are read from HBM exactly once for all m <= 8 activation rows.
//
// Arithmetic: f32 throughout.  qmv_stream accumulates sum((q+offset)*x) per (sub-)block with packed
// f32x2 FMAs, then applies scale*(S - offset*sum(x)); offset is 0 for Q8_0, 136 for Q4_0 and 160 for
// Q6_K (the quants are spliced into an f32 mantissa under a 2^7 exponent, which costs one byte
// permute per element instead of an integer-to-float conversion).
#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"

namespace mlxn {

// =================================================================================================
// qmv_simple
// =================================================================================================
template <int T, int M>
__device__ __forceinline__ void dot_row_simple(const uint8_t *wrow, const float *x, uint32_t k, uint32_t lane,
                                               float (&acc)[M]) {
    if constexpr (T == GT_Q4_0) {
        const uint32_t nb = k / 32;
        for (uint32_t b = lane; b < nb; b += 32) {
            const uint8_t *blk = wrow + 18u * b;
            const float d = half_bits_to_float(ld_u16(blk));
            const float *xb = x + 32u * b;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint32_t q = ld_u16(blk + 2 + 2 * j);
                const float w0 = d * (float)((int)(q & 15u) - 8);
                const float w1 = d * (float)((int)((q >> 8) & 15u) - 8);
                const float w2 = d * (float)((int)((q >> 4) & 15u) - 8);
                const float w3 = d * (float)((int)(q >> 12) - 8);
#pragma unroll
                for (int t = 0; t < M; t++) {
                    const float *xt = xb + (size_t)t * k;
                    acc[t] = fmaf(w0, __ldg(xt + 2 * j), acc[t]);
                    acc[t] = fmaf(w1, __ldg(xt + 2 * j + 1), acc[t]);
                    acc[t] = fmaf(w2, __ldg(xt + 16 + 2 * j), acc[t]);
                    acc[t] = fmaf(w3, __ldg(xt + 16 + 2 * j + 1), acc[t]);
                }
            }
        }
    } else if constexpr (T == GT_Q8_0) {
        const uint32_t nb = k / 32;
        for (uint32_t b = lane; b < nb; b += 32) {
            const uint8_t *blk = wrow + 34u * b;
            const float d = half_bits_to_float(ld_u16(blk));
            const float *xb = x + 32u * b;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const uint32_t q = ld_u16(blk + 2 + 2 * j);
                const float w0 = d * (float)(int)(int8_t)(q & 0xFFu);
                const float w1 = d * (float)(int)(int8_t)(q >> 8);
#pragma unroll
                for (int t = 0; t < M; t++) {
                    const float *xt = xb + (size_t)t * k;
                    acc[t] = fmaf(w0, __ldg(xt + 2 * j), acc[t]);
                    acc[t] = fmaf(w1, __ldg(xt + 2 * j + 1), acc[t]);
                }
            }
        }
    } else if constexpr (T == GT_Q4_K) {
        // task = 8 consecutive bytes of one pair of sub-blocks (low nibbles: sub-block 2p, high: 2p+1): 16 per block
        const uint32_t ntask = (k / 256) * 16;
        for (uint32_t tk = lane; tk < ntask; tk += 32) {
            const uint32_t b = tk >> 4, p = (tk >> 2) & 3u, l0 = 8 * (tk & 3u);
            const uint8_t *blk = wrow + 144u * b;
            uint32_t sc1, m1, sc2, m2;
            q4k_scale_min(2 * p, blk + 4, sc1, m1);
            q4k_scale_min(2 * p + 1, blk + 4, sc2, m2);
            const float d = half_bits_to_float(ld_u16(blk)), dmin = half_bits_to_float(ld_u16(blk + 2));
            const float d1 = __fmul_rn(d, (float)sc1), min1 = __fmul_rn(dmin, (float)m1);
            const float d2 = __fmul_rn(d, (float)sc2), min2 = __fmul_rn(dmin, (float)m2);
            const uint8_t *q = blk + 16 + 32 * p + l0;
            const float *xb = x + 256u * b + 64u * p + l0;
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                const uint32_t qq = ld_u16(q + i);
                const float w0 = __fsub_rn(__fmul_rn(d1, (float)(qq & 15u)), min1);
                const float w1 = __fsub_rn(__fmul_rn(d1, (float)((qq >> 8) & 15u)), min1);
                const float w2 = __fsub_rn(__fmul_rn(d2, (float)((qq >> 4) & 15u)), min2);
                const float w3 = __fsub_rn(__fmul_rn(d2, (float)(qq >> 12)), min2);
#pragma unroll
                for (int t = 0; t < M; t++) {
                    const float *xt = xb + (size_t)t * k;
                    acc[t] = fmaf(w0, __ldg(xt + i), acc[t]);
                    acc[t] = fmaf(w1, __ldg(xt + i + 1), acc[t]);
                    acc[t] = fmaf(w2, __ldg(xt + 32 + i), acc[t]);
                    acc[t] = fmaf(w3, __ldg(xt + 32 + i + 1), acc[t]);
                }
            }
        }
    } else if constexpr (T == GT_Q5_K) {
        // src/gguf/mod.rs:469-540: f16 d, f16 dmin, scales[12] (as Q4_K), qh[32] (one high bit per value), qs[128].
        // task = 8 consecutive bytes of one pair of sub-blocks (low nibbles + bit 2p of qh: sub-block 2p; high nibbles
        // + bit 2p+1: sub-block 2p+1); value = (d*sc)*q - dmin*m with every product and the difference rounded in f32
        const uint32_t ntask = (k / 256) * 16;
        for (uint32_t tk = lane; tk < ntask; tk += 32) {
            const uint32_t b = tk >> 4, p = (tk >> 2) & 3u, l0 = 8 * (tk & 3u);
            const uint8_t *blk = wrow + 176u * b;
            uint32_t sc1, m1, sc2, m2;
            q4k_scale_min(2 * p, blk + 4, sc1, m1);
            q4k_scale_min(2 * p + 1, blk + 4, sc2, m2);
            const float d = half_bits_to_float(ld_u16(blk)), dmin = half_bits_to_float(ld_u16(blk + 2));
            const float d1 = __fmul_rn(d, (float)sc1), min1 = __fmul_rn(dmin, (float)m1);
            const float d2 = __fmul_rn(d, (float)sc2), min2 = __fmul_rn(dmin, (float)m2);
            const uint8_t *q = blk + 48 + 32 * p + l0, *qh = blk + 16 + l0;
            const float *xb = x + 256u * b + 64u * p + l0;
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                const uint32_t qq = ld_u16(q + i), hh = ld_u16(qh + i) >> (2 * p);
                const float w0 = __fsub_rn(__fmul_rn(d1, (float)((qq & 15u) + ((hh & 1u) << 4))), min1);
                const float w1 = __fsub_rn(__fmul_rn(d1, (float)(((qq >> 8) & 15u) + (((hh >> 8) & 1u) << 4))), min1);
                const float w2 = __fsub_rn(__fmul_rn(d2, (float)(((qq >> 4) & 15u) + (((hh >> 1) & 1u) << 4))), min2);
                const float w3 = __fsub_rn(__fmul_rn(d2, (float)((qq >> 12) + (((hh >> 9) & 1u) << 4))), min2);
#pragma unroll
                for (int t = 0; t < M; t++) {
                    const float *xt = xb + (size_t)t * k;
                    acc[t] = fmaf(w0, __ldg(xt + i), acc[t]);
                    acc[t] = fmaf(w1, __ldg(xt + i + 1), acc[t]);
                    acc[t] = fmaf(w2, __ldg(xt + 32 + i), acc[t]);
                    acc[t] = fmaf(w3, __ldg(xt + 32 + i + 1), acc[t]);
                }
            }
        }
    } else {  // Q6_K: 16 strips of 4 (x4 groups) per block
        const uint32_t ntask = (k / 256) * 16;
        for (uint32_t tk = lane; tk < ntask; tk += 32) {
            const uint32_t b = tk >> 4, l4 = tk & 15, h = l4 >> 3, l0 = 4 * (l4 & 7);
            const uint8_t *blk = wrow + 210u * b;
            const float d = half_bits_to_float(ld_u16(blk + 208));
            const uint32_t A = ld_u32_2(blk + 64 * h + l0);
            const uint32_t B = ld_u32_2(blk + 64 * h + 32 + l0);
            const uint32_t H = ld_u32_2(blk + 128 + 32 * h + l0);
            const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192 + 8 * h + (l0 >> 4));
            const float s0 = d * (float)sc[0], s1 = d * (float)sc[2], s2 = d * (float)sc[4], s3 = d * (float)sc[6];
            const float *xb = x + 256u * b + 128u * h + l0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t a = (A >> (8 * i)) & 0xFFu, bb = (B >> (8 * i)) & 0xFFu, hh = (H >> (8 * i)) & 0xFFu;
                const float w0 = s0 * (float)((int)((a & 15u) | ((hh & 3u) << 4)) - 32);
                const float w1 = s1 * (float)((int)((bb & 15u) | (((hh >> 2) & 3u) << 4)) - 32);
                const float w2 = s2 * (float)((int)((a >> 4) | (((hh >> 4) & 3u) << 4)) - 32);
                const float w3 = s3 * (float)((int)((bb >> 4) | ((hh >> 6) << 4)) - 32);
#pragma unroll
                for (int t = 0; t < M; t++) {
                    const float *xt = xb + (size_t)t * k + i;
                    acc[t] = fmaf(w0, __ldg(xt), acc[t]);
                    acc[t] = fmaf(w1, __ldg(xt + 32), acc[t]);
                    acc[t] = fmaf(w2, __ldg(xt + 64), acc[t]);
                    acc[t] = fmaf(w3, __ldg(xt + 96), acc[t]);
                }
            }
        }
    }
}

// grid ceil(n/8) * nprob; 256 threads; CTA b works on problem b / ceil(n/8), and its warp w owns
// weight row 8*(b % ceil(n/8)) + w.
template <int T, int M>
__global__ void __launch_bounds__(256) qmv_simple_kernel(const QmvArgs a) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t gx = (a.n + 7) / 8;
    const uint32_t row = (blockIdx.x % gx) * 8 + warp;
    if (row >= a.n) return;
    const uint32_t p = blockIdx.x / gx;
    const uint8_t *w = a.w;
    const float *x = a.x;
    float *y = a.y;
    if (a.ids) {
        const uint32_t e = a.ids[p];
        y += (size_t)p * a.n;
        if (e >= a.n_experts) {  // upstream reads out of bounds here; this build writes zeros instead
            if (lane == 0) y[row] = 0.0f;
            return;
        }
        w += (size_t)e * a.expert_stride;
        x += (size_t)(p / a.top_k) * a.k;
    }
    const size_t row_bytes = (size_t)(a.k / BlockTraits<T>::QK) * BlockTraits<T>::BYTES;
    float acc[M];
#pragma unroll
    for (int t = 0; t < M; t++) acc[t] = 0.0f;
    dot_row_simple<T, M>(w + row * row_bytes, x, a.k, lane, acc);
#pragma unroll
    for (int t = 0; t < M; t++) {
        const float s = warp_sum(acc[t]);
        if (lane == 0) {
            const size_t off = a.ids ? (size_t)t * a.n + row : (size_t)t * qmv_ld(a) + a.y_col0 + row;
            y[off] = s;
            for (uint32_t pr = 0; pr < a.n_peer; pr++) a.y_peer[pr][off] = s;
        }
    }
}

// =================================================================================================
// qmv_stream
// =================================================================================================
constexpr int kRows = 4;         // weight rows per pipeline stage
constexpr int kMaxStages = 16;

struct StreamCfg {
    uint32_t ks;          // K-slice length in elements (multiple of 256)
    uint32_t nslices;
    uint32_t wpg;         // warps cooperating on one stage (power of two)
    uint32_t lg_wpg;
    uint32_t stages;      // ring depth (power of two, multiple of the number of warp groups)
    uint32_t lg_stages;
    uint32_t seg_stride;  // shared-memory bytes reserved per row segment (multiple of 16)
    uint32_t cpp;         // CTAs per problem
    uint32_t xs_off, xsum_off, red_off, stage_off;  // byte offsets into dynamic shared memory
    uint32_t debug;       // experiment switches: 1 = skip the arithmetic, 2 = skip the weight copies
};

template <int T> struct StreamTraits;
template <> struct StreamTraits<GT_Q4_0> { static constexpr int E = 32, SUB = 32; };   // task = one block
template <> struct StreamTraits<GT_Q8_0> { static constexpr int E = 32, SUB = 32; };
template <> struct StreamTraits<GT_Q6_K> { static constexpr int E = 64, SUB = 16; };   // task = 4 sub-blocks of 16

// float4-index swizzle of the staged activations, so that the eight lanes of a quarter warp (eight
// consecutive tasks) hit eight different 16-byte bank groups.
template <int T> __device__ __forceinline__ uint32_t xswz(uint32_t f) {
    if constexpr (T == GT_Q6_K) return f ^ ((f >> 5) & 3u);
    else return f ^ ((f >> 3) & 7u);
}

// Walks the (work item, K-slice, row group) sequence of one CTA.  Producer and consumers run the same
// walk, so iteration numbers (ring slots, mbarrier phases) agree without communication.
struct Walk {
    uint32_t item, item_end, item_step;  // work items: (problem, sub-range)
    uint32_t s, g, g0, g1;
    uint32_t p;
    __device__ __forceinline__ void set_item(const QmvArgs &a, const StreamCfg &c) {
        p = item / c.cpp;
        const uint32_t sub = item % c.cpp;
        const uint32_t G = (a.n + kRows - 1) / kRows;
        g0 = (uint32_t)(((uint64_t)G * sub) / c.cpp);
        g1 = (uint32_t)(((uint64_t)G * (sub + 1)) / c.cpp);
        s = 0;
        g = g0;
    }
    __device__ __forceinline__ bool init(const QmvArgs &a, const StreamCfg &c) {
        item = blockIdx.x;
        item_end = a.nprob * c.cpp;
        item_step = gridDim.x;
        while (item < item_end) {
            set_item(a, c);
            if (g0 < g1) return true;
            item += item_step;
        }
        return false;
    }
    // move to the first group of the next slice (or of the next work item); false at the end of the walk
    __device__ __forceinline__ bool next_slice(const QmvArgs &a, const StreamCfg &c) {
        if (++s < c.nslices) {
            g = g0;
            return true;
        }
        item += item_step;
        while (item < item_end) {
            set_item(a, c);
            if (g0 < g1) return true;
            item += item_step;
        }
        return false;
    }
    // advance by n iterations; false if the walk ends first
    __device__ __forceinline__ bool advance(uint32_t n, const QmvArgs &a, const StreamCfg &c) {
        for (;;) {
            const uint32_t rem = g1 - g;
            if (n < rem) {
                g += n;
                return true;
            }
            n -= rem;
            if (!next_slice(a, c)) return false;
        }
    }
};

__device__ __forceinline__ const uint8_t *problem_weights(const QmvArgs &a, uint32_t p, bool &valid) {
    valid = true;
    if (!a.ids) return a.w;
    const uint32_t e = a.ids[p];
    if (e >= a.n_experts) {
        valid = false;
        return a.w;
    }
    return a.w + (size_t)e * a.expert_stride;
}

// ---- per-type task bodies ---------------------------------------------------------------------
// A task is E consecutive-in-block elements of kRows weight rows times M activation rows.
// `seg[r]` is the shared-memory address of row r's segment (first byte of the slice's first block).
// `xs` is the swizzled activation slice ([M][ks/4] float4), `xsum` the per-SUB sums ([M][ks/SUB]).

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint32_t v;
    asm volatile("{ .reg .u16 t; ld.shared.u16 t, [%1]; cvt.u32.u16 %0, t; }" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void lds128(uint32_t addr, uint64_t &lo, uint64_t &hi) {
    asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(lo), "=l"(hi) : "r"(addr));
}

// Reads NW logical 32-bit words starting at the 2-byte-aligned shared address `addr`.
template <int NW> __device__ __forceinline__ void lds_words(uint32_t addr, uint32_t (&out)[NW]) {
    const uint32_t al = addr & ~3u;
    const uint32_t sh = (addr & 2u) * 8u;
    uint32_t prev = lds32(al);
#pragma unroll
    for (int j = 0; j < NW; j++) {
        const uint32_t nxt = lds32(al + 4 * (j + 1));
        out[j] = __funnelshift_rc(prev, nxt, sh);
        prev = nxt;
    }
}

// byte i of `v` spliced into an f32 mantissa: 128 + byte (byte < 128)
template <int I> __device__ __forceinline__ uint32_t splice_128(uint32_t v) {
    return __byte_perm(v, 0x43000000u, 0x7044u | (I << 8));
}
// byte i of `v` as 2^23 + byte
template <int I> __device__ __forceinline__ uint32_t splice_2p23(uint32_t v) {
    return __byte_perm(v, 0x4B000000u, 0x7540u | I);
}

template <int M>
__device__ __forceinline__ void task_q4_0(const uint32_t (&seg)[kRows], uint32_t c, uint32_t xs, uint32_t xsum,
                                          uint32_t ks, float (&acc)[kRows][M]) {
    uint32_t lo[kRows][4], hi[kRows][4];
    float d[kRows];
#pragma unroll
    for (int r = 0; r < kRows; r++) {
        const uint32_t o = seg[r] + 18u * c;
        d[r] = half_bits_to_float(lds16(o));
        uint32_t q[4];
        lds_words<4>(o + 2, q);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            lo[r][j] = q[j] & 0x0F0F0F0Fu;
            hi[r][j] = (q[j] >> 4) & 0x0F0F0F0Fu;
        }
    }
    uint64_t S[kRows][M];
#pragma unroll
    for (int r = 0; r < kRows; r++)
#pragma unroll
        for (int t = 0; t < M; t++) S[r][t] = 0ull;
#pragma unroll
    for (int jj = 0; jj < 8; jj++) {
        uint64_t xa[M], xb[M];
        const uint32_t f = xswz<GT_Q4_0>(8u * c + jj);
#pragma unroll
        for (int t = 0; t < M; t++) lds128(xs + (t * (ks >> 2) + f) * 16u, xa[t], xb[t]);
#pragma unroll
        for (int r = 0; r < kRows; r++) {
            const uint32_t v = jj < 4 ? lo[r][jj & 3] : hi[r][jj & 3];
            const uint64_t p0 = pack2u(splice_128<0>(v), splice_128<1>(v));
            const uint64_t p1 = pack2u(splice_128<2>(v), splice_128<3>(v));
#pragma unroll
            for (int t = 0; t < M; t++) {
                S[r][t] = ffma2(p0, xa[t], S[r][t]);
                S[r][t] = ffma2(p1, xb[t], S[r][t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < M; t++) {
        float X;
        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(X) : "r"(xsum + (t * (ks >> 5) + c) * 4u));
#pragma unroll
        for (int r = 0; r < kRows; r++) acc[r][t] = fmaf(d[r], fmaf(-136.0f, X, sum2(S[r][t])), acc[r][t]);
    }
}

template <int M>
__device__ __forceinline__ void task_q8_0(const uint32_t (&seg)[kRows], uint32_t c, uint32_t xs, uint32_t /*xsum*/,
                                          uint32_t ks, float (&acc)[kRows][M]) {
    uint32_t q[kRows][8];
    float d[kRows];
#pragma unroll
    for (int r = 0; r < kRows; r++) {
        const uint32_t o = seg[r] + 34u * c;
        d[r] = half_bits_to_float(lds16(o));
        lds_words<8>(o + 2, q[r]);
#pragma unroll
        for (int j = 0; j < 8; j++) q[r][j] ^= 0x80808080u;
    }
    uint64_t S[kRows][M];
#pragma unroll
    for (int r = 0; r < kRows; r++)
#pragma unroll
        for (int t = 0; t < M; t++) S[r][t] = 0ull;
    const uint64_t negC = pack2(-8388736.0f, -8388736.0f);  // -(2^23 + 128)
#pragma unroll
    for (int jj = 0; jj < 8; jj++) {
        uint64_t xa[M], xb[M];
        const uint32_t f = xswz<GT_Q8_0>(8u * c + jj);
#pragma unroll
        for (int t = 0; t < M; t++) lds128(xs + (t * (ks >> 2) + f) * 16u, xa[t], xb[t]);
#pragma unroll
        for (int r = 0; r < kRows; r++) {
            const uint32_t v = q[r][jj];
            const uint64_t p0 = fadd2(pack2u(splice_2p23<0>(v), splice_2p23<1>(v)), negC);
            const uint64_t p1 = fadd2(pack2u(splice_2p23<2>(v), splice_2p23<3>(v)), negC);
#pragma unroll
            for (int t = 0; t < M; t++) {
                S[r][t] = ffma2(p0, xa[t], S[r][t]);
                S[r][t] = ffma2(p1, xb[t], S[r][t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < M; t++)
#pragma unroll
        for (int r = 0; r < kRows; r++) acc[r][t] = fmaf(d[r], sum2(S[r][t]), acc[r][t]);
}

// Q6_K task c: block b = c>>2, half h = (c>>1)&1, strip-half is = c&1; the task covers, for g = 0..3,
// elements 256b + 128h + 32g + 16is + [0,16).
template <int M>
__device__ __forceinline__ void task_q6_k(const uint32_t (&seg)[kRows], uint32_t c, uint32_t xs, uint32_t xsum,
                                          uint32_t ks, float (&acc)[kRows][M]) {
    const uint32_t b = c >> 2, h = (c >> 1) & 1u, is = c & 1u;
    uint32_t A[kRows][4], B[kRows][4], H[kRows][4];
    float ds[kRows][4];
#pragma unroll
    for (int r = 0; r < kRows; r++) {
        const uint32_t o = seg[r] + 210u * b;
        lds_words<4>(o + 64 * h + 16 * is, A[r]);
        lds_words<4>(o + 64 * h + 32 + 16 * is, B[r]);
        lds_words<4>(o + 128 + 32 * h + 16 * is, H[r]);
        const float d = half_bits_to_float(lds16(o + 208));
#pragma unroll
        for (int g = 0; g < 4; g++) ds[r][g] = d * (float)lds_s8(o + 192 + 8 * h + is + 2 * g);
    }
    const uint32_t fbase = 64u * b + 32u * h + 4u * is;  // float4 index of element group g=0, q=0
    const uint32_t subbase = 16u * b + 8u * h + is;      // 16-element sub-block index of group g=0
#pragma unroll
    for (int g = 0; g < 4; g++) {
        uint64_t S[kRows][M];
#pragma unroll
        for (int r = 0; r < kRows; r++)
#pragma unroll
            for (int t = 0; t < M; t++) S[r][t] = 0ull;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            uint64_t xa[M], xb[M];
            const uint32_t f = xswz<GT_Q6_K>(fbase + 8u * g + q);
#pragma unroll
            for (int t = 0; t < M; t++) lds128(xs + (t * (ks >> 2) + f) * 16u, xa[t], xb[t]);
#pragma unroll
            for (int r = 0; r < kRows; r++) {
                uint32_t v;
                if (g == 0) v = (A[r][q] & 0x0F0F0F0Fu) | ((H[r][q] << 4) & 0x30303030u);
                else if (g == 1) v = (B[r][q] & 0x0F0F0F0Fu) | ((H[r][q] << 2) & 0x30303030u);
                else if (g == 2) v = ((A[r][q] >> 4) & 0x0F0F0F0Fu) | (H[r][q] & 0x30303030u);
                else v = ((B[r][q] >> 4) & 0x0F0F0F0Fu) | ((H[r][q] >> 2) & 0x30303030u);
                const uint64_t p0 = pack2u(splice_128<0>(v), splice_128<1>(v));
                const uint64_t p1 = pack2u(splice_128<2>(v), splice_128<3>(v));
#pragma unroll
                for (int t = 0; t < M; t++) {
                    S[r][t] = ffma2(p0, xa[t], S[r][t]);
                    S[r][t] = ffma2(p1, xb[t], S[r][t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < M; t++) {
            float X;
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(X) : "r"(xsum + (t * (ks >> 4) + subbase + 2 * g) * 4u));
#pragma unroll
            for (int r = 0; r < kRows; r++) acc[r][t] = fmaf(ds[r][g], fmaf(-160.0f, X, sum2(S[r][t])), acc[r][t]);
        }
    }
}

template <int T, int M, int NW>
__global__ void __launch_bounds__(NW * 32, 1) qmv_stream_kernel(const QmvArgs a, const StreamCfg c) {
    constexpr int kStreamThreads = NW * 32;
    constexpr int kConsumerWarps = NW;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages];
    __shared__ uint32_t done_cnt[kMaxStages];  // warps of the owning group that have finished with a slot
    __shared__ volatile uint32_t abort_flag;

    constexpr int QK = BlockTraits<T>::QK, BB = BlockTraits<T>::BYTES;
    constexpr int E = StreamTraits<T>::E, SUB = StreamTraits<T>::SUB;
    constexpr int V = kRows * M;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t row_bytes = (a.k / QK) * BB;
    const uint32_t slice_bytes = (c.ks / QK) * BB;
    const uint32_t ngrp = kConsumerWarps / c.wpg;

    if (tid == 0) {
        abort_flag = 0;
        for (uint32_t s = 0; s < c.stages; s++) {
            mbar_init(&full_bar[s], 1);
            done_cnt[s] = 0;
        }
        mbar_init_fence();
    }
    __syncthreads();

    const uint32_t smem_base = smem_u32(smem);
    const uint32_t xs = smem_base + c.xs_off;
    const uint32_t xsum = smem_base + c.xsum_off;
    float *red = reinterpret_cast<float *>(smem + c.red_off);  // [stages][8 warps][V]
    const uint32_t stage_bytes = kRows * c.seg_stride;

    // Every warp belongs to a group of c.wpg warps; group cg owns iterations it with it % ngrp == cg and,
    // because c.stages is a multiple of ngrp, also the ring slots those iterations use.  Warp 0 of a group
    // refills a slot (bulk copies of the next kRows row segments) as soon as the group has finished with it.
    const uint32_t cg = warp >> c.lg_wpg, wig = warp & (c.wpg - 1u);
    const bool leader = wig == 0;

    // lanes 0..kRows-1 of a group's leader warp each issue one row-segment copy of iteration `it`
    auto issue = [&](const Walk &w, uint32_t it) {
        const uint32_t slot = it & (c.stages - 1u);
        bool valid;
        const uint8_t *wb = problem_weights(a, w.p, valid);
        const uint32_t row0 = w.g * kRows;
        const uint32_t nrows = min((uint32_t)kRows, a.n - row0);
        const uint32_t kb = min(c.ks, a.k - w.s * c.ks);  // elements in this slice
        const uint32_t seg_bytes = (kb / QK) * BB;
        const uint8_t *src = wb + (size_t)(row0 + lane) * row_bytes + (size_t)w.s * slice_bytes;
        const uint32_t pre = (uint32_t)((uintptr_t)src & 15u);
        const uint32_t bytes = (valid && lane < nrows && !(MLXN_DBG(c) & 2u)) ? ((pre + seg_bytes + 15u) & ~15u) : 0u;
        uint32_t total = bytes;
        total += __shfl_xor_sync(0xffffffffu, total, 1);
        total += __shfl_xor_sync(0xffffffffu, total, 2);
        if (lane == 0) {
            if (total == 0) mbar_arrive(&full_bar[slot]);
            else mbar_expect_tx(&full_bar[slot], total);
        }
        __syncwarp();
        if (bytes) bulk_g2s(smem + c.stage_off + slot * stage_bytes + lane * c.seg_stride, src - pre, bytes, &full_bar[slot]);
    };

    Walk w;
    bool more = w.init(a, c);
    const uint32_t smask = c.stages - 1;
    // This kernel may have been scheduled while the one ahead of it in the stream is still running.  Weights
    // that no kernel writes can be requested right away; everything else waits for the kernels ahead.
    if (!a.early_weights) grid_dependency_wait();
    // prime the ring: each group's leader issues the iterations it owns among the first c.stages
    if (more && leader) {
        for (uint32_t i = cg; i < c.stages; i += ngrp) {
            Walk t = w;
            if (!t.advance(i, a, c)) break;
            issue(t, i);
        }
    }
    if (a.early_weights) grid_dependency_wait();
    allow_dependents();

    // Each warp steps through the whole walk slice by slice (every warp stages every activation slice) but
    // jumps straight between the iterations its group owns: it, it + ngrp, ...
    uint32_t it = 0;        // iteration number of the cursor position
    uint32_t skip = cg;     // iterations between the cursor and this group's next own iteration
    const uint32_t ks4 = c.ks >> 2;
    bool staged = false;
    while (more) {
        if (!staged) {
            // ---- stage the activation slice of (w.item, w.s) (all warps) ----
            staged = true;
            named_bar_sync(1, kStreamThreads);  // everyone is done with the previous slice
            const float *xg = a.x + (a.ids ? (size_t)(w.p / a.top_k) * a.k : 0);
            const uint32_t k0 = w.s * c.ks;
            // loads are issued in batches of eight per thread before any is stored, so that the L2 latency is
            // paid once per batch instead of once per element
            constexpr int kBatch = 8;
            for (uint32_t base = 0; base < M * ks4; base += kBatch * kStreamThreads) {
                float4 v[kBatch];
#pragma unroll
                for (int u = 0; u < kBatch; u++) {
                    const uint32_t idx = base + u * kStreamThreads + tid;
                    v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (idx < M * ks4) {
                        const uint32_t t = idx / ks4, f = idx - t * ks4;
                        if (k0 + 4 * f < a.k) {
                            v[u] = __ldg(reinterpret_cast<const float4 *>(xg + (size_t)t * a.k + k0) + f);
                            if (a.x2) {   // fused SwiGLU: silu(gate) * up (src/shaders/quantized_matmul_id_ggml.metal:231-319)
                                const float4 up = __ldg(reinterpret_cast<const float4 *>(xg + (a.x2 - a.x) + (size_t)t * a.k + k0) + f);
                                v[u].x = v[u].x / (1.0f + expf(-v[u].x)) * up.x;
                                v[u].y = v[u].y / (1.0f + expf(-v[u].y)) * up.y;
                                v[u].z = v[u].z / (1.0f + expf(-v[u].z)) * up.z;
                                v[u].w = v[u].w / (1.0f + expf(-v[u].w)) * up.w;
                            }
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < kBatch; u++) {
                    const uint32_t idx = base + u * kStreamThreads + tid;
                    if (idx < M * ks4) {
                        const uint32_t t = idx / ks4, f = idx - t * ks4;
                        *reinterpret_cast<float4 *>(smem + c.xs_off + (size_t)(t * ks4 + xswz<T>(f)) * 16) = v[u];
                    }
                }
            }
            named_bar_sync(1, kStreamThreads);
            if constexpr (T != GT_Q8_0) {
                const uint32_t nsub = c.ks / SUB;
                for (uint32_t idx = tid; idx < M * nsub; idx += kStreamThreads) {
                    const uint32_t t = idx / nsub, sb = idx - t * nsub;
                    float s = 0.0f;
#pragma unroll
                    for (int q = 0; q < SUB / 4; q++) {
                        const float4 v = *reinterpret_cast<const float4 *>(
                            smem + c.xs_off + (size_t)(t * ks4 + xswz<T>(sb * (SUB / 4) + q)) * 16);
                        s += v.x;
                        s += v.y;
                        s += v.z;
                        s += v.w;
                    }
                    reinterpret_cast<float *>(smem + c.xsum_off)[t * nsub + sb] = s;
                }
                named_bar_sync(1, kStreamThreads);
            }
        }
        const uint32_t rem = w.g1 - w.g;  // iterations left in this slice, cursor included
        if (skip >= rem) {                // this group's next iteration lies beyond this slice
            skip -= rem;
            it += rem;
            more = w.next_slice(a, c);
            staged = false;
            continue;
        }
        w.g += skip;
        it += skip;
        skip = ngrp;
        {
            const uint32_t slot = it & smask;
            bool valid;
            const uint8_t *wb = problem_weights(a, w.p, valid);
            const uint32_t row0 = w.g * kRows;
            const uint32_t kb = min(c.ks, a.k - w.s * c.ks);
            const uint32_t ntasks = kb / E;
            uint32_t seg[kRows];
#pragma unroll
            for (int r = 0; r < kRows; r++) {
                const uint32_t rr = min(row0 + r, a.n - 1);
                const uint8_t *src = wb + (size_t)rr * row_bytes + (size_t)w.s * slice_bytes;
                seg[r] = smem_base + c.stage_off + slot * stage_bytes + r * c.seg_stride + (uint32_t)((uintptr_t)src & 15u);
            }
            float acc[kRows][M];
#pragma unroll
            for (int r = 0; r < kRows; r++)
#pragma unroll
                for (int t = 0; t < M; t++) acc[r][t] = 0.0f;
            const bool landed = !abort_flag && mbar_wait(&full_bar[slot], (it >> c.lg_stages) & 1u, &abort_flag, a.status, ST_WAIT_FULL_TIMEOUT, 100);
            if (valid && landed && !(MLXN_DBG(c) & 1u)) {
                for (uint32_t task = wig * 32 + lane; task < ntasks; task += 32 * c.wpg) {
                    if constexpr (T == GT_Q4_0) task_q4_0<M>(seg, task, xs, xsum, c.ks, acc);
                    else if constexpr (T == GT_Q8_0) task_q8_0<M>(seg, task, xs, xsum, c.ks, acc);
                    else task_q6_k<M>(seg, task, xs, xsum, c.ks, acc);
                }
            }
            // butterfly reduce-scatter across the warp: V values per lane -> lane L holds total number idx(L)
            constexpr int VP = V <= 4 ? 4 : V <= 8 ? 8 : V <= 16 ? 16 : 32;
            float v[VP];
#pragma unroll
            for (int i = 0; i < VP; i++) v[i] = i < V ? acc[i / M][i % M] : 0.0f;
            uint32_t idx = 0;
            {
                int hs = VP / 2;
                int bit = 16;
#pragma unroll
                for (int step = 0; step < 5; step++) {
                    if (hs >= 1) {
                        const bool upper = (lane & bit) != 0;
#pragma unroll
                        for (int i = 0; i < hs; i++) {
                            const float send = upper ? v[i] : v[i + hs];
                            const float keep = upper ? v[i + hs] : v[i];
                            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
                        }
                        if (upper) idx += hs;
                        hs >>= 1;
                    } else {
                        v[0] += __shfl_xor_sync(0xffffffffu, v[0], bit);
                    }
                    bit >>= 1;
                }
            }
            constexpr uint32_t kIdleMask = VP >= 32 ? 0u : (32u / VP) - 1u;  // lanes whose low bits are 0 write
            if ((lane & kIdleMask) == 0 && idx < V) red[(slot * kConsumerWarps + wig) * V + idx] = v[0];
            // No warp waits for another: the last warp of the group to finish with this slot (counted in
            // shared memory) adds up the group's partial sums, writes y and refills the slot.
            __syncwarp();
            uint32_t last = 0;
            if (lane == 0) {
                __threadfence_block();
                last = (atomicAdd(&done_cnt[slot], 1u) == c.wpg - 1u) ? 1u : 0u;
                if (last) {
                    done_cnt[slot] = 0;
                    __threadfence_block();
                }
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                if (lane < V) {
                    const uint32_t r = lane / M, t = lane % M;
                    if (row0 + r < a.n && landed) {
                        float s = 0.0f;
                        for (uint32_t w8 = 0; w8 < c.wpg; w8++)
                            s += *reinterpret_cast<volatile float *>(&red[(slot * kConsumerWarps + w8) * V + lane]);
                        const size_t off = (a.ids ? (size_t)w.p * a.n : (size_t)t * qmv_ld(a) + a.y_col0) + row0 + r;
                        if (w.s != 0) s += a.y[off];   // later K slices add to what the earlier ones left (same thread)
                        a.y[off] = s;
                        for (uint32_t pr = 0; pr < a.n_peer; pr++) a.y_peer[pr][off] = s;
                    }
                }
                __syncwarp();
                if (!abort_flag) {  // iteration it + c.stages reuses this slot
                    Walk t = w;
                    if (t.advance(c.stages, a, c)) issue(t, it + c.stages);
                }
            }
        }
    }
    if (abort_flag) {  // let copies in flight land before the CTA's shared memory is released
        for (int i = 0; i < 200; i++) __nanosleep(5000);
    }
}

// =================================================================================================
// host-side launchers
// =================================================================================================
static inline uint32_t round_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

template <int T>
static bool stream_config(const QmvArgs &a, int sm_count, size_t smem_limit, uint32_t nw, StreamCfg &c, uint32_t &grid, size_t &smem) {
    const uint32_t kConsumerWarps = nw;
    constexpr int QK = BlockTraits<T>::QK, BB = BlockTraits<T>::BYTES;
    constexpr int E = StreamTraits<T>::E, SUB = StreamTraits<T>::SUB;
    if (a.k % 256 != 0 || a.k < 256) return false;
    if (((uintptr_t)a.w & 1u) || (a.expert_stride & 1u)) return false;
    if (((uintptr_t)a.x & 15u) || (a.k % 4)) return false;
    const uint32_t m = a.m;
    // K-slicing: keep the staged activations within ~96 KiB
    const uint32_t xmax = 96 * 1024;
    uint32_t nslices = 1;
    uint32_t ks = a.k;
    while ((size_t)m * ks * 4 > xmax) {
        nslices++;
        ks = round_up((a.k + nslices - 1) / nslices, 256);
    }
    nslices = (a.k + ks - 1) / ks;
    const uint32_t seg_bytes = ks / QK * BB;
    const uint32_t seg_stride = round_up(seg_bytes + 15, 16) + 16;
    const uint32_t stage_bytes = kRows * seg_stride;
    const uint32_t xs_bytes = m * ks * 4;
    const uint32_t xsum_bytes = round_up(m * (ks / SUB) * 4, 16);
    const uint32_t red_bytes_per_stage = kConsumerWarps * kRows * m * 4;
    size_t fixed = (size_t)xs_bytes + xsum_bytes + 1024;
    if (fixed + 2 * (size_t)(stage_bytes + red_bytes_per_stage) > smem_limit) return false;
    uint32_t stages = (uint32_t)((smem_limit - fixed) / (stage_bytes + red_bytes_per_stage));
    if (stages > kMaxStages) stages = kMaxStages;
    // enough ring depth for ~96 KiB in flight is plenty
    while (stages > 3 && (size_t)(stages - 1) * stage_bytes > 128 * 1024) stages--;
    uint32_t tasks = ks / E;
    uint32_t wpg = 1;
    while (wpg < kConsumerWarps && wpg * 32 < tasks) wpg *= 2;
    const uint32_t ngrp = kConsumerWarps / wpg;
    uint32_t p2 = 1, lg = 0;
    while (p2 * 2 <= stages) {
        p2 *= 2;
        lg++;
    }
    stages = p2;                      // power of two: ring slot and phase come from masks and shifts
    if (stages < ngrp || stages < 2) return false;   // every group refills the ring slots it owns
    uint32_t lg_wpg = 0;
    while ((1u << lg_wpg) < wpg) lg_wpg++;
    c.lg_stages = lg;
    c.lg_wpg = lg_wpg;
    {
        const char *dbg = exp_env("MLXN_MV_DEBUG");
        c.debug = dbg ? (uint32_t)atoi(dbg) : 0u;
    }
    c.ks = ks;
    c.nslices = nslices;
    c.wpg = wpg;
    c.stages = stages;
    c.seg_stride = seg_stride;
    c.xs_off = 0;
    c.xsum_off = xs_bytes;
    c.red_off = c.xsum_off + xsum_bytes;
    c.stage_off = round_up(c.red_off + stages * red_bytes_per_stage, 128);
    smem = (size_t)c.stage_off + (size_t)stages * stage_bytes;
    if (smem > smem_limit) return false;
    const uint32_t G = (a.n + kRows - 1) / kRows;
    uint32_t g = (uint32_t)sm_count;
    if (a.nprob >= g) {
        c.cpp = 1;
    } else {
        c.cpp = g / a.nprob;
        if (c.cpp > G) c.cpp = G;
        if (c.cpp == 0) c.cpp = 1;
    }
    const uint32_t items = a.nprob * c.cpp;
    grid = items < g ? items : g;
    return grid > 0;
}

template <int T, int M, int NW> static cudaError_t launch_stream_tm(const QmvArgs &a, const StreamCfg &c, uint32_t grid, size_t smem,
                                                            cudaStream_t st) {
    static size_t attr_smem[64] = {};  // largest dynamic shared-memory size enabled so far, per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (smem > attr_smem[dev]) {
        cudaError_t e = cudaFuncSetAttribute(qmv_stream_kernel<T, M, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_smem[dev] = smem;
    }
    cudaError_t le = launch_overlapped(qmv_stream_kernel<T, M, NW>, dim3(grid), dim3(NW * 32), smem, st, a, c);
    if (le != cudaSuccess) return le;
    return cudaGetLastError();
}

template <int T, int M> static cudaError_t launch_simple_tm(const QmvArgs &a, cudaStream_t st) {
    const uint64_t blocks = (uint64_t)((a.n + 7) / 8) * a.nprob;
    if (blocks > 0x7FFFFFFFull) return cudaErrorInvalidConfiguration;
    qmv_simple_kernel<T, M><<<(unsigned)blocks, 256, 0, st>>>(a);
    return cudaGetLastError();
}

template <int T> static cudaError_t launch_t(const QmvArgs &a, bool want_stream, int sm_count, cudaStream_t st,
                                             const char **kname) {
    StreamCfg c{};
    uint32_t grid = 0;
    size_t smem = 0;
    const uint32_t nw = a.m <= 2 ? 16 : 8;
    const bool stream = want_stream && stream_config<T>(a, sm_count, 227 * 1024 - 2048, nw, c, grid, smem);
    *kname = stream ? "qmv_stream" : "qmv_simple";
#define MLXN_CASE(MM)                                                                   \
    case MM:                                                                            \
        return stream ? launch_stream_tm<T, MM, (MM <= 2 ? 16 : 8)>(a, c, grid, smem, st) : launch_simple_tm<T, MM>(a, st);
    switch (a.m) {
        MLXN_CASE(1)
        MLXN_CASE(2)
        MLXN_CASE(3)
        MLXN_CASE(4)
        MLXN_CASE(5)
        MLXN_CASE(6)
        MLXN_CASE(7)
        MLXN_CASE(8)
    default:
        return cudaErrorInvalidValue;
    }
#undef MLXN_CASE
}

// Whether launch_qmv would run the streaming kernel for these arguments (the only one of the two that knows the fused
// SwiGLU form, QmvArgs::x2).
bool qmv_stream_available(int ggml_type, const QmvArgs &a, int sm_count) {
    StreamCfg c{};
    uint32_t grid = 0;
    size_t smem = 0;
    const uint32_t nw = a.m <= 2 ? 16 : 8;
    switch (ggml_type) {
    case GT_Q4_0: return stream_config<GT_Q4_0>(a, sm_count, 227 * 1024 - 2048, nw, c, grid, smem);
    case GT_Q8_0: return stream_config<GT_Q8_0>(a, sm_count, 227 * 1024 - 2048, nw, c, grid, smem);
    case GT_Q6_K: return stream_config<GT_Q6_K>(a, sm_count, 227 * 1024 - 2048, nw, c, grid, smem);
    default: return false;
    }
}

// Launches the mat-vec for a.m in [1,8] (dense) or the routed form (a.ids != nullptr, a.m == 1).
cudaError_t launch_qmv(int ggml_type, const QmvArgs &a, bool want_stream, int sm_count, cudaStream_t st,
                       const char **kname) {
    switch (ggml_type) {
    case GT_Q4_0: return launch_t<GT_Q4_0>(a, want_stream, sm_count, st, kname);
    case GT_Q8_0: return launch_t<GT_Q8_0>(a, want_stream, sm_count, st, kname);
    case GT_Q6_K: return launch_t<GT_Q6_K>(a, want_stream, sm_count, st, kname);
    case GT_Q4_K: {   // the simple kernel only (no streaming or tensor-core form yet)
        *kname = "qmv_simple";
        switch (a.m) {
        case 1: return launch_simple_tm<GT_Q4_K, 1>(a, st);
        case 2: return launch_simple_tm<GT_Q4_K, 2>(a, st);
        case 3: return launch_simple_tm<GT_Q4_K, 3>(a, st);
        case 4: return launch_simple_tm<GT_Q4_K, 4>(a, st);
        case 5: return launch_simple_tm<GT_Q4_K, 5>(a, st);
        case 6: return launch_simple_tm<GT_Q4_K, 6>(a, st);
        case 7: return launch_simple_tm<GT_Q4_K, 7>(a, st);
        case 8: return launch_simple_tm<GT_Q4_K, 8>(a, st);
        default: return cudaErrorInvalidValue;
        }
    }
    case GT_Q5_K:   // the expert-routed mat-vec only, as upstream (src/shaders/quantized_matmul_id_ggml.metal:401-509)
        *kname = "qmv_simple";
        if (a.m != 1) return cudaErrorInvalidValue;
        return launch_simple_tm<GT_Q5_K, 1>(a, st);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace mlxn
