// Mat-mat kernels for GGML Q4_0 / Q8_0 / Q6_K weights (prefill path, m > 8), dense and grouped by expert.
//
// Replaces upstream kernel_mul_mm_*_tensor_f32 (src/shaders/quantized_matmul_mm_tensor.metal:170-343),
// kernel_mul_mm_id_*_tensor_f32 (src/shaders/quantized_matmul_id_mm_tensor.metal:165-341) and the
// simdgroup variants beside them.  Operand semantics are those of the upstream tensor path: weights
// are dequantised in f32 and rounded once to f16, activations are rounded f32 -> f16, products are
// accumulated in f32.
//
//   qmm_tc    tcgen05 kernel.  Per CTA one output tile of 128 weight rows x NT activation rows.
//             Activations are packed once per call into f16 tiles already in the tensor core's
//             K-major 128-byte-swizzled shared-memory layout (pack_x), so the GEMM fetches them with
//             one bulk async copy per 64-wide K chunk.  Raw weight blocks are bulk-copied into a
//             staging ring, eight warps dequantise them into the swizzled f16 A tile, one thread
//             issues tcgen05.mma (M=128, N=NT, K=16) accumulating in tensor memory, and the same
//             eight warps read the accumulator back with tcgen05.ld and store y.
//   qmm_simt  plain CUDA-core tile kernel with the same operand rounding; used for shapes the
//             tcgen05 kernel does not take and as an on-device cross-check.
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "ptx.cuh"
#include "tensor_map.cuh"

namespace mlxn {

// =================================================================================================
// element-wise dequantisation helpers
// =================================================================================================
// Exact value of element `e` of a weight row stored as raw GGML blocks (global memory).
template <int T> __device__ __forceinline__ float dequant_elem(const uint8_t *row, uint32_t e) {
    if constexpr (T == GT_Q4_0) {
        const uint8_t *blk = row + 18u * (e >> 5);
        const uint32_t i = e & 31u;
        const uint32_t byte = blk[2 + (i & 15u)];
        const int nib = (i < 16) ? (int)(byte & 15u) : (int)(byte >> 4);
        return half_bits_to_float(ld_u16(blk)) * (float)(nib - 8);
    } else if constexpr (T == GT_Q8_0) {
        const uint8_t *blk = row + 34u * (e >> 5);
        return half_bits_to_float(ld_u16(blk)) * (float)(int)(int8_t)blk[2 + (e & 31u)];
    } else if constexpr (T == GT_Q4_K) {
        // f16 d, f16 dmin, scales[12], qs[128]; sub-block j = e / 32 of the super-block, byte (j / 2) * 32 + l,
        // low nibble for even j (src/gguf/mod.rs:582-644).  (d sc) q - (dmin m), each step rounded in f32.
        const uint8_t *blk = row + 144u * (e >> 8);
        const uint32_t r = e & 255u, j = r >> 5, l = r & 31u;
        uint32_t sc, mn;
        q4k_scale_min(j, blk + 4, sc, mn);
        const uint32_t byte = blk[16 + 32 * (j >> 1) + l];
        const uint32_t q = (j & 1u) ? (byte >> 4) : (byte & 15u);
        const float dj = __fmul_rn(half_bits_to_float(ld_u16(blk)), (float)sc);
        const float mj = __fmul_rn(half_bits_to_float(ld_u16(blk + 2)), (float)mn);
        return __fsub_rn(__fmul_rn(dj, (float)q), mj);
    } else {
        const uint8_t *blk = row + 210u * (e >> 8);
        const uint32_t r = e & 255u, h = r >> 7, g = (r & 127u) >> 5, l = r & 31u;
        const uint32_t qlb = blk[64 * h + 32 * (g & 1u) + l];
        const uint32_t nib = (g < 2) ? (qlb & 15u) : (qlb >> 4);
        const uint32_t hb = (blk[128 + 32 * h + l] >> (2 * g)) & 3u;
        const int q = (int)(nib | (hb << 4)) - 32;
        const float sc = (float)(int)(int8_t)blk[192 + 8 * h + (l >> 4) + 2 * g];
        return half_bits_to_float(ld_u16(blk + 208)) * sc * (float)q;
    }
}

__device__ __forceinline__ float round_f16(float v) { return __half2float(__float2half_rn(v)); }

// =================================================================================================
// qmm_simt: 64 x 64 output tile, K step 32, 256 threads, 4 x 4 outputs per thread
// =================================================================================================
// grid (ceil(rows/64), ceil(n/64), n_experts or 1)
template <int T>
__global__ void __launch_bounds__(256) qmm_simt_kernel(const QmmArgs a) {
    __shared__ float Ws[32][64 + 1];
    __shared__ float Xs[32][64 + 1];
    __shared__ int32_t orow[64];  // output row of each tile row, -1 if none
    __shared__ int32_t xrow[64];  // activation row of each tile row
    const uint32_t tid = threadIdx.x;
    const uint32_t r1 = blockIdx.x * 64, r0 = blockIdx.y * 64, e = blockIdx.z;
    const uint8_t *w = a.w;
    uint32_t nrows = a.m;
    if (a.hids) {
        nrows = a.htpe[e];
        if (r1 >= nrows) return;
        w += (size_t)e * a.expert_stride;
    }
    if (tid < 64) {
        int32_t o = -1, xr = 0;
        if (r1 + tid < nrows) {
            if (a.hids) {
                const int32_t id = a.hids[(size_t)e * a.hids_stride + r1 + tid];
                if (id >= 0 && (uint32_t)id < a.total_rows) {
                    o = id;
                    xr = id / (int32_t)a.top_k;
                }
            } else {
                o = (int32_t)(r1 + tid);
                xr = o;
            }
        }
        orow[tid] = o;
        xrow[tid] = xr;
    }
    __syncthreads();
    const size_t row_bytes = (size_t)(a.k / BlockTraits<T>::QK) * BlockTraits<T>::BYTES;
    const uint32_t tx = tid & 15, ty = tid >> 4;  // tx: weight-row quad, ty: activation-row quad
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    for (uint32_t k0 = 0; k0 < a.k; k0 += 32) {
        for (uint32_t idx = tid; idx < 64 * 32; idx += 256) {
            const uint32_t rr = idx >> 5, kk = idx & 31u;
            float wv = 0.0f, xv = 0.0f;
            if (k0 + kk < a.k) {
                if (r0 + rr < a.n) wv = round_f16(dequant_elem<T>(w + (size_t)(r0 + rr) * row_bytes, k0 + kk));
                if (orow[rr] >= 0) xv = round_f16(a.x[(size_t)xrow[rr] * a.k + k0 + kk]);
            }
            Ws[kk][rr] = wv;
            Xs[kk][rr] = xv;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < 32; kk++) {
            float wv[4], xv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                wv[i] = Ws[kk][tx * 4 + i];
                xv[i] = Xs[kk][ty * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int32_t o = orow[ty * 4 + i];
        if (o < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t col = r0 + tx * 4 + j;
            if (col < a.n) a.y[(size_t)o * a.n + col] = acc[i][j];
        }
    }
}

// =================================================================================================
// routed tile list + activation packing for qmm_tc
// =================================================================================================
// Scratch header written by build_tiles: [0] = number of tiles, [1..] = (expert, row-tile) pairs.
// One CTA of 256 threads: thread i takes expert base + i, a block-wide exclusive prefix sum of the experts' tile
// counts gives each expert its place in the list (experts ascending, row tiles ascending inside an expert).
__global__ void __launch_bounds__(256) build_tiles_kernel(const uint32_t *htpe, uint32_t n_experts, uint32_t nt,
                                                          uint32_t max_tiles, uint32_t *tiles) {
    __shared__ uint32_t warp_tot[8];
    __shared__ uint32_t carry_s;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    if (tid == 0) carry_s = 0;
    __syncthreads();
    for (uint32_t base = 0; base < n_experts; base += 256) {
        const uint32_t e = base + tid;
        const uint32_t cnt = e < n_experts ? (htpe[e] + nt - 1) / nt : 0u;
        uint32_t incl = cnt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= (uint32_t)d) incl += v;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        uint32_t before = carry_s;
        for (uint32_t w = 0; w < warp; w++) before += warp_tot[w];
        uint32_t pos = before + incl - cnt;
        for (uint32_t mt = 0; mt < cnt && pos < max_tiles; mt++, pos++) {
            tiles[1 + 2 * pos] = e;
            tiles[2 + 2 * pos] = mt;
        }
        __syncthreads();
        if (tid == 255) carry_s = before + incl;
        __syncthreads();
    }
    if (tid == 0) tiles[0] = carry_s < max_tiles ? carry_s : max_tiles;
}

// Packs activation rows into f16 tiles of NT rows x 64 columns laid out exactly as the tensor core
// reads a K-major 128-byte-swizzled operand: row r, 16-byte chunk j (8 halves) of a tile lives at
// (r/8)*1024 + (r%8)*128 + ((j ^ (r%8)) * 16).  Tile (t, kc) starts at ((t*nchunks + kc) * NT*128) bytes.
// grid (nchunks, ntile_bound); 256 threads.
template <int NT>
__global__ void __launch_bounds__(256) pack_x_kernel(const QmmArgs a, uint8_t *xpack, uint32_t nchunks, uint32_t zero_y) {
    // grid (K-chunk lanes, tiles): CTA (c, t) packs the chunks c, c + gridDim.x, ... of tile t, so that the tile's
    // routing lookups (a chain of dependent loads) are paid once per CTA, not once per chunk.
    const uint32_t t = blockIdx.y;
    allow_dependents();   // the mat-mat kernel behind may set itself up; it waits for this grid before it reads anything
    if (zero_y) {  // split-K tiles add their halves into y with atomics (dense form only)
        const size_t total = (size_t)a.m * a.n, ncta = (size_t)gridDim.x * gridDim.y, cta = (size_t)t * gridDim.x + blockIdx.x;
        const size_t per = (total + ncta - 1) / ncta, lo = cta * per, hi = lo + per < total ? lo + per : total;
        for (size_t i = lo + threadIdx.x; i < hi; i += 256) a.y[i] = 0.f;
    }
    uint32_t e = 0, mt = t, nrows = a.m;
    if (a.hids) {
        if (t >= a.tiles[0]) return;
        e = a.tiles[1 + 2 * t];
        mt = a.tiles[2 + 2 * t];
        nrows = a.htpe[e];
    }
    constexpr int kPer = (NT * 8 + 255) / 256;   // (row, 16-byte column) pairs per thread: the same ones in every chunk
    const float *src_row[kPer];
#pragma unroll
    for (int i = 0; i < kPer; i++) {
        const uint32_t q = threadIdx.x + i * 256, r = q >> 3;
        const uint32_t row = mt * NT + r;
        src_row[i] = nullptr;
        if (q < NT * 8 && row < nrows) {
            int64_t src = row;
            if (a.hids) {
                const int32_t id = a.hids[(size_t)e * a.hids_stride + row];
                src = (id >= 0 && (uint32_t)id < a.total_rows) ? id / (int32_t)a.top_k : -1;
            }
            // (perm021 form: the pointer only marks the row as present; the element addresses are formed per chunk)
            if (src >= 0) src_row[i] = a.x_bf16 ? reinterpret_cast<const float *>(a.x_bf16) : a.x + (size_t)src * a.k;
        }
    }
    for (uint32_t kc = blockIdx.x; kc < nchunks; kc += gridDim.x) {
        uint8_t *tile = xpack + ((size_t)t * nchunks + kc) * (size_t)(NT * 128);
#pragma unroll
        for (int i = 0; i < kPer; i++) {
            const uint32_t q = threadIdx.x + i * 256;
            if (q >= NT * 8) break;
            const uint32_t r = q >> 3, j = q & 7u;
            const uint32_t k0 = kc * 64 + 8 * j;
            uint4 out = make_uint4(0, 0, 0, 0);
            if (src_row[i] && k0 < a.k) {
                const float *xp = src_row[i] + k0;
                float v[8];
                if (a.x_bf16) {
                    // eight consecutive K values lie inside one head (head_dim is a multiple of 32): 16 bytes of bf16
                    const uint32_t h = k0 / a.head_dim, d0 = k0 - h * a.head_dim, row = mt * NT + r;
                    const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(a.x_bf16 + ((size_t)h * a.m + row) * a.head_dim + d0));
                    const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int u = 0; u < 4; u++) {   // bf16 -> f32 is exact; f32 -> f16 rounds to nearest even below
                        v[2 * u] = __uint_as_float(w4[u] << 16);
                        v[2 * u + 1] = __uint_as_float(w4[u] & 0xFFFF0000u);
                    }
                } else if (k0 + 8 <= a.k && (((uintptr_t)xp) & 15u) == 0) {
                    const float4 lo = __ldg(reinterpret_cast<const float4 *>(xp));
                    const float4 hi = __ldg(reinterpret_cast<const float4 *>(xp) + 1);
                    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
                    v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
                } else {
#pragma unroll
                    for (int u = 0; u < 8; u++) v[u] = (k0 + u < a.k) ? xp[u] : 0.0f;
                }
                if (a.x2) {   // fused SwiGLU: the same expression as the stand-alone kernel, so the same f32 values
                    const float *up = a.x2 + (xp - a.x);
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const float uv = (k0 + u < a.k) ? __ldg(up + u) : 0.0f;
                        v[u] = v[u] / (1.0f + expf(-v[u])) * uv;
                    }
                }
                __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
                __half2 h2 = __floats2half2_rn(v[4], v[5]), h3 = __floats2half2_rn(v[6], v[7]);
                out.x = *reinterpret_cast<uint32_t *>(&h0);
                out.y = *reinterpret_cast<uint32_t *>(&h1);
                out.z = *reinterpret_cast<uint32_t *>(&h2);
                out.w = *reinterpret_cast<uint32_t *>(&h3);
            }
            *reinterpret_cast<uint4 *>(tile + (r >> 3) * 1024 + (r & 7u) * 128 + ((j ^ (r & 7u)) << 4)) = out;
        }
    }
}

// =================================================================================================
// qmm_tc
// =================================================================================================
constexpr int kTcDequantWarps = 16;  // two sets of 8: set s dequantises the K stages with st % 2 == s
constexpr int kTcThreads = (kTcDequantWarps + 4) * 32;  // + activation producer, MMA, weight producer, second MMA warp
constexpr int kTcRowsW = 128;                           // weight rows per tile (UMMA M)

template <int T> struct TcTraits;
template <> struct TcTraits<GT_Q4_0> { static constexpr int KR = 256; };  // raw-stage K extent
template <> struct TcTraits<GT_Q8_0> { static constexpr int KR = 256; };
template <> struct TcTraits<GT_Q6_K> { static constexpr int KR = 256; };
template <> struct TcTraits<GT_Q4_K> { static constexpr int KR = 256; };

__device__ __forceinline__ uint32_t lds32s(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16s(uint32_t addr) {
    uint32_t v;
    asm volatile("{ .reg .u16 t; ld.shared.u16 t, [%1]; cvt.u32.u16 %0, t; }" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ int lds_s8s(uint32_t addr) {
    int v;
    asm volatile("{ .reg .s16 t; ld.shared.s8 t, [%1]; cvt.s32.s16 %0, t; }" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }

// NWORDS logical 32-bit words at a 2-byte-aligned shared address
template <int NWORDS> __device__ __forceinline__ void lds_words_n(uint32_t addr, uint32_t (&out)[NWORDS]) {
    const uint32_t al = addr & ~3u, sh = (addr & 2u) * 8u;
    uint32_t prev = lds32s(al);
#pragma unroll
    for (int j = 0; j < NWORDS; j++) {
        const uint32_t nxt = lds32s(al + 4 * (j + 1));
        out[j] = __funnelshift_rc(prev, nxt, sh);
        prev = nxt;
    }
}
// four bytes (each < 128 after the caller's masking) -> two half2 of (1024 + byte)
__device__ __forceinline__ void bytes_to_h2(uint32_t w, __half2 &lo, __half2 &hi) {
    lo = u32_as_h2(__byte_perm(w, 0x64646464u, 0x4140));
    hi = u32_as_h2(__byte_perm(w, 0x64646464u, 0x4342));
}

// Thirty-two consecutive elements [e, e+32) (e a multiple of 32) of one weight row segment in shared
// memory -> four 16-byte groups of eight f16 values, each the exact product rounded once (RNE).
template <int T> __device__ __forceinline__ void dequant32(uint32_t seg, uint32_t e, uint4 (&out)[4]) {
    if constexpr (T == GT_Q4_0) {
        const uint32_t o = seg + 18u * (e >> 5);
        const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)lds16s(o)));
        const __half2 off = __float2half2_rn(1032.0f);  // 1024 + 8
        uint32_t q[4];
        lds_words_n<4>(o + 2, q);
#pragma unroll
        for (int j = 0; j < 4; j++) {  // j = 0,1: low nibbles of bytes 0-7, 8-15; j = 2,3: high nibbles
            const uint32_t w0 = ((j & 2) ? (q[2 * (j & 1)] >> 4) : q[2 * (j & 1)]) & 0x0F0F0F0Fu;
            const uint32_t w1 = ((j & 2) ? (q[2 * (j & 1) + 1] >> 4) : q[2 * (j & 1) + 1]) & 0x0F0F0F0Fu;
            __half2 a, b, cc, dd;
            bytes_to_h2(w0, a, b);
            bytes_to_h2(w1, cc, dd);
            out[j].x = h2_as_u32(__hmul2(__hsub2(a, off), d2));
            out[j].y = h2_as_u32(__hmul2(__hsub2(b, off), d2));
            out[j].z = h2_as_u32(__hmul2(__hsub2(cc, off), d2));
            out[j].w = h2_as_u32(__hmul2(__hsub2(dd, off), d2));
        }
    } else if constexpr (T == GT_Q8_0) {
        const uint32_t o = seg + 34u * (e >> 5);
        const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)lds16s(o)));
        const __half2 off = __float2half2_rn(1152.0f);  // 1024 + 128
        uint32_t q[8];
        lds_words_n<8>(o + 2, q);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            __half2 a, b, cc, dd;
            bytes_to_h2(q[2 * j] ^ 0x80808080u, a, b);
            bytes_to_h2(q[2 * j + 1] ^ 0x80808080u, cc, dd);
            out[j].x = h2_as_u32(__hmul2(__hsub2(a, off), d2));
            out[j].y = h2_as_u32(__hmul2(__hsub2(b, off), d2));
            out[j].z = h2_as_u32(__hmul2(__hsub2(cc, off), d2));
            out[j].w = h2_as_u32(__hmul2(__hsub2(dd, off), d2));
        }
    } else if constexpr (T == GT_Q4_K) {
        // sub-block j of the 144-byte super-block: 32 nibbles of the bytes 16 + 32 (j / 2) ..., low for even j;
        // value = (d sc) q - (dmin m) (src/gguf/mod.rs:582-644), formed in f32 and rounded to f16 once
        const uint32_t o = seg + 144u * (e >> 8);
        const uint32_t j = (e & 255u) >> 5;
        const uint32_t dd = lds16s(o) | (lds16s(o + 2) << 16);
        uint32_t sw[3];
        lds_words_n<3>(o + 4, sw);                      // scales[0..11]
        uint32_t sc, mn;
        if (j < 4) {
            sc = (sw[0] >> (8 * j)) & 63u;
            mn = (sw[1] >> (8 * j)) & 63u;
        } else {
            const uint32_t sh = 8 * (j - 4);
            sc = ((sw[2] >> sh) & 15u) | ((((sw[0] >> sh) >> 6) & 3u) << 4);
            mn = (((sw[2] >> sh) >> 4) & 15u) | ((((sw[1] >> sh) >> 6) & 3u) << 4);
        }
        const float ds = half_bits_to_float(dd & 0xFFFFu) * (float)sc;
        const float dm = half_bits_to_float(dd >> 16) * (float)mn;
        const float c = fmaf(-128.0f, ds, -dm);
        uint32_t Q[8];
        lds_words_n<8>(o + 16 + 32 * (j >> 1), Q);
        const uint32_t ash = (j & 1u) ? 4u : 0u;
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            uint32_t res[4];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const uint32_t u = (Q[2 * jj + i] >> ash) & 0x0F0F0F0Fu;
                // 128 + u spliced into an f32 mantissa; fma(128 + u, ds, -128 ds - dm) = ds u - dm
                const float f0 = fmaf(__uint_as_float(__byte_perm(u, 0x43000000u, 0x7044)), ds, c);
                const float f1 = fmaf(__uint_as_float(__byte_perm(u, 0x43000000u, 0x7144)), ds, c);
                const float f2 = fmaf(__uint_as_float(__byte_perm(u, 0x43000000u, 0x7244)), ds, c);
                const float f3 = fmaf(__uint_as_float(__byte_perm(u, 0x43000000u, 0x7344)), ds, c);
                res[2 * i] = h2_as_u32(__floats2half2_rn(f0, f1));
                res[2 * i + 1] = h2_as_u32(__floats2half2_rn(f2, f3));
            }
            out[jj] = make_uint4(res[0], res[1], res[2], res[3]);
        }
    } else {
        const uint32_t o = seg + 210u * (e >> 8);
        const uint32_t r = e & 255u, h = r >> 7, g = (r & 127u) >> 5;
        uint32_t A[8], H[8];
        lds_words_n<8>(o + 64 * h + 32 * (g & 1u), A);
        lds_words_n<8>(o + 128 + 32 * h, H);
        const float d = half_bits_to_float(lds16s(o + 208));
        const float ds0 = d * (float)lds_s8s(o + 192 + 8 * h + 2 * g);
        const float ds1 = d * (float)lds_s8s(o + 192 + 8 * h + 2 * g + 1);
        const uint32_t hsh = 2 * g, ash = (g & 2u) ? 4u : 0u;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float ds = j < 2 ? ds0 : ds1;
            const float c = -160.0f * ds;  // exact: ds has <= 18 significant bits
            uint32_t res[4];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const uint32_t u = ((A[2 * j + i] >> ash) & 0x0F0F0F0Fu) | (((H[2 * j + i] >> hsh) & 0x03030303u) << 4);
                // 128 + u spliced into an f32 mantissa; fma(128+u, ds, -160 ds) = ds*(u-32) exactly
                const float f0 = fmaf(__uint_as_float(__byte_perm(u, 0x43000000u, 0x7044)), ds, c);
                const float f1 = fmaf(__uint_as_float(__byte_perm(u, 0x43000000u, 0x7144)), ds, c);
                const float f2 = fmaf(__uint_as_float(__byte_perm(u, 0x43000000u, 0x7244)), ds, c);
                const float f3 = fmaf(__uint_as_float(__byte_perm(u, 0x43000000u, 0x7344)), ds, c);
                res[2 * i] = h2_as_u32(__floats2half2_rn(f0, f1));
                res[2 * i + 1] = h2_as_u32(__floats2half2_rn(f2, f3));
            }
            out[j] = make_uint4(res[0], res[1], res[2], res[3]);
        }
    }
}

// ---- rows that start on 16-byte boundaries: 16-byte shared loads at compile-time offsets ----------------------
// The generic routines above read the raw rows with 32-bit loads at 2-byte granular addresses; with rows an odd
// multiple of 16 bytes apart those are 4-way bank-conflicted (two thirds of the kernel's shared-memory wavefronts).
// When every weight row starts on a 16-byte boundary and the raw stage is a whole number of 16-byte units per row
// (k % 256 == 0), each thread's 64 elements sit at a compile-time byte offset of the row's stage, so they can
// be fetched with conflict-free 16-byte loads and static funnel shifts.
__device__ __forceinline__ void q4_0_block_to_h(uint32_t dbits, const uint32_t (&q)[4], uint32_t *out /*16 words*/) {
    const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)dbits));
    const __half2 off = __float2half2_rn(1032.0f);  // 1024 + 8
#pragma unroll
    for (int j = 0; j < 4; j++) {  // j = 0,1: low nibbles of bytes 0-7, 8-15; j = 2,3: high nibbles
        const uint32_t w0 = ((j & 2) ? (q[2 * (j & 1)] >> 4) : q[2 * (j & 1)]) & 0x0F0F0F0Fu;
        const uint32_t w1 = ((j & 2) ? (q[2 * (j & 1) + 1] >> 4) : q[2 * (j & 1) + 1]) & 0x0F0F0F0Fu;
        __half2 a, b, cc, dd;
        bytes_to_h2(w0, a, b);
        bytes_to_h2(w1, cc, dd);
        out[4 * j + 0] = h2_as_u32(__hmul2(__hsub2(a, off), d2));
        out[4 * j + 1] = h2_as_u32(__hmul2(__hsub2(b, off), d2));
        out[4 * j + 2] = h2_as_u32(__hmul2(__hsub2(cc, off), d2));
        out[4 * j + 3] = h2_as_u32(__hmul2(__hsub2(dd, off), d2));
    }
}
__device__ __forceinline__ void q8_0_block_to_h(uint32_t dbits, const uint32_t (&q)[8], uint32_t *out /*16 words*/) {
    const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)dbits));
    const __half2 off = __float2half2_rn(1152.0f);  // 1024 + 128
#pragma unroll
    for (int j = 0; j < 8; j++) {
        __half2 a, b;
        bytes_to_h2(q[j] ^ 0x80808080u, a, b);
        out[2 * j + 0] = h2_as_u32(__hmul2(__hsub2(a, off), d2));
        out[2 * j + 1] = h2_as_u32(__hmul2(__hsub2(b, off), d2));
    }
}
// Quarter S4 (64 elements = 2 blocks) of a row's 256-wide raw stage at the 16-byte aligned shared address `unit`.
template <int T, int S4> __device__ __forceinline__ void dequant64_aligned(uint32_t unit, uint32_t (&r)[32]) {
    constexpr int SUB = 2 * BlockTraits<T>::BYTES;   // bytes of two blocks
    constexpr int c0 = (SUB * S4) >> 4;              // first 16-byte chunk touched
    constexpr int wo = ((SUB * S4) & 15) >> 2;       // word offset inside it (SUB * S4 is a multiple of 4)
    if constexpr (T == GT_Q4_0) {
        uint32_t W[12];
#pragma unroll
        for (int i = 0; i < 3; i++) lds128(unit + 16 * (c0 + i), W[4 * i], W[4 * i + 1], W[4 * i + 2], W[4 * i + 3]);
        uint32_t q0[4], q1[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            q0[i] = __funnelshift_r(W[wo + i], W[wo + i + 1], 16);  // block 0's codes start 2 bytes into a word
            q1[i] = W[wo + 5 + i];                                  // block 1's are word aligned
        }
        q4_0_block_to_h(W[wo] & 0xFFFFu, q0, r);
        q4_0_block_to_h(W[wo + 4] >> 16, q1, r + 16);
    } else {
        uint32_t W[20];
#pragma unroll
        for (int i = 0; i < 5; i++) lds128(unit + 16 * (c0 + i), W[4 * i], W[4 * i + 1], W[4 * i + 2], W[4 * i + 3]);
        uint32_t q0[8], q1[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            q0[i] = __funnelshift_r(W[wo + i], W[wo + i + 1], 16);
            q1[i] = W[wo + 9 + i];
        }
        q8_0_block_to_h(W[wo] & 0xFFFFu, q0, r);
        q8_0_block_to_h(W[wo + 8] >> 16, q1, r + 16);
    }
}
// Q6_K: the 32-element run (h, g) of the super-block that starts PRE bytes into the row's aligned stage.
template <int PRE> __device__ __forceinline__ void dequant32_q6k_aligned(uint32_t stage_row, uint32_t h, uint32_t g, uint32_t *out) {
    uint32_t A[8], H[8];
    lds_field<PRE, 8>(stage_row + 64 * h + 32 * (g & 1u), A);
    lds_field<PRE, 8>(stage_row + 128 + 32 * h, H);
    const float d = half_bits_to_float(lds_u16(stage_row + PRE + 208));
    const float ds0 = d * (float)lds_s8(stage_row + PRE + 192 + 8 * h + 2 * g);
    const float ds1 = d * (float)lds_s8(stage_row + PRE + 192 + 8 * h + 2 * g + 1);
    const uint32_t hsh = 2 * g, ash = (g & 2u) ? 4u : 0u;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float ds = j < 2 ? ds0 : ds1;
        const float c = -160.0f * ds;  // exact: ds has <= 18 significant bits
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const uint32_t u = ((A[2 * j + i] >> ash) & 0x0F0F0F0Fu) | (((H[2 * j + i] >> hsh) & 0x03030303u) << 4);
            const float f0 = fmaf(__uint_as_float(__byte_perm(u, 0x43000000u, 0x7044)), ds, c);
            const float f1 = fmaf(__uint_as_float(__byte_perm(u, 0x43000000u, 0x7144)), ds, c);
            const float f2 = fmaf(__uint_as_float(__byte_perm(u, 0x43000000u, 0x7244)), ds, c);
            const float f3 = fmaf(__uint_as_float(__byte_perm(u, 0x43000000u, 0x7344)), ds, c);
            out[4 * j + 2 * i] = h2_as_u32(__floats2half2_rn(f0, f1));
            out[4 * j + 2 * i + 1] = h2_as_u32(__floats2half2_rn(f2, f3));
        }
    }
}
__device__ __forceinline__ void dequant32_q6k_aligned_p(uint32_t p8, uint32_t stage_row, uint32_t h, uint32_t g, uint32_t *out) {
    switch (p8) {  // uniform over the CTA
    case 0: dequant32_q6k_aligned<0>(stage_row, h, g, out); break;
    case 1: dequant32_q6k_aligned<2>(stage_row, h, g, out); break;
    case 2: dequant32_q6k_aligned<4>(stage_row, h, g, out); break;
    case 3: dequant32_q6k_aligned<6>(stage_row, h, g, out); break;
    case 4: dequant32_q6k_aligned<8>(stage_row, h, g, out); break;
    case 5: dequant32_q6k_aligned<10>(stage_row, h, g, out); break;
    case 6: dequant32_q6k_aligned<12>(stage_row, h, g, out); break;
    default: dequant32_q6k_aligned<14>(stage_row, h, g, out); break;
    }
}

// position in a ring of `stages` slots plus the phase bit of the slot's current use (no divisions)
struct RingPos {
    uint32_t s = 0, ph = 0;
    __device__ __forceinline__ void adv(uint32_t n, uint32_t stages) {
        s += n;
        while (s >= stages) {
            s -= stages;
            ph ^= 1u;
        }
    }
};

struct TcCfg {
    uint32_t nchunks;     // ceil(k / 64)
    uint32_t b_stages;    // depth of the activation ring, in 64-wide K chunks
    uint32_t seg_stride;  // bytes reserved per raw row segment
    uint32_t b_off, raw_off;
    uint32_t raw_slots;   // depth of the raw weight ring (2..6)
    uint32_t aligned;     // every weight row starts on a 16-byte boundary and k % 256 == 0: static-offset 16-byte raw reads
    uint32_t debug;       // experiment switches: 1 = skip dequantisation, 2 = skip raw copies, 4 = skip MMA, 8 = skip B copies
    uint32_t n_wt;        // weight-row tiles, ceil(n / 128)
    uint32_t ntiles;      // activation tiles: the count (dense) or its bound (routed: the list's length is read on the device)
    uint32_t ksplit;      // K split factor (1 or 2)
    uint32_t stage_off;   // byte offset of the two staged output tiles (narrow tiles only), 0 = write y straight from registers
    uint32_t raw_tma;     // raw weight stages arrive as one tensor copy each (needs `aligned`); otherwise 16-byte cp.async
};

// ring of dequantised weight stages held in tensor memory: the columns the accumulators leave free.  Tiles of 64
// activation rows (two 64-column accumulators) keep six stages in columns [128, 512), wider ones four in [256, 512):
// the ring's depth over the latency of the loop dequantise -> MMA -> commit -> reuse is what bounds a narrow tile.
template <int NT> struct TcRing {
    static constexpr int kStages = NT <= 64 ? 6 : 4;
    static constexpr int kColBase = NT <= 64 ? 128 : 256;
};
constexpr int kTcACols = 64;       // one stage: 128 K values as f16 pairs = 64 32-bit columns
constexpr int kTcTmemCols = 512;

// grid = min(work items, SMs) persistent CTAs; kTcThreads threads; 1 CTA per SM.
//
// Data flow per work item (one 128-row weight tile x one NT-row activation tile, all of K or one K split):
//   raw GGML blocks  --cp.async-->  shared-memory ring  --dequantise (16 warps)-->  f16 pairs in registers
//   --tcgen05.st-->  tensor-memory ring (A operand)  --tcgen05.mma, B = packed activations from the bulk-copy
//   ring in shared memory-->  f32 accumulator in tensor memory  --tcgen05.ld-->  y.
// The dequantised weights never touch shared memory: its bandwidth is the scarce resource here (the tensor
// core already reads the whole activation tile from it for every MMA).
template <int T, int NT, bool SH>
__global__ void __launch_bounds__(kTcThreads, 1) qmm_tc_kernel(const QmmArgs a, const TcCfg c, const uint8_t *xpack,
                                                                const __grid_constant__ CUtensorMap wmap) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // tensor-core operand tiles need 1024-byte alignment (128-byte swizzle atoms): align by hand
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int QK = BlockTraits<T>::QK, BB = BlockTraits<T>::BYTES, KR = TcTraits<T>::KR;
    constexpr int kMaxB = 8, kMaxRaw = 6;
    constexpr int kTcAStages = TcRing<NT>::kStages, kTcAColBase = TcRing<NT>::kColBase;
    static_assert(kMaxB / 2 <= kTcAStages, "an activation chunk's place is freed by a stage_done phase the producer can still see");
    constexpr int kNumMma = NT <= 128 ? 2 : 1;   // issuing threads, each with its own accumulator
    __shared__ __align__(8) uint64_t a_full[kTcAStages], stage_done[kTcAStages], b_full[kMaxB];
    __shared__ __align__(8) uint64_t raw_full[kMaxRaw], raw_empty[kMaxRaw], acc_full, acc_empty, orow_ready[2], stage_ready[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile uint32_t abort_flag;
    __shared__ int32_t orow[2][NT];
    // SH (row-sharded result): the peers' result buffers, copied out of the parameter block once.  The plain form is a
    // separate instantiation: the peer stores' presence alone cost it 15 % (indexed reads of the parameter block).
    __shared__ float *peer_y[SH ? 7 : 1];

    // Warps 0-3 are the four single-thread roles (one per scheduler partition, and the lowest warp numbers, so that
    // they are served before the dequantising warps whenever both have an instruction ready: these threads are the
    // critical path and lose hundreds of cycles per K stage otherwise); warps 4-19 dequantise.
    constexpr uint32_t kWarpActs = 0, kWarpMma0 = 1, kWarpWeights = 2, kWarpMma1 = 3, kCtrlWarps = 4;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t tid = threadIdx.x - kCtrlWarps * 32;   // index among the dequantising threads (wraps for warps 0-3)
    const uint32_t row_bytes = (a.k / QK) * BB;

    // ---- set-up that needs nothing from the kernels ahead in the stream (it overlaps their tail: the kernel is
    // ---- launched with programmatic stream serialisation), then the wait for them
    if (threadIdx.x == 0) {
        abort_flag = 0;
        if constexpr (SH) {
            peer_y[0] = a.y_peer[0]; peer_y[1] = a.y_peer[1]; peer_y[2] = a.y_peer[2]; peer_y[3] = a.y_peer[3];
            peer_y[4] = a.y_peer[4]; peer_y[5] = a.y_peer[5]; peer_y[6] = a.y_peer[6];
        }
        for (uint32_t s = 0; s < kTcAStages; s++) {
            mbar_init(&a_full[s], kTcDequantWarps / 2);  // the eight warps of one set
            mbar_init(&stage_done[s], 1);
        }
        for (uint32_t s = 0; s < c.b_stages; s++) mbar_init(&b_full[s], 1);
        for (uint32_t s = 0; s < c.raw_slots; s++) {
            // one asynchronous arrival per copying thread, or the weight producer's single arrival with the byte count
            mbar_init(&raw_full[s], c.raw_tma ? 1u : kTcDequantWarps * 32);
            mbar_init(&raw_empty[s], kTcDequantWarps);
        }
        mbar_init(&acc_full, kNumMma);
        mbar_init(&acc_empty, kTcDequantWarps);
        for (int s = 0; s < 2; s++) {
            mbar_init(&orow_ready[s], kTcDequantWarps);
            mbar_init(&stage_ready[s], kTcDequantWarps);
        }
        mbar_init_fence();
    }
    if (warp == kWarpMma0) {  // the first MMA warp owns tensor memory
        tmem_alloc(&tmem_base_s, kTcTmemCols);
        tmem_relinquish();
    }
    grid_dependency_wait();   // the packed activations, the tile list and (split-K) the zeroed y are complete
    allow_dependents();

    // ---- work items: (weight-row tile, K split, token tile), weight tile fastest; CTA b takes items b, b + grid, ...
    // Every role walks the same item sequence; ring slots and barrier phases run on across items, so the next
    // item's weights are already on their way while this item's accumulator is read back.
    const uint32_t n_tt = a.hids ? min(a.tiles[0], c.ntiles) : c.ntiles;   // uniform for the whole CTA
    const uint32_t total_items = c.n_wt * c.ksplit * n_tt;
    const uint32_t nraw_all = (a.k + KR - 1) / KR;
    struct Item {
        uint32_t tt, e, mt, n0, r_lo, nraw, nst, nck, kc_lo;
        const uint8_t *wbase;
    };
    // routed: the (expert, row tile) pairs of the CTA's first items, fetched once (a lookup per item would put a
    // global-memory round trip in front of every role's start on the item)
    constexpr uint32_t kMetaItems = 32;
    __shared__ uint32_t meta[kMetaItems][2];
    if (a.hids && threadIdx.x < kMetaItems) {
        const uint32_t item = blockIdx.x + threadIdx.x * gridDim.x;
        if (item < total_items) {
            const uint32_t tt = item / (c.n_wt * c.ksplit);
            meta[threadIdx.x][0] = a.tiles[1 + 2 * tt];
            meta[threadIdx.x][1] = a.tiles[2 + 2 * tt];
        }
    }
    auto load_item = [&](uint32_t item) -> Item {
        Item it;
        const uint32_t rest = item / c.n_wt, wt = item - rest * c.n_wt;
        const uint32_t z = c.ksplit == 1 ? 0u : rest % c.ksplit;
        it.tt = c.ksplit == 1 ? rest : rest / c.ksplit;
        it.e = 0;
        it.mt = it.tt;
        if (a.hids) {
            const uint32_t li = (item - blockIdx.x) / gridDim.x;   // the CTA's li-th item
            if (li < kMetaItems) {
                it.e = meta[li][0];
                it.mt = meta[li][1];
            } else {
                it.e = a.tiles[1 + 2 * it.tt];
                it.mt = a.tiles[2 + 2 * it.tt];
            }
        }
        it.wbase = a.w + (size_t)it.e * a.expert_stride;
        it.n0 = wt * kTcRowsW;
        // split-K: this item takes the raw stages [r_lo, r_hi) of K and adds its part of the tile into y
        it.r_lo = c.ksplit == 1 ? 0u : (z * nraw_all) / c.ksplit;   // (ksplit <= 2 and nraw_all < 2^24: no overflow)
        const uint32_t r_hi = c.ksplit == 1 ? nraw_all : ((z + 1) * nraw_all) / c.ksplit;
        it.nraw = r_hi - it.r_lo;
        it.kc_lo = it.r_lo * (KR / 64);
        it.nst = min((a.k + 127) / 128, r_hi * (KR / 128)) - it.r_lo * (KR / 128);   // tensor-memory stages
        it.nck = min(c.nchunks, r_hi * (KR / 64)) - it.kc_lo;                         // 64-wide activation chunks
        return it;
    };

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = tmem_base_s;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t b_bytes = NT * 128;                 // one 64-wide K chunk of the activation tile
    const uint32_t raw_stage_bytes = kTcRowsW * c.seg_stride;
    // wait styles: the single producer / MMA warps spin (they are the critical path and cost one warp's issue
    // slots); the dequantising warps space their polls out
    const uint32_t wmode_cr = (MLXN_DBG(c) & 32u) ? 0u : 0xFFFFFFFFu;
    const uint32_t wmode_dq = (MLXN_DBG(c) & 16u) ? 0xFFFFFFFFu : 0u;
#ifdef MLXN_TC_TRACE
    // experiment: CTA 0 logs (event, clock) pairs into y (use with debug 256, which keeps the epilogue from writing y)
    uint32_t trace_n = 0;
    auto TRACE = [&](uint32_t role, uint32_t code, uint32_t x) {
        if ((MLXN_DBG(c) & 512u) && blockIdx.x == 0 && lane == 0 && trace_n < 500) {
            uint32_t *t = reinterpret_cast<uint32_t *>(a.y) + role * 1024 + 2 * trace_n;
            t[0] = (code << 16) | (x & 0xFFFFu);
            t[1] = (uint32_t)clock64();
            trace_n++;
        }
    };
#else
#define TRACE(role, code, x) ((void)0)
#endif

    if (warp == kWarpActs) {
        // ======================= producer warp: bulk copies of the packed activation tiles =======================
        // Every K stage owns two consecutive chunk slots of the ring (a K tail of 64 leaves its second one empty;
        // the producer still arrives on it so that the slot's phase moves on).  Chunk slot G reuses the place of
        // chunk slot G - b_stages, which belonged to K stage (G - b_stages) / 2: free once that stage's MMAs have
        // completed (stage_done, the same barrier the dequantising warps wait on before they overwrite the stage's
        // weights in tensor memory).  G and the stage numbers count on across items.
        if (lane == 0) {
            uint32_t s = 0, G = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
                const Item it = load_item(item);
                for (uint32_t kc = 0; kc < 2 * it.nst; kc++, G++) {
                    if (G >= c.b_stages) {
                        const uint32_t j = (G - c.b_stages) >> 1;
                        if (!mbar_wait(&stage_done[j % kTcAStages], (j / kTcAStages) & 1u, &abort_flag, a.status,
                                       ST_WAIT_EMPTY_TIMEOUT, wmode_cr)) {
                            ok = false;
                            break;
                        }
                    }
                    if (kc >= it.nck || (MLXN_DBG(c) & 8u)) {
                        mbar_arrive(&b_full[s]);
                    } else {
                        mbar_expect_tx(&b_full[s], b_bytes);
                        bulk_g2s(smem + c.b_off + s * b_bytes,
                                 xpack + ((size_t)it.tt * c.nchunks + it.kc_lo + kc) * (size_t)b_bytes, b_bytes, &b_full[s]);
                    }
                    if (++s == c.b_stages) s = 0;
                }
            }
        }
    } else if (warp == kWarpWeights) {
        // ======================= weight producer warp: one tensor copy per raw stage =======================
        // The weights as a 3-D tensor of 32-bit words [expert][row][row_bytes / 4]; a raw stage is the box
        // (1, 128 rows, seg_stride / 4 words) at the stage's K offset, rounded down to 16 bytes for Q6_K
        // (210-byte super-blocks; readers skip the lead-in).  Rows past n arrive as zeros.  The copies run
        // raw_slots - 1 stages ahead of the dequantisation, across item boundaries.
        if (c.raw_tma && lane == 0) {
            const uint32_t R = c.raw_slots;
            uint32_t slot = 0, ph = 0, requested = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
                const Item it = load_item(item);
                for (uint32_t r = 0; r < it.nraw; r++, requested++) {
                    if (requested >= R &&
                        !mbar_wait(&raw_empty[slot], ph ^ 1u, &abort_flag, a.status, ST_WAIT_EMPTY_TIMEOUT, wmode_cr)) {
                        ok = false;
                        break;
                    }
                    TRACE(0, 1, requested);
                    const uint32_t kb = ((it.r_lo + r) * (KR / QK) * BB) & ~15u;   // byte offset of the stage in the row
                    mbar_expect_tx(&raw_full[slot], raw_stage_bytes);
                    asm volatile(
                        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                        ::"r"(smem_base + c.raw_off + slot * raw_stage_bytes), "l"(&wmap), "r"(kb >> 2), "r"(it.n0), "r"(it.e),
                          "r"(smem_u32(&raw_full[slot]))
                        : "memory");
                    if (++slot == R) { slot = 0; ph ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == kWarpMma0 || warp == kWarpMma1) {
        // ======================= MMA warps: one thread each issues tcgen05.mma =======================
        // A lone thread gets through one of these instructions (MMA, commit, barrier test) every 50-100 cycles, and
        // a K stage costs about thirteen of them, which bounds a narrow tile (NT <= 128: the MMAs themselves are
        // short) well before the tensor core does.  So narrow tiles use two issuing threads: thread w takes the K
        // stages st with st % 2 == w and accumulates them in its own accumulator (columns [w NT, (w+1) NT)); the
        // epilogue adds the two.  NT = 256 keeps one thread (tensor memory has no room for a second accumulator,
        // and there the MMAs are long enough to hide the issue).
        const uint32_t w = warp == kWarpMma0 ? 0u : 1u;
        if (lane == 0 && w < (uint32_t)kNumMma) {
            constexpr uint32_t idesc = umma_idesc_f16(kTcRowsW, NT);
            const uint64_t bd0 = umma_desc_k_sw128(smem_base + c.b_off);
            const uint64_t b_step = b_bytes >> 4;  // descriptor address field is in 16-byte units
            const bool do_mma = !(MLXN_DBG(c) & 4u);
            const uint32_t d_col = tmem_d + w * NT;
            uint32_t sa = 0, aph = 0, sb = 0, bph = 0, nitem = 0;   // ring positions of the stage being looked at
            bool ok = true;
            for (uint32_t item = blockIdx.x; ok && item < total_items; item += gridDim.x, nitem++) {
                const Item it = load_item(item);
                // the accumulators of the item before have been read back
                if (nitem > 0 &&
                    !mbar_wait(&acc_empty, (nitem - 1) & 1u, &abort_flag, a.status, ST_WAIT_EMPTY_TIMEOUT, wmode_cr))
                    break;
                tc_fence_after();
                TRACE(1 + 3 * w, 1, nitem);
                bool issued = false;
                for (uint32_t st = 0; st < it.nst; st++) {
                    if ((st & (uint32_t)(kNumMma - 1)) == w) {
                        if (!mbar_wait(&a_full[sa], aph, &abort_flag, a.status, ST_WAIT_FULL_TIMEOUT, wmode_cr)) { ok = false; break; }
                        TRACE(1 + 3 * w, 2, st);
                        if (!mbar_wait(&b_full[sb], bph, &abort_flag, a.status, ST_WAIT_FULL_TIMEOUT, wmode_cr)) { ok = false; break; }
                        tc_fence_after();
                        TRACE(1 + 3 * w, 4, st);
                        const uint32_t a_col = tmem_d + kTcAColBase + sa * kTcACols;
                        const uint64_t bd = bd0 + sb * b_step;
                        if (do_mma) {
                            umma_f16_ts(d_col, a_col, bd, idesc, issued ? 1u : 0u);
                            umma_f16_ts(d_col, a_col + 8, bd + 2, idesc, 1u);
                            umma_f16_ts(d_col, a_col + 16, bd + 4, idesc, 1u);
                            umma_f16_ts(d_col, a_col + 24, bd + 6, idesc, 1u);
                        }
                        issued = true;
                        if (2 * st + 1 < it.nck) {
                            const uint32_t sb1 = sb + 1 == c.b_stages ? 0u : sb + 1;
                            const uint32_t bph1 = sb + 1 == c.b_stages ? bph ^ 1u : bph;
                            if (!mbar_wait(&b_full[sb1], bph1, &abort_flag, a.status, ST_WAIT_FULL_TIMEOUT, wmode_cr)) { ok = false; break; }
                            const uint64_t bd1 = bd0 + sb1 * b_step;
                            if (do_mma) {
                                umma_f16_ts(d_col, a_col + 32, bd1, idesc, 1u);
                                umma_f16_ts(d_col, a_col + 40, bd1 + 2, idesc, 1u);
                                umma_f16_ts(d_col, a_col + 48, bd1 + 4, idesc, 1u);
                                umma_f16_ts(d_col, a_col + 56, bd1 + 6, idesc, 1u);
                            }
                        }
                        TRACE(1 + 3 * w, 5, st);
                        umma_commit(&stage_done[sa]);  // frees the stage's weights and its two activation chunks
                        TRACE(1 + 3 * w, 3, st);
                    }
                    // on to the next stage's ring places (two activation chunk slots per stage, used or not)
                    sb += 2;
                    if (sb >= c.b_stages) { sb -= c.b_stages; bph ^= 1u; }
                    if (++sa == kTcAStages) { sa = 0; aph ^= 1u; }
                }
                if (!ok) break;
                // this thread's share of the item is issued: its accumulator is complete when these MMAs are
                if (issued) umma_commit(&acc_full);
                else mbar_arrive(&acc_full);
            }
        }
        __syncwarp();
    } else {
        // ======================= dequantise warps, then epilogue =======================
        // The 16 warps form two sets of 8; set s fills the K stages st with st % 2 == s, so that a warp has two
        // stage times for each of its turns.  Within a set, thread (warp w, lane l) owns weight row
        // 32 (w % 4) + l of the tile -- the tensor-memory lane its warp may address -- and the 64-element half
        // (w / 4) % 2 of the stage: thirty-two packed f16 pairs = one 32-column store.
        const uint32_t dw = warp - kCtrlWarps;   // 0..15
        const uint32_t q4 = dw & 3u, half = (dw >> 2) & 1u, set = dw >> 3;
        const uint32_t rr = q4 * 32 + lane;
        // Raw weight rows are short (144..272 bytes per stage and row), too short for one bulk copy each to be
        // efficient, so all dequantising threads stream them as 16-byte cp.async chunks, a few raw stages ahead
        // of the one being dequantised.  Each row is fetched as the 16-byte aligned superset of its (only
        // 2-byte aligned) segment; readers skip the lead-in bytes.
        // The (row, 16-byte chunk) pairs a thread copies are the same in every raw stage and every item; per item
        // only the rows' base addresses change, per stage only the K offset.
        constexpr int kRawSlots = 5;            // (128 rows x at most 19 chunks) / 512 threads, rounded up
        constexpr uint32_t kSegFull = (KR / QK) * BB;
        constexpr uint32_t kCmax = (kSegFull + 30u) >> 4;  // most 16-byte chunks a row segment can need
        static_assert(kTcRowsW * kCmax <= kRawSlots * kTcDequantWarps * 32, "raw copy slots");
        static_assert(KR == 256, "a raw stage feeds one K stage of each set");
        const uint8_t *slot_src[kRawSlots];     // start of the thread's row (global), for the item being requested
        uint32_t slot_dst[kRawSlots];           // row's place inside a raw stage + chunk offset (shared, relative)
        uint32_t slot_cc[kRawSlots];            // chunk index within the row, 0xFFFFFFFF = unused in this item
        // request cursor: runs ahead of the dequantisation, across item boundaries
        uint32_t q_item = blockIdx.x, q_r = 0, q_nraw = 0, q_rlo = 0;
        auto open_request_item = [&]() {
            const Item it = load_item(q_item);
            const uint32_t rows_here = min((uint32_t)kTcRowsW, a.n - it.n0);
#pragma unroll
            for (int i = 0; i < kRawSlots; i++) {
                const uint32_t idx = tid + i * (kTcDequantWarps * 32);
                const uint32_t row = idx / kCmax, cc = idx - row * kCmax;
                const bool used = row < rows_here;
                slot_src[i] = it.wbase + (size_t)(it.n0 + (used ? row : 0)) * row_bytes;
                slot_dst[i] = row * c.seg_stride + cc * 16u;
                slot_cc[i] = used ? cc : 0xFFFFFFFFu;
            }
            q_r = 0;
            q_nraw = it.nraw;
            q_rlo = it.r_lo;
        };
        if (!c.raw_tma && q_item < total_items) open_request_item();
        auto issue_raw = [&](uint32_t r, uint32_t slot) {
            const uint32_t k0 = r * KR;
            const uint32_t seg_bytes = (min((uint32_t)KR, a.k - k0) / QK) * BB;
            const uint32_t koff = (k0 / QK) * BB;
            const uint32_t dst0 = smem_base + c.raw_off + slot * raw_stage_bytes;
#pragma unroll
            for (int i = 0; i < kRawSlots; i++) {
                const uint8_t *src = slot_src[i] + koff;
                const uint32_t pre_b = (uint32_t)((uintptr_t)src & 15u);
                if (slot_cc[i] != 0xFFFFFFFFu && slot_cc[i] * 16u < pre_b + seg_bytes && !(MLXN_DBG(c) & 2u))
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + slot_dst[i]),
                                 "l"(src - pre_b + slot_cc[i] * 16u)
                                 : "memory");
            }
            // the thread's arrival on the slot's barrier fires once its copies have landed; nobody blocks on it
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&raw_full[slot])) : "memory");
        };
        // raw ring: a stage is requested raw_slots-1 stages before it is read; slots and phases count on across items
        const uint32_t R = c.raw_slots, D = R - 1;
        uint32_t islot = 0, iph = 0;   // slot / use-parity of the next stage to request
        uint32_t requested = 0, consumed = 0;
        uint32_t rs = 0, rph = 0;      // slot / parity of the raw stage being read
        uint32_t J0 = 0;               // K stages of the items before this one (tensor-memory ring position)
        uint32_t nitem = 0;
        bool ok = true;
        const uint32_t a_dst = tmem_d + ((q4 * 32) << 16) + kTcAColBase + 32 * half;
        const uint32_t g = dw >> 2;
        for (uint32_t item = blockIdx.x; ok && item < total_items; item += gridDim.x, nitem++) {
            const Item it = load_item(item);
            const uint32_t n0 = it.n0;
            const bool row_ok = n0 + rr < a.n;
            const uint32_t row_lo4 = (uint32_t)((uintptr_t)(it.wbase + (size_t)(n0 + rr) * row_bytes) & 15u);
            // the item's output-row table: every thread fetches the entries it will publish now (the loads stay in
            // flight behind the K loop) and stores them just before the epilogue
            static_assert(NT <= kTcDequantWarps * 32, "one output-row entry per thread");
            if (q4 == 0 && half == 0) TRACE(2 + set, 1, nitem);
            uint32_t o_nrows = a.m;
            int32_t o_id = -1;
            const uint32_t o_row = it.mt * NT + tid;
            if (a.hids && tid < NT) {
                o_nrows = a.htpe[it.e];
                if (o_row < a.hids_stride) o_id = a.hids[(size_t)it.e * a.hids_stride + o_row];
            }
            for (uint32_t r = 0; ok && r < it.nraw; r++) {
                // keep D raw stages requested ahead of the one being read
                while (!c.raw_tma && q_item < total_items && requested - consumed < D + 1) {
                    if (requested >= R &&
                        !mbar_wait(&raw_empty[islot], iph ^ 1u, &abort_flag, a.status, ST_WAIT_EMPTY_TIMEOUT, wmode_dq)) {
                        ok = false;
                        break;
                    }
                    issue_raw(q_rlo + q_r, islot);
                    requested++;
                    if (++islot == R) { islot = 0; iph ^= 1u; }
                    if (++q_r == q_nraw) {
                        q_item += gridDim.x;
                        if (!c.raw_tma && q_item < total_items) open_request_item();
                    }
                }
                if (!ok) break;
                if (!mbar_wait(&raw_full[rs], rph, &abort_flag, a.status, ST_WAIT_FULL_TIMEOUT, wmode_dq)) { ok = false; break; }
                if (q4 == 0 && half == 0) TRACE(2 + set, 2, r);
                const uint32_t st = 2 * r + set;       // this set's K stage inside raw stage r
                if (st < it.nst) {
                    const uint32_t J = J0 + st;        // its number in the CTA's whole run
                    const uint32_t sa = J % kTcAStages;
                    // the MMAs that read this ring place's previous contents (K stage J - 4) have completed
                    if (J >= kTcAStages &&
                        !mbar_wait(&stage_done[sa], ((J / kTcAStages) & 1u) ^ 1u, &abort_flag, a.status, ST_WAIT_EMPTY_TIMEOUT,
                                   wmode_dq)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    if (q4 == 0 && half == 0) TRACE(2 + set, 3, r);
                    const uint32_t r_abs = it.r_lo + r;
                    const uint32_t pre = (row_lo4 + ((r_abs * KR) / QK) * BB) & 15u;
                    const uint32_t seg = smem_base + c.raw_off + rs * raw_stage_bytes + rr * c.seg_stride + pre;
                uint32_t regs[32];
                if (T != GT_Q4_K && c.aligned && row_ok && !(MLXN_DBG(c) & 1u)) {   // (Q4_K: the generic extraction below)
                    const uint32_t stage_row = smem_base + c.raw_off + rs * raw_stage_bytes + rr * c.seg_stride;
                    if constexpr (T == GT_Q6_K) {
                        dequant32_q6k_aligned_p(r_abs & 7u, stage_row, set, 2 * half, regs);
                        dequant32_q6k_aligned_p(r_abs & 7u, stage_row, set, 2 * half + 1, regs + 16);
                    } else if constexpr (T != GT_Q4_K) {
                        switch (2 * set + half) {  // uniform per warp
                        case 0: dequant64_aligned<T, 0>(stage_row, regs); break;
                        case 1: dequant64_aligned<T, 1>(stage_row, regs); break;
                        case 2: dequant64_aligned<T, 2>(stage_row, regs); break;
                        default: dequant64_aligned<T, 3>(stage_row, regs); break;
                        }
                    }
                } else {
#pragma unroll
                    for (uint32_t hh = 0; hh < 2; hh++) {
                        uint4 v[4];
                        const uint32_t e0 = 128 * set + 64 * half + 32 * hh;  // element offset inside the raw stage
                        if (row_ok && r_abs * KR + e0 < a.k && !(MLXN_DBG(c) & 1u)) {
                            dequant32<T>(seg, e0, v);
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; i++) v[i] = make_uint4(0, 0, 0, 0);
                        }
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            regs[16 * hh + 4 * i + 0] = v[i].x;
                            regs[16 * hh + 4 * i + 1] = v[i].y;
                            regs[16 * hh + 4 * i + 2] = v[i].z;
                            regs[16 * hh + 4 * i + 3] = v[i].w;
                        }
                    }
                }
                    if (q4 == 0 && half == 0) TRACE(2 + set, 8, r);
                    tmem_st_32x32_x32(a_dst + sa * kTcACols, regs);
                    tmem_st_wait();
                    if (q4 == 0 && half == 0) TRACE(2 + set, 9, r);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_full[sa]);
                    if (q4 == 0 && half == 0) TRACE(2 + set, 4, r);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[rs]);  // this warp is done reading the raw stage
                if (q4 == 0 && half == 0) TRACE(2 + set, 10, r);
                consumed++;
                if (++rs == R) { rs = 0; rph ^= 1u; }
            }
            if (!ok) break;
            J0 += it.nst;
            // ---- epilogue: TMEM -> registers -> y ----
            {   // double-buffered: the table of the item before may still be in use by a warp that is behind
                int32_t *wtab = orow[nitem & 1u];
                if (tid < NT) {
                    int32_t o = -1;
                    if (o_row < o_nrows) {
                        if (a.hids) {
                            if (o_id >= 0 && (uint32_t)o_id < a.total_rows) o = o_id;
                        } else {
                            o = (int32_t)o_row;
                        }
                    }
                    wtab[tid] = o;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&orow_ready[nitem & 1u]);
            }
            if (!mbar_wait(&orow_ready[nitem & 1u], (nitem >> 1) & 1u, &abort_flag, a.status, ST_WAIT_EMPTY_TIMEOUT, wmode_dq)) break;
            if (q4 == 0 && half == 0) TRACE(2 + set, 5, nitem);
            if (!mbar_wait(&acc_full, nitem & 1u, &abort_flag, a.status, ST_WAIT_MMA_TIMEOUT, wmode_dq)) break;
            tc_fence_after();
            if (q4 == 0 && half == 0) TRACE(2 + set, 6, nitem);
            const int32_t *tab = orow[nitem & 1u];
            const uint32_t wrow = n0 + rr;
            if (c.stage_off) {
                // Staged read-back (narrow tiles): the accumulator goes to shared memory as [activation row][weight
                // row], tensor memory is handed back to the MMA warps at once, and every warp then writes whole
                // 512-byte output rows with 16-byte stores (the direct form below writes 128 bytes per instruction).
                constexpr uint32_t kPitch = kTcRowsW + 4;   // floats per staged row
                float *stg = reinterpret_cast<float *>(smem + c.stage_off) + (nitem & 1u) * (NT * kPitch);
#pragma unroll 1
                for (uint32_t col = g * 32; col < NT; col += (kTcDequantWarps / 4) * 32) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_d + ((q4 * 32) << 16) + col, v);
                    if (kNumMma == 2 && it.nst >= 2) {
                        uint32_t v1[32];
                        tmem_ld_32x32(tmem_d + ((q4 * 32) << 16) + NT + col, v1);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(v1[j]));
                    }
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++) stg[(col + j) * kPitch + rr] = __uint_as_float(v[j]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&acc_empty);                      // the MMA warps may start the next item
                    mbar_arrive(&stage_ready[nitem & 1u]);        // this warp's part of the staged tile is written
                }
                if (!mbar_wait(&stage_ready[nitem & 1u], (nitem >> 1) & 1u, &abort_flag, a.status, ST_WAIT_EMPTY_TIMEOUT, wmode_dq)) break;
                if (!(MLXN_DBG(c) & 256u)) {
                    const uint32_t c4 = n0 + 4 * lane;
                    for (uint32_t r = dw; r < NT; r += kTcDequantWarps) {
                        const int32_t o = tab[r];
                        if (o < 0) continue;
                        const float4 val = *reinterpret_cast<const float4 *>(stg + r * kPitch + 4 * lane);
                        // (the staged form is never chosen for a call that also stores to peers)
                        float *dst = SH ? a.y + ((size_t)o * qmm_ld(a) + a.y_col0 + c4) : a.y + ((size_t)o * a.n + c4);
                        if (c4 + 3 < a.n) {
                            *reinterpret_cast<float4 *>(dst) = val;
                        } else {
                            if (c4 < a.n) dst[0] = val.x;
                            if (c4 + 1 < a.n) dst[1] = val.y;
                            if (c4 + 2 < a.n) dst[2] = val.z;
                        }
                    }
                }
                if (q4 == 0 && half == 0) TRACE(2 + set, 7, nitem);
                continue;
            }
#pragma unroll 1
            for (uint32_t col = g * 32; col < NT; col += (kTcDequantWarps / 4) * 32) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_d + ((q4 * 32) << 16) + col, v);
                if (kNumMma == 2 && it.nst >= 2) {   // the odd K stages went into the second accumulator
                    uint32_t v1[32];
                    tmem_ld_32x32(tmem_d + ((q4 * 32) << 16) + NT + col, v1);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(v1[j]));
                }
                tmem_ld_wait();
                if (wrow < a.n && !(MLXN_DBG(c) & 256u)) {
                    if constexpr (!SH) {   // a plain [m, n] result of this GPU: nothing between the 32 stores
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const int32_t o = tab[col + j];
                            if (o >= 0) {
                                if (c.ksplit > 1) atomicAdd(&a.y[(size_t)o * a.n + wrow], __uint_as_float(v[j]));
                                else a.y[(size_t)o * a.n + wrow] = __uint_as_float(v[j]);
                            }
                        }
                    } else {           // row-sharded: leading dimension, column offset, the same tile to every peer
#pragma unroll 4
                        for (int j = 0; j < 32; j++) {
                            const int32_t o = tab[col + j];
                            if (o >= 0) {
                                const size_t off = (size_t)o * qmm_ld(a) + a.y_col0 + wrow;
                                a.y[off] = __uint_as_float(v[j]);
                                for (uint32_t pr = 0; pr < a.n_peer; pr++) peer_y[pr][off] = __uint_as_float(v[j]);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty);   // the MMA warp may start the next item's accumulation
            if (q4 == 0 && half == 0) TRACE(2 + set, 7, nitem);
        }
    }
    if (abort_flag) {  // let copies in flight land before the CTA's shared memory is released
        for (int i = 0; i < 200; i++) __nanosleep(5000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kWarpMma0) {
        tc_fence_after();
        tmem_dealloc(tmem_d, kTcTmemCols);
    }
}

// =================================================================================================
// host-side launchers
// =================================================================================================
static inline uint32_t round_up_u(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }
static int sm_count_of_device() {
    static int sms[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 148;
    if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    return sms[dev] ? sms[dev] : 148;
}

// Bytes of scratch the tcgen05 path needs for one call (tile list + packed activations).
size_t qmm_tc_scratch_bytes(const QmmArgs &a, uint32_t nt, bool routed) {
    const uint32_t nchunks = (a.k + 63) / 64;
    size_t tiles;
    size_t header = 0;
    if (routed) {
        tiles = (size_t)a.total_rows / nt + a.n_experts;
        if (tiles > a.total_rows) tiles = a.total_rows;
        if (tiles == 0) tiles = 1;
        header = ((1 + 2 * tiles) * 4 + 1023) / 1024 * 1024;
    } else {
        tiles = (a.m + nt - 1) / nt;
    }
    return header + tiles * nchunks * (size_t)nt * 128;
}

// Activation rows per tile.  Routed calls use 64 (few rows per expert).  Dense calls take the tile that
// minimises waves x per-tile cost, where a tile costs about max(NT, 160) (tensor time vs the fixed
// dequantisation of its 128 weight rows); ties go to the larger tile, which dequantises less in total.
// Split-K factor for a dense call: 2 when the tile grid alone would fill at most ~half of the SMs and K is long
// enough to share (two halves added onto a zeroed y give the same sum in either order).
uint32_t qmm_tc_ksplit(uint32_t nt, uint32_t rows, uint32_t n, uint32_t k, int sm_count, bool routed) {
    if (routed || exp_env("MLXN_TC_NO_SPLITK")) return 1;
    const uint64_t tiles = (uint64_t)((n + kTcRowsW - 1) / kTcRowsW) * ((rows + nt - 1) / nt);
    return (tiles * 2 <= (uint64_t)sm_count + sm_count / 8 && k >= 2048) ? 2u : 1u;
}

uint32_t qmm_tc_pick_nt(int ggml_type, uint32_t rows, uint32_t n, int sm_count, bool routed) {
    if (routed || rows <= 64) return 64;
    (void)ggml_type;
    const uint32_t cap = 256u;
    const uint32_t cands[3] = {256, 128, 64};
    uint32_t best = cap;
    uint64_t best_cost = ~0ull;
    const uint32_t wt = (n + kTcRowsW - 1) / kTcRowsW;
    for (uint32_t nt : cands) {
        if (nt > cap) continue;
        if (nt / 2 >= rows && nt > 64) continue;  // more than half of the tile would be padding
        // (K is not known here: assume it is long enough to split when the grid is small)
        const uint64_t ks = qmm_tc_ksplit(nt, rows, n, 4096, sm_count, false);
        const uint64_t tiles = (uint64_t)wt * ((rows + nt - 1) / nt) * ks;
        const uint64_t waves = (tiles + sm_count - 1) / (uint64_t)sm_count;
        const uint64_t cost = waves * (nt > 160 ? nt : 160) / ks;
        if (cost < best_cost) {
            best_cost = cost;
            best = nt;
        }
    }
    return best;
}

bool qmm_tc_supported(const QmmArgs &a) {
    if (a.k % 32 != 0 || a.k < 32) return false;
    if (((uintptr_t)a.w & 1u) || (a.expert_stride & 1u)) return false;
    return true;
}

template <int T, int NT, bool SH>
static cudaError_t launch_tc_tn(QmmArgs a, bool routed, uint8_t *scratch, cudaStream_t st, int *launches) {
    constexpr int QK = BlockTraits<T>::QK, BB = BlockTraits<T>::BYTES, KR = TcTraits<T>::KR;
    TcCfg c{};
    {
        const char *dbg = exp_env("MLXN_TC_DEBUG");
        c.debug = dbg ? (uint32_t)atoi(dbg) : 0u;
    }
    {
        const uint32_t row_bytes = (a.k / QK) * BB;
        c.aligned = ((((uintptr_t)a.w | a.expert_stride) & 15u) == 0 && row_bytes % 16 == 0 && a.k % 256 == 0) ? 1u : 0u;
        if (exp_env("MLXN_TC_NO_ALIGNED")) c.aligned = 0;  // experiment switch
    }
    c.nchunks = (a.k + 63) / 64;
    c.seg_stride = round_up_u((KR / QK) * BB + 15, 16) + 16;
    if ((c.seg_stride / 16) % 2 == 0) c.seg_stride += 16;  // odd multiple of 16 B: rows spread over the banks
    // Aligned weights arrive by tensor copies: one per raw stage instead of 16-byte copies from every thread.
    // The box is the stage's bytes of 128 rows (Q6_K: 224 bytes cover 210 plus the lead-in; 240 keeps the row
    // pitch an odd multiple of 16).  A 3-D map [expert][row][words]; dense calls are one expert.
    alignas(64) CUtensorMap wmap;
    memset(&wmap, 0, sizeof(wmap));
    if (c.aligned && !exp_env("MLXN_TC_NO_TMA")) {
        EncodeTiledFn enc = encode_tiled_fn();
        const uint32_t row_bytes = (a.k / QK) * BB;
        const uint32_t box_bytes = T == GT_Q6_K ? 240u : (uint32_t)((KR / QK) * BB);
        const uint32_t n_exp = routed ? a.n_experts : 1u;
        const uint64_t estride = routed ? a.expert_stride : (uint64_t)a.n * row_bytes;
        if (enc && n_exp >= 1 && (uint64_t)row_bytes * a.n <= estride) {
            const cuuint64_t gdim[3] = {row_bytes / 4, a.n, n_exp};
            const cuuint64_t gstride[2] = {row_bytes, estride};
            const cuuint32_t box[3] = {box_bytes / 4, (cuuint32_t)kTcRowsW, 1};
            const cuuint32_t estr[3] = {1, 1, 1};
            if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<uint8_t *>(a.w), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
                c.raw_tma = 1;
                c.seg_stride = box_bytes;
            }
        }
    }
    const uint32_t b_bytes = NT * 128;  // one 64-wide K chunk of the activation tile
    const uint32_t raw_slot = kTcRowsW * c.seg_stride;
    uint32_t limit = 222 * 1024;  // + 1 KB alignment slack + ~3 KB of static shared memory <= 227 KB
    // narrow tiles stage their result in shared memory (two tiles of NT x 132 floats) and write whole output rows
    const uint32_t stage_bytes = 2u * NT * (kTcRowsW + 4) * 4u;
    // (the row-sharded form never splits K: its tiles go straight to every rank's buffer)
    constexpr bool sharded = SH;                         // a.y_ld != 0 || a.n_peer != 0
    const bool staged = NT == 64 && (sharded || qmm_tc_ksplit(NT, a.m, a.n, a.k, sm_count_of_device(), routed) == 1) &&
                        ((((uintptr_t)a.y) | ((uintptr_t)qmm_ld(a) * 4u) | ((uintptr_t)a.y_col0 * 4u)) & 15u) == 0 && a.n_peer == 0 &&
                        !exp_env("MLXN_TC_NO_STAGED_OUT");
    if (staged) limit -= stage_bytes;
    // activation ring first (at least two raw slots kept back), the rest goes to the raw weight ring
    uint32_t b_stages = (limit - 2 * raw_slot) / b_bytes;
    // (a 64-row tile's chunks are 8 KB: eight of them where four raw slots still fit beside them, the loop being
    // bound by how far the copies run ahead of the MMAs)
    const uint32_t b_cap = (NT == 64 && limit >= 8 * b_bytes + 4 * raw_slot) ? 8u : 6u;
    if (b_stages > b_cap) b_stages = b_cap;
    if (const char *e = exp_env("MLXN_TC_STAGES")) {  // experiment switch
        const uint32_t v = (uint32_t)atoi(e);
        if (v >= 4 && v <= b_stages) b_stages = v;
    }
    if (b_stages < 4) return cudaErrorInvalidConfiguration;   // (shallower rings are untested)
    uint32_t raw_slots = (limit - b_stages * b_bytes) / raw_slot;
    if (raw_slots > 6) raw_slots = 6;
    if (const char *e = exp_env("MLXN_TC_RAW")) {  // experiment switch
        const uint32_t v = (uint32_t)atoi(e);
        if (v >= 2 && v <= raw_slots) raw_slots = v;
    }
    const uint32_t raw_bytes = raw_slots * raw_slot;
    c.b_stages = b_stages;
    c.raw_slots = raw_slots;
    c.b_off = 0;
    c.raw_off = b_stages * b_bytes;
    if (staged) c.stage_off = c.raw_off + raw_bytes;
    const size_t smem = (size_t)c.raw_off + raw_bytes + (staged ? stage_bytes : 0u) + 1024;  // + slack for manual 1024-byte alignment

    const uint32_t ksplit = sharded ? 1u : qmm_tc_ksplit(NT, a.m, a.n, a.k, sm_count_of_device(), routed);
    size_t tiles;
    uint8_t *xpack = scratch;
    if (routed) {
        tiles = (size_t)a.total_rows / NT + a.n_experts;
        if (tiles > a.total_rows) tiles = a.total_rows;
        if (tiles == 0) tiles = 1;
        const size_t header = ((1 + 2 * tiles) * 4 + 1023) / 1024 * 1024;
        uint32_t *tl = reinterpret_cast<uint32_t *>(scratch);
        if (!(a.reuse & 1u)) {   // (an earlier call of the same layer built the list: same buckets, same NT)
            build_tiles_kernel<<<1, 256, 0, st>>>(a.htpe, a.n_experts, NT, (uint32_t)tiles, tl);
            (*launches)++;
        }
        a.tiles = tl;
        xpack = scratch + header;
    } else {
        tiles = (a.m + NT - 1) / NT;
        a.tiles = nullptr;
    }
    if (!(a.reuse & 2u)) {   // (... or packed the same activation rows already)
        // enough CTAs to fill the GPU a few times over, few enough that a tile's routing lookups are amortised
        uint32_t lanes = c.nchunks;
        while (lanes > 1 && (uint64_t)lanes * tiles > 2048) lanes = (lanes + 1) / 2;
        dim3 grid(lanes, (unsigned)tiles);
        pack_x_kernel<NT><<<grid, 256, 0, st>>>(a, xpack, c.nchunks, ksplit > 1 ? 1u : 0u);
        (*launches)++;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    static size_t attr_smem[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (smem > attr_smem[dev]) {
        cudaError_t e = cudaFuncSetAttribute(qmm_tc_kernel<T, NT, SH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_smem[dev] = smem;
    }
    c.n_wt = (a.n + kTcRowsW - 1) / kTcRowsW;
    c.ntiles = (uint32_t)tiles;
    c.ksplit = ksplit;
    // persistent CTAs, one per SM, each walking its share of the (weight tile, K split, activation tile) items
    const uint64_t items = (uint64_t)c.n_wt * tiles * ksplit;
    uint32_t ctas = (uint32_t)sm_count_of_device();
    if (const char *e = exp_env("MLXN_TC_CTAS")) {  // experiment switch
        const int v = atoi(e);
        if (v >= 1 && v <= 4096) ctas = (uint32_t)v;
    }
    if (items < ctas) ctas = (uint32_t)items;
    if (ctas == 0) return cudaSuccess;
    (*launches)++;
    return launch_overlapped(qmm_tc_kernel<T, NT, SH>, dim3(ctas), dim3(kTcThreads), smem, st, a, c, xpack, wmap);
}

template <int T> static cudaError_t launch_tc_t(const QmmArgs &a, bool routed, uint32_t nt, uint8_t *scratch, cudaStream_t st,
                                                int *launches) {
    if (a.y_ld != 0 || a.n_peer != 0) {   // row-sharded result: the instantiation with the peer stores
        switch (nt) {
        case 64: return launch_tc_tn<T, 64, true>(a, routed, scratch, st, launches);
        case 128: return launch_tc_tn<T, 128, true>(a, routed, scratch, st, launches);
        case 256: return launch_tc_tn<T, 256, true>(a, routed, scratch, st, launches);
        default: return cudaErrorInvalidValue;
        }
    }
    switch (nt) {
    case 64: return launch_tc_tn<T, 64, false>(a, routed, scratch, st, launches);
    case 128: return launch_tc_tn<T, 128, false>(a, routed, scratch, st, launches);
    case 256: return launch_tc_tn<T, 256, false>(a, routed, scratch, st, launches);
    default: return cudaErrorInvalidValue;
    }
}

// tcgen05 mat-mat.  `scratch` must hold qmm_tc_scratch_bytes(a, nt, routed) bytes and start on a 256-byte boundary (the packed
// tiles in it are sources of bulk copies: 16-byte alignment is what the hardware needs; their offsets are multiples of 1024).
cudaError_t launch_qmm_tc(int ggml_type, const QmmArgs &a, bool routed, uint32_t nt, uint8_t *scratch, cudaStream_t st,
                          int *launches) {
    switch (ggml_type) {
    case GT_Q4_0: return launch_tc_t<GT_Q4_0>(a, routed, nt, scratch, st, launches);
    case GT_Q8_0: return launch_tc_t<GT_Q8_0>(a, routed, nt, scratch, st, launches);
    case GT_Q6_K: return launch_tc_t<GT_Q6_K>(a, routed, nt, scratch, st, launches);
    case GT_Q4_K: return launch_tc_t<GT_Q4_K>(a, routed, nt, scratch, st, launches);
    default: return cudaErrorInvalidValue;
    }
}

template <int T> static cudaError_t launch_simt_t(const QmmArgs &a, bool routed, uint32_t max_rows, cudaStream_t st) {
    dim3 grid((max_rows + 63) / 64, (a.n + 63) / 64, routed ? a.n_experts : 1);
    qmm_simt_kernel<T><<<grid, 256, 0, st>>>(a);
    return cudaGetLastError();
}

// CUDA-core mat-mat.  max_rows: a.m (dense) or the largest possible rows per expert (routed).
cudaError_t launch_qmm_simt(int ggml_type, const QmmArgs &a, bool routed, uint32_t max_rows, cudaStream_t st) {
    switch (ggml_type) {
    case GT_Q4_0: return launch_simt_t<GT_Q4_0>(a, routed, max_rows, st);
    case GT_Q8_0: return launch_simt_t<GT_Q8_0>(a, routed, max_rows, st);
    case GT_Q6_K: return launch_simt_t<GT_Q6_K>(a, routed, max_rows, st);
    case GT_Q4_K: return launch_simt_t<GT_Q4_K>(a, routed, max_rows, st);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace mlxn

// =================================================================================================
// mat-mat entry point that allocates nothing
// =================================================================================================
// Some callers may not allocate device memory at the moment they need a mat-mat: code running inside a
// memory-budgeted serving process whose allocator owns every byte of HBM, a real-time loop that must not
// hit the driver's allocation lock, or a plug-in that is only handed pointers.  For them the packed
// activation tiles of the tensor-core path live in this fixed array instead of the encoder's arena.
// Every GPU that loads the library carries the array until the process exits.
#include <cstdio>
#include <mutex>

#include "../../include/mlxn_b200.h"

int mlxn_detail_fail(int status, const char *msg);
void mlxn_detail_count_launches(int launches);

#define MLXN_NOALLOC_SCRATCH_BYTES (16u * 1024u * 1024u)
static __device__ __align__(256) uint8_t g_noalloc_scratch[MLXN_NOALLOC_SCRATCH_BYTES];

namespace {
std::mutex g_noalloc_mu;
uint8_t *g_noalloc_ptr[64] = {};  // device address of g_noalloc_scratch, per device ordinal
int g_noalloc_sms[64] = {};
}  // namespace

extern "C" size_t mlxn_noalloc_scratch_limit(void) { return MLXN_NOALLOC_SCRATCH_BYTES; }

extern "C" int mlxn_quantized_matmul_ggml_mm_noalloc(void *cuda_stream, const void *input_dev, const void *weight_dev,
                                                     void *output_dev, const mlxn_qmm_params *params) {
    using namespace mlxn;
    if (!input_dev || !weight_dev || !output_dev || !params)
        return mlxn_detail_fail(MLXN_INVALID_ARGUMENT, "Invalid argument: pointers and params must not be null");
    const int t = (int)params->ggml_type;
    if (t != GT_Q4_0 && t != GT_Q8_0 && t != GT_Q6_K)
        return mlxn_detail_fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_ggml_mm_noalloc supports Q4_0, Q8_0 and Q6_K only");
    if (params->m == 0 || params->k == 0 || params->n == 0)
        return mlxn_detail_fail(MLXN_INVALID_ARGUMENT, "Invalid argument: M, K, and N must all be > 0");
    if (params->k % ggml_qk(t) != 0 || params->k % 32 != 0)
        return mlxn_detail_fail(MLXN_INVALID_ARGUMENT, "Invalid argument: K must be divisible by the block QK and by 32");
    if (((uintptr_t)weight_dev & 1u) || ((uintptr_t)input_dev & 3u) || ((uintptr_t)output_dev & 3u))
        return mlxn_detail_fail(MLXN_INVALID_ARGUMENT, "Invalid argument: weights must be 2-byte aligned, f32 buffers 4-byte aligned");
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return mlxn_detail_fail(MLXN_DEVICE_NOT_FOUND, "No usable current CUDA device for quantized_matmul_ggml_mm_noalloc");
#if CUDART_VERSION >= 12080
    {
        // the kernels are launched on the CURRENT device: a stream of another device would be refused by the launch with an
        // error that does not say why
        int sdev = -1;
        if (cudaStreamGetDevice(static_cast<cudaStream_t>(cuda_stream), &sdev) == cudaSuccess && sdev != dev) {
            char msg[160];
            snprintf(msg, sizeof(msg), "Invalid argument: quantized_matmul_ggml_mm_noalloc: the stream belongs to device %d but device %d is current",
                     sdev, dev);
            return mlxn_detail_fail(MLXN_INVALID_ARGUMENT, msg);
        }
        cudaGetLastError();
    }
#endif
    uint8_t *scratch = nullptr;
    int sms = 0;
    {
        // first call on this device (with the device current): look up where the array lives on it.
        // The array's name is a host-side stand-in; only the address returned here may be given to a kernel.
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        if (!g_noalloc_ptr[dev]) {
            void *p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p) {
                cudaGetLastError();
                return mlxn_detail_fail(MLXN_COMMAND_BUFFER_ERROR, "Command buffer error: cudaGetSymbolAddress failed for the static scratch array");
            }
            int n = 0;
            e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess || n <= 0) {
                cudaGetLastError();
                return mlxn_detail_fail(MLXN_COMMAND_BUFFER_ERROR, "Command buffer error: cannot query the SM count");
            }
            g_noalloc_sms[dev] = n;
            g_noalloc_ptr[dev] = static_cast<uint8_t *>(p);
        }
        scratch = g_noalloc_ptr[dev];
        sms = g_noalloc_sms[dev];
    }
    QmmArgs a{};
    a.w = static_cast<const uint8_t *>(weight_dev);
    a.x = static_cast<const float *>(input_dev);
    a.y = static_cast<float *>(output_dev);
    a.m = params->m;
    a.n = params->n;
    a.k = params->k;
    a.top_k = 1;
    a.n_experts = 1;
    a.total_rows = params->m;
    a.status = nullptr;  // no status word: a wait that gives up still ends the kernel, but is not reported
    const uint32_t nt = qmm_tc_pick_nt(t, a.m, a.n, sms, false);
    const size_t need = qmm_tc_scratch_bytes(a, nt, false);
    if (need > MLXN_NOALLOC_SCRATCH_BYTES) {
        char msg[256];
        snprintf(msg, sizeof(msg),
                 "Invalid argument: quantized_matmul_ggml_mm_noalloc needs %zu bytes of packed activations for m=%u k=%u, "
                 "the static scratch holds %u (about m*k <= 8M elements); use quantized_matmul_ggml instead",
                 need, a.m, a.k, MLXN_NOALLOC_SCRATCH_BYTES);
        return mlxn_detail_fail(MLXN_INVALID_ARGUMENT, msg);
    }
    int launches = 0;
    cudaError_t e = launch_qmm_tc(t, a, false, nt, scratch, static_cast<cudaStream_t>(cuda_stream), &launches);
    if (e != cudaSuccess) {
        cudaGetLastError();
        char msg[256];
        snprintf(msg, sizeof(msg), "Command buffer error: mat-mat launch: %s", cudaGetErrorString(e));
        return mlxn_detail_fail(MLXN_COMMAND_BUFFER_ERROR, msg);
    }
    mlxn_detail_count_launches(launches);
    return MLXN_OK;
}
