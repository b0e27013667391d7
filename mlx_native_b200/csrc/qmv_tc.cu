// Tensor-core mat-vec for 1..8 activation rows (decode): y[m, n] = x[m, k] . W[n, k]^T with W in GGML blocks.
//
// The weight stream is the whole cost of this operation, so the kernel is built around two ideas:
//
//  * The tensor core does the multiply-adds.  A weight tile of 128 rows is turned into *exact integers*
//    (the 4/8-bit codes, written as f16 subnormals n * 2^-24, which costs one or two bit operations per
//    pair of codes) and stored straight into tensor memory as the A operand of tcgen05.mma.  The
//    activations are the B operand: each row is split into hi + lo f16 halves (8 rows x 2 = N = 16), so
//    that their sum carries ~22 significant bits.  Products of an f16 subnormal integer and an f16 value
//    are exact and accumulate in f32, so each MMA yields the exact integer dot product of one block.
//  * The per-block scale d (and the code offset, -8 / -128) cannot ride through the MMA -- it differs per
//    row and block -- so every block gets its own 16-column accumulator, which the row's thread reads back
//    (tcgen05.ld) and folds into a running f32 sum:  y += d * (2^24 * (D_hi + D_lo) - offset * sum(x_block)).
//    That is ~0.5 instructions per weight element instead of one FMA per element and activation row.
//
// A small kernel in front packs the activations (one CTA per 256-wide K unit) and zeroes y; the mat-vec kernel
// is launched as its programmatic dependent, so that its set-up and first weight copies overlap the packing.
//
// Work is split stream-K style: the (row tile, 256-wide K unit) grid is cut into one contiguous range per
// CTA, so every SM streams the same number of bytes whatever the matrix shape.  A tile whose K range is
// shared by several CTAs is summed into y with f32 atomic adds (the packing kernel zeroes y first); two
// partial sums add up the same in either order, three or more may differ in the last bit from run to run.
//
// Supported here: Q4_0, Q8_0 (k % 256 == 0) and Q6_K (k % 2048 == 0), dense form, 16-byte aligned weight rows.
// Everything else takes the SIMT kernels.
#include "tensor_map.cuh"  // CUtensorMap + the encoder, fetched through the runtime (no libcuda link)

#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"

namespace mlxn {

constexpr int kVtRows = 128;            // weight rows per tile (UMMA M)
constexpr int kVtGroups = 4;            // convert/readout groups; group g owns sub-step g of every K unit
constexpr int kVtCvtWarps = 4 * kVtGroups;
constexpr int kVtMmaWarps = 2;
constexpr int kVtThreads = (kVtCvtWarps + 1 + kVtMmaWarps) * 32;  // + producer warp
constexpr int kVtSlotCols = 64;         // tensor-memory columns per (group, parity) slot: 32 A + 32 D
constexpr int kVtTmemCols = 512;
constexpr int kVtUnitK = 256;           // K elements per unit (8 blocks: a multiple of 16 bytes in both formats)
constexpr int kVtMaxSlots = 8;          // raw ring depth bound
constexpr int kVtMaxCtas = 160;

// UB: bytes of a K unit of one row.  SS: sub-steps a group runs per unit (a sub-step is what one thread converts
// and stores at a time: 64 K = 2 blocks, or for Q6_K 32 K = 2 scale groups).  SG: elements per scale (= per
// accumulator).  AUX: bytes of per-unit side data (sums of x per scale group [256/SG][8] f32, scales [2][8] f32).
template <int T> struct VtTraits;
template <> struct VtTraits<GT_Q4_0> { static constexpr int UB = 144, SUB = 36, OFFSET = 8, SS = 1, SG = 32, AUX = 320; };
template <> struct VtTraits<GT_Q8_0> { static constexpr int UB = 272, SUB = 68, OFFSET = 128, SS = 1, SG = 32, AUX = 320; };
template <> struct VtTraits<GT_Q6_K> { static constexpr int UB = 210, SUB = 0, OFFSET = 32, SS = 2, SG = 16, AUX = 576; };
constexpr int kVtQ6Box = 240;  // bytes per row of a Q6_K stage: the 210-byte super-block and its lead-in, an odd multiple of 16

__host__ __device__ inline uint32_t vt_aux_bytes(int ggml_type) { return ggml_type == GT_Q6_K ? 576u : 320u; }

// K permutation inside a unit: packed position P (tensor-memory column P/2, half P%2, in the order the
// sub-steps are stored) holds element vt_src(P) of the unit.  It follows from the cheapest way to pull code
// pairs out of a 32-bit word of the block (mask / shift, or byte select); the activations are packed the same way.
__host__ __device__ inline uint32_t vt_src(int ggml_type, uint32_t P) {
    if (ggml_type == GT_Q6_K) {
        // sub-step ss = 4 n + 2 pairB + lh (32 positions): two scale groups (q1|q2 then q3|q4 of the same 16 l's)
        const uint32_t ss = P >> 5, p = P & 31u;
        const uint32_t n = ss >> 2, pair_b = (ss >> 1) & 1u, lh = ss & 1u;
        const uint32_t grp = p >> 4, col = (p & 15u) >> 1, hl = p & 1u;
        const uint32_t l = 16 * lh + 4 * (col >> 1) + (col & 1u) + 2 * hl;
        return 128 * n + l + 32 * pair_b + 64 * grp;
    }
    const uint32_t blk = P >> 5, p = P & 31u;
    const uint32_t col = p >> 1, hl = p & 1u;
    if (ggml_type == GT_Q4_0) {
        // word i = bytes 4i..4i+3 (low nibbles: elements 4i..4i+3, high nibbles: 16+4i..); four pairs per word
        const uint32_t i = col >> 2, j = col & 3u;
        return 32 * blk + 4 * i + ((j & 1u) ? 16u : 0u) + ((j & 2u) ? 1u : 0u) + 2 * hl;
    }
    // Q8_0: word i = elements 4i..4i+3; pairs (b0, b2) and (b1, b3)
    const uint32_t i = col >> 1, j = col & 1u;
    return 32 * blk + 4 * i + j + 2 * hl;
}

struct VtCfg {
    uint32_t tiles, upt;        // row tiles, K units per tile
    uint32_t total_units;
    uint32_t cu;                // K units per raw stage (one tensor copy of 128 rows x cu * UB bytes)
    uint32_t nslots;            // raw ring depth
    uint32_t row_stride;        // shared-memory bytes per weight row of a stage = cu * UB (odd multiple of 16)
    uint32_t slot_bytes;        // B tiles + block sums + raw rows, multiple of 1024
    uint32_t xs_off, raw_off;   // offsets inside a slot
    uint32_t debug;
    uint32_t pairs;             // Q6_K rows of 16 n + 8 bytes: the tensor map's rows are pairs of weight rows (see launch_vt_t)
    uint32_t row_bytes;
};

constexpr int kVtMaxUnits = 1024; // K units per row the flag words cover (k <= 262144)

struct VtScratch {
    uint8_t *xpack;      // [k/64][16 rows][128 B] f16 hi/lo tiles, 128-byte swizzled
    uint8_t *aux;        // [k/256][aux bytes of the format]
};

__device__ __forceinline__ uint32_t pack_h2(__half lo, __half hi) {
    return (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
}

// ------------------------------------------------------------------------------------------------
// activation packing: one warp per (activation row, 128-wide half of a K unit)
// ------------------------------------------------------------------------------------------------
// 128 values of x -> (a) pre-scale by a power of two so that their largest magnitude lands in [2^13, 2^14)
// (exact, undone when the half's partial sums are added up; keeps hi and lo inside the f16 normal range
// whatever the magnitude of the activations), (b) hi = f16(x), lo = f16(x - hi), (c) the per-block sums of
// hi + lo, (d) both written in the tensor core's K-major 128-byte-swizzled tile layout with the per-block
// K permutation of the weight format.
__device__ __forceinline__ void vt_pack_half(const float *xr, uint32_t ku, uint32_t t, uint32_t h, uint32_t lane, int ggml_type,
                                             const VtScratch &s) {
    const uint32_t p0 = 128 * h + 4 * lane;            // first of the lane's 4 packed positions inside the unit
    float v[4];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[i] = xr[(size_t)ku * kVtUnitK + vt_src(ggml_type, p0 + i)];
        amax = fmaxf(amax, fabsf(v[i]));
    }
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // scale = 2^(13 - floor(log2(amax))), clamped to the normal f32 range; 1 for an all-zero or non-finite run
    float scale = 1.f, inv = 1.f;
    if (amax > 0.f && amax < 3.0e38f) {
        int e = 13 - (int)((__float_as_uint(amax) >> 23) & 0xff) + 127;
        e = max(-100, min(100, e));
        scale = __uint_as_float((uint32_t)(e + 127) << 23);
        inv = __uint_as_float((uint32_t)(127 - e) << 23);
    }
    __half hi[4], lo[4];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float xs = v[i] * scale;
        hi[i] = __float2half_rn(xs);
        lo[i] = __float2half_rn(xs - __half2float(hi[i]));
        sum += __half2float(hi[i]) + __half2float(lo[i]);
    }
    const uint32_t chunk = p0 >> 6, q = p0 & 63u, j = q >> 3;
    uint8_t *tile = s.xpack + ((size_t)ku * 4 + chunk) * 2048 + t * 128 + ((j ^ t) << 4) + (q & 7u) * 2;
    *reinterpret_cast<uint2 *>(tile) = make_uint2(pack_h2(hi[0], hi[1]), pack_h2(hi[2], hi[3]));          // row t
    *reinterpret_cast<uint2 *>(tile + 1024) = make_uint2(pack_h2(lo[0], lo[1]), pack_h2(lo[2], lo[3]));   // row 8 + t
    // sums per scale group: 32 positions (8 lanes) for Q4_0 / Q8_0, 16 positions (4 lanes) for Q6_K
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    float *aux = reinterpret_cast<float *>(s.aux + (size_t)ku * vt_aux_bytes(ggml_type));
    if (ggml_type == GT_Q6_K) {
        if ((lane & 3u) == 0) aux[(p0 >> 4) * 8 + t] = sum;
        if (lane == 0) aux[128 + h * 8 + t] = inv;
    } else {
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if ((lane & 7u) == 0) aux[(p0 >> 5) * 8 + t] = sum;
        if (lane == 0) aux[64 + h * 8 + t] = inv;
    }
}

// grid = (K units, ceil(2 m / 4)), 128 threads (small enough to share an SM with a mat-vec CTA of the operation
// ahead): each warp packs one (activation row, half) of the CTA's unit; all threads zero a slice of y (tiles
// split between CTAs of the mat-vec kernel are summed into it with atomic adds).
__global__ void __launch_bounds__(128) qmv_tc_pack_kernel(const QmvArgs a, int ggml_type, VtScratch s, uint32_t debug) {
    const float *x = a.x;
    const uint32_t m = a.m, n = a.n, k = a.k;
    grid_dependency_wait();  // x (and y, which is zeroed here) belong to the kernels ahead until they are done
    allow_dependents();      // the mat-vec kernel may set itself up and start its weight stream
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t ncta = gridDim.x * gridDim.y, cta = blockIdx.y * gridDim.x + blockIdx.x;
    const uint32_t total = m * n, per = (total + ncta - 1) / ncta;
    const uint32_t lo = min(total, cta * per), hi = min(total, lo + per);
    {
        const uint32_t ld = qmv_ld(a);
        for (uint32_t i = lo + tid; i < hi; i += blockDim.x) {
            const uint32_t t = i / n, col = i - t * n;
            const size_t off = (size_t)t * ld + a.y_col0 + col;
            a.y[off] = 0.f;
            for (uint32_t pr = 0; pr < a.n_peer; pr++) a.y_peer[pr][off] = 0.f;
        }
    }
    const uint32_t task = blockIdx.y * 4 + warp;
    if (task < 2 * m) vt_pack_half(x + (size_t)(task >> 1) * k, blockIdx.x, task >> 1, task & 1u, lane, ggml_type, s);
}

// ------------------------------------------------------------------------------------------------
// code extraction: one sub-step (64 K elements = 2 blocks) of one weight row -> 32 packed f16 pairs
// ------------------------------------------------------------------------------------------------
// `unit` = shared address of the row's 16-byte aligned K unit; S4 = which quarter of the unit (compile time,
// so every byte offset below is static).  d0 / d1 receive the two blocks' scales.
template <int T, int S4> __device__ __forceinline__ void vt_extract(uint32_t unit, uint32_t (&r)[32], float &d0, float &d1) {
    constexpr int SUB = VtTraits<T>::SUB;
    constexpr int c0 = (SUB * S4) >> 4;             // first 16-byte chunk touched
    constexpr int wo = ((SUB * S4) & 15) >> 2;      // word offset of the sub-step inside that chunk
    if constexpr (T == GT_Q4_0) {
        uint32_t W[12];
#pragma unroll
        for (int i = 0; i < 3; i++) lds128(unit + 16 * (c0 + i), W[4 * i], W[4 * i + 1], W[4 * i + 2], W[4 * i + 3]);
        d0 = half_bits_to_float(W[wo] & 0xFFFFu);
        d1 = half_bits_to_float(W[wo + 4] >> 16);
#pragma unroll
        for (int b = 0; b < 2; b++) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                // block 0's codes start 2 bytes into a word, block 1's are word aligned
                const uint32_t w = b == 0 ? __funnelshift_r(W[wo + i], W[wo + i + 1], 16) : W[wo + 5 + i];
                r[16 * b + 4 * i + 0] = w & 0x000F000Fu;
                r[16 * b + 4 * i + 1] = (w >> 4) & 0x000F000Fu;
                r[16 * b + 4 * i + 2] = (w >> 8) & 0x000F000Fu;
                r[16 * b + 4 * i + 3] = (w >> 12) & 0x000F000Fu;
            }
        }
    } else {
        uint32_t W[20];
#pragma unroll
        for (int i = 0; i < 5; i++) lds128(unit + 16 * (c0 + i), W[4 * i], W[4 * i + 1], W[4 * i + 2], W[4 * i + 3]);
        d0 = half_bits_to_float(W[wo] & 0xFFFFu);
        d1 = half_bits_to_float(W[wo + 8] >> 16);
#pragma unroll
        for (int b = 0; b < 2; b++) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                uint32_t w = b == 0 ? __funnelshift_r(W[wo + i], W[wo + i + 1], 16) : W[wo + 9 + i];
                w ^= 0x80808080u;  // signed byte -> byte + 128
                r[16 * b + 2 * i + 0] = __byte_perm(w, 0u, 0x4240);
                r[16 * b + 2 * i + 1] = __byte_perm(w, 0u, 0x4341);
            }
        }
    }
}

// Q6_K: one sub-step = the 16 l's [16 lh, 16 lh + 16) of half n of the super-block, for the quant pair
// (q1, q3) or (q2, q4): two scale groups of 16 codes -> 16 packed pairs.  The super-block starts PRE bytes
// into the row's 16-byte aligned stage (PRE = 2 (unit index % 8), the same for every row, so it is a
// compile-time constant of the variant); every field offset below is PRE plus a multiple of 16.
template <int PRE>
__device__ __forceinline__ void vt_extract_q6k(uint32_t stage_row, uint32_t n, uint32_t g, uint32_t (&r)[16], float &d0, float &d1) {
    const uint32_t pair_b = g >> 1, lh = g & 1u;
    uint32_t ql[4], qh[4];
    lds_field16<PRE>(stage_row + 64 * n + 32 * pair_b + 16 * lh, ql);
    lds_field16<PRE>(stage_row + 128 + 32 * n + 16 * lh, qh);
    const uint32_t sc_addr = stage_row + PRE + 192 + 8 * n + lh + 2 * pair_b;
    const float d = half_bits_to_float(lds_u16(stage_row + PRE + 208));
    d0 = d * (float)lds_s8(sc_addr);
    d1 = d * (float)lds_s8(sc_addr + 4);
    const uint32_t s_up = pair_b ? 2u : 4u, s_dn = pair_b ? 2u : 0u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t first = (ql[i] & 0x0F0F0F0Fu) | ((qh[i] << s_up) & 0x30303030u);
        const uint32_t second = ((ql[i] >> 4) & 0x0F0F0F0Fu) | ((qh[i] >> s_dn) & 0x30303030u);
        r[2 * i + 0] = __byte_perm(first, 0u, 0x4240);
        r[2 * i + 1] = __byte_perm(first, 0u, 0x4341);
        r[8 + 2 * i + 0] = __byte_perm(second, 0u, 0x4240);
        r[8 + 2 * i + 1] = __byte_perm(second, 0u, 0x4341);
    }
}
__device__ __forceinline__ void vt_extract_q6k_p(uint32_t p8, uint32_t stage_row, uint32_t n, uint32_t g, uint32_t (&r)[16],
                                                 float &d0, float &d1) {
    switch (p8) {  // uniform over the CTA
    case 0: vt_extract_q6k<0>(stage_row, n, g, r, d0, d1); break;
    case 1: vt_extract_q6k<2>(stage_row, n, g, r, d0, d1); break;
    case 2: vt_extract_q6k<4>(stage_row, n, g, r, d0, d1); break;
    case 3: vt_extract_q6k<6>(stage_row, n, g, r, d0, d1); break;
    case 4: vt_extract_q6k<8>(stage_row, n, g, r, d0, d1); break;
    case 5: vt_extract_q6k<10>(stage_row, n, g, r, d0, d1); break;
    case 6: vt_extract_q6k<12>(stage_row, n, g, r, d0, d1); break;
    default: vt_extract_q6k<14>(stage_row, n, g, r, d0, d1); break;
    }
}

template <int T> __device__ __forceinline__ void vt_extract_g(uint32_t g, uint32_t unit, uint32_t (&r)[32], float &d0, float &d1) {
    switch (g) {  // uniform per warp
    case 0: vt_extract<T, 0>(unit, r, d0, d1); break;
    case 1: vt_extract<T, 1>(unit, r, d0, d1); break;
    case 2: vt_extract<T, 2>(unit, r, d0, d1); break;
    default: vt_extract<T, 3>(unit, r, d0, d1); break;
    }
}

// first unit of CTA c's contiguous range
__host__ __device__ inline uint32_t vt_range_begin(uint32_t c, uint32_t total, uint32_t grid) {
    return (uint32_t)(((uint64_t)c * total) / grid);
}

// A CTA's walk over its unit range, one raw stage (up to cu units of one tile) at a time.  Every role of the
// CTA walks the same sequence; the ring slot and its phase bit move along.  One division, at the start.
struct VtWalk {
    uint32_t u, u1, upt, cu, nslots;
    uint32_t tile, kun, cnt;   // current stage: tile, first K unit inside the tile, units
    uint32_t slot, ph;         // raw ring slot of the stage and the parity of this use of it
    uint32_t sidx;
    bool seg_end;              // the tile's segment (run of stages of this tile inside the CTA's range) ends with this stage
    __device__ __forceinline__ void setup() {
        cnt = min(cu, min(upt - kun, u1 - u));
        seg_end = (kun + cnt == upt) || (u + cnt == u1);
    }
    __device__ __forceinline__ void init(uint32_t u0, uint32_t u1_, uint32_t upt_, uint32_t cu_, uint32_t nslots_) {
        u = u0; u1 = u1_; upt = upt_; cu = cu_; nslots = nslots_;
        tile = u0 / upt_;
        kun = u0 - tile * upt_;
        slot = 0; ph = 0; sidx = 0;
        setup();
    }
    __device__ __forceinline__ bool done() const { return u >= u1; }
    __device__ __forceinline__ void next() {
        u += cnt;
        kun += cnt;
        if (kun == upt) { kun = 0; tile++; }
        if (++slot == nslots) { slot = 0; ph ^= 1u; }
        sidx++;
        if (u < u1) setup();
    }
};

// MP = activation row pairs carried (1, 2 or 4)
template <int T, int MP>
__global__ void __launch_bounds__(kVtThreads, 1)
    qmv_tc_kernel(const QmvArgs a, const VtCfg c, const VtScratch sc, const __grid_constant__ CUtensorMap wmap) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int UB = VtTraits<T>::UB, SS = VtTraits<T>::SS, AUX = VtTraits<T>::AUX;
    constexpr float kOff = (float)VtTraits<T>::OFFSET;
    // byte coordinate of a unit's tensor copy inside the row: Q6_K units start at the 16-byte boundary below them
    auto unit_x = [](uint32_t kun) -> uint32_t { return T == GT_Q6_K ? ((kun * UB) & ~15u) >> 2 : kun * (UB / 4); };
    // One tensor copy brings a stage's 128 rows.  Pair mode (Q6_K rows that are 8 bytes past a 16-byte boundary every
    // other row): the map's rows are pairs of weight rows, so two copies of 64 map rows each bring the even weight
    // rows (stage rows 0-63) and the odd ones (stage rows 64-127), each from the 16-byte boundary below its unit.
    auto issue_weights = [&](uint32_t dst, uint32_t kun, uint32_t tile, uint32_t bar) {
        if (T == GT_Q6_K && c.pairs) {
            const uint32_t xe = ((kun * UB) & ~15u) >> 2, xo = ((c.row_bytes + kun * UB) & ~15u) >> 2;
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                ::"r"(dst), "l"(&wmap), "r"(xe), "r"(tile * (kVtRows / 2)), "r"(bar)
                : "memory");
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                ::"r"(dst + (kVtRows / 2) * c.row_stride), "l"(&wmap), "r"(xo), "r"(tile * (kVtRows / 2)), "r"(bar)
                : "memory");
        } else {
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                ::"r"(dst), "l"(&wmap), "r"(unit_x(kun)), "r"(tile * kVtRows), "r"(bar)
                : "memory");
        }
    };
    __shared__ __align__(8) uint64_t raw_full[kVtMaxSlots], raw_empty[kVtMaxSlots];
    __shared__ __align__(8) uint64_t a_full[2 * kVtGroups], d_full[2 * kVtGroups];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile uint32_t abort_flag;
    __shared__ __align__(8) uint64_t fin_all[2];  // bounded stand-ins for bar.sync among the convert warps
    __shared__ __align__(16) float red[(kVtGroups - 1) * 2 * MP * kVtRows];

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t grid = gridDim.x, cta = blockIdx.x;
    const uint32_t u0 = vt_range_begin(cta, c.total_units, grid), u1 = vt_range_begin(cta + 1, c.total_units, grid);
    const uint32_t row_bytes = (a.k / BlockTraits<T>::QK) * BlockTraits<T>::BYTES;

    if (warp == kVtCvtWarps && lane == 0) {
        // the producer's lane sets the barriers up and has the first weight stage on its way before the rest
        // of the CTA (tensor-memory allocation, the wait for the packing kernel) is ready
        abort_flag = 0;
        for (uint32_t s = 0; s < c.nslots; s++) {
            mbar_init(&raw_full[s], 1);
            mbar_init(&raw_empty[s], kVtCvtWarps + kVtMmaWarps);
        }
        for (int s = 0; s < 2 * kVtGroups; s++) {
            mbar_init(&a_full[s], 4);   // the four lane-quarter warps of a group
            mbar_init(&d_full[s], 1);
        }
        for (int s = 0; s < 2; s++) mbar_init(&fin_all[s], kVtCvtWarps);
        mbar_init_fence();
        if (!(MLXN_DBG(c) & 2u)) {
            VtWalk st;
            st.init(u0, u1, c.upt, c.cu, c.nslots);
            mbar_expect_tx(&raw_full[0], kVtRows * c.row_stride + st.cnt * (4 * 2048 + AUX));
            issue_weights(smem_u32(smem + c.raw_off), st.kun, st.tile, smem_u32(&raw_full[0]));
        }
    }
    if (warp == kVtCvtWarps + 1) {
        tmem_alloc(&tmem_base_s, kVtTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    const uint32_t smem_base = smem_u32(smem);
    allow_dependents();  // the next overlapped launch in the stream (its blocks wait for this grid before reading anything)
    const uint32_t wspin = (MLXN_DBG(c) & 64u) ? 0u : ((MLXN_DBG(c) & 128u) ? 40u : 0xFFFFFFFFu);   // MMA warps poll back to back (experiments: suspend / sleep)
    const uint32_t wdq = (MLXN_DBG(c) & 16u) ? 0xFFFFFFFFu : ((MLXN_DBG(c) & 32u) ? 20u : 0u);  // convert warps: suspend / spin / short sleeps

    if (warp == kVtCvtWarps) {
        // ======================= producer warp: one tensor copy of weights per stage + the packed activations =======================
        VtWalk st;
        for (st.init(u0, u1, c.upt, c.cu, c.nslots); !st.done(); st.next()) {
            const uint32_t slot = st.slot, sidx = st.sidx;
            if (sidx >= c.nslots && !mbar_wait(&raw_empty[slot], st.ph ^ 1u, &abort_flag, a.status, ST_WAIT_EMPTY_TIMEOUT, 0u))
                break;
            uint8_t *sl = smem + slot * c.slot_bytes;
            if (lane == 0) {
                if (MLXN_DBG(c) & 2u) {
                    mbar_arrive(&raw_full[slot]);  // experiment: no copies
                } else {
                    // one tensor copy brings the stage's 128 rows (rows past n arrive as zeros); the box is always
                    // cu units wide, a stage that uses fewer just ignores the rest (reads past a row's end are zeros too)
                    if (sidx != 0) {  // stage 0's weights were requested during set-up
                        mbar_expect_tx(&raw_full[slot], kVtRows * c.row_stride + st.cnt * (4 * 2048 + AUX));
                        issue_weights(smem_u32(sl + c.raw_off), st.kun, st.tile, smem_u32(&raw_full[slot]));
                    }
                    if (sidx == 0) grid_dependency_wait();  // the packed activations come from the kernel before
                    bulk_g2s(sl, sc.xpack + (size_t)st.kun * 4 * 2048, st.cnt * 4 * 2048, &raw_full[slot]);
                    bulk_g2s(sl + c.xs_off, sc.aux + (size_t)st.kun * AUX, st.cnt * AUX, &raw_full[slot]);
                }
            }
            __syncwarp();
        }
    } else if (warp > kVtCvtWarps) {
        // ======================= MMA warps: warp w2 serves groups w2 and w2 + 2 =======================
        grid_dependency_wait();
        if (lane == 0) {
            const uint32_t w2 = warp - kVtCvtWarps - 1;
            constexpr uint32_t idesc = umma_idesc_f16(kVtRows, 16);
            uint32_t uc = 0;
            bool ok = true;
            VtWalk st;
            for (st.init(u0, u1, c.upt, c.cu, c.nslots); ok && !st.done(); st.next()) {
                const uint32_t slot = st.slot;
                if (!mbar_wait(&raw_full[slot], st.ph, &abort_flag, a.status, ST_WAIT_FULL_TIMEOUT, wspin)) break;
                const uint64_t bd0 = umma_desc_k_sw128(smem_base + slot * c.slot_bytes);
                for (uint32_t ul = 0; ok && ul < st.cnt; ul++) {
#pragma unroll
                    for (uint32_t n = 0; n < (uint32_t)SS; n++, uc++) {   // uc counts sub-steps per group
                        const uint32_t p = uc & 1u, par = (uc >> 1) & 1u;
#pragma unroll
                        for (uint32_t h = 0; h < 2; h++) {
                            const uint32_t g = w2 + 2 * h, sl = 2 * g + p;
                            if (!mbar_wait(&a_full[sl], par, &abort_flag, a.status, ST_WAIT_FULL_TIMEOUT, wspin)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after();
                            const uint32_t acol = tmem + sl * kVtSlotCols, dcol = acol + 32;
                            if (!(MLXN_DBG(c) & 4u)) {
                                if constexpr (T == GT_Q6_K) {
                                    // sub-step ss = 4 n + g: 32 K = half of 64-wide chunk ss / 2; one MMA per scale group
                                    const uint32_t ss = 4 * n + g;
                                    const uint64_t bd = bd0 + (uint64_t)((ul * 4 + (ss >> 1)) * (2048 >> 4) + (ss & 1u) * 4);
                                    umma_f16_ts(dcol, acol, bd, idesc, 0u);
                                    umma_f16_ts(dcol + 16, acol + 8, bd + 2, idesc, 0u);
                                } else {
                                    const uint64_t bd = bd0 + (uint64_t)((ul * 4 + g) * (2048 >> 4));
                                    umma_f16_ts(dcol, acol, bd, idesc, 0u);
                                    umma_f16_ts(dcol, acol + 8, bd + 2, idesc, 1u);
                                    umma_f16_ts(dcol + 16, acol + 16, bd + 4, idesc, 0u);
                                    umma_f16_ts(dcol + 16, acol + 24, bd + 6, idesc, 1u);
                                }
                            }
                            umma_commit(&d_full[sl]);
                        }
                        if (!ok) break;
                    }
                }
                if (ok) umma_commit(&raw_empty[slot]);  // this warp's MMAs no longer read the stage's activation tiles
            }
        }
        __syncwarp();
    } else {
        // ======================= convert + readout warps =======================
        // Thread (warp w, lane l): group g = w / 4 owns sub-step g (64 K) of every K unit; the thread owns
        // weight row 32 (w % 4) + l of the tile, which is also the tensor-memory lane its warp may address.
        grid_dependency_wait();
        const uint32_t q4 = warp & 3u, g = warp >> 2;
        const uint32_t row = q4 * 32 + lane;
        const uint32_t lane_base = tmem + ((q4 * 32) << 16);
        uint64_t acc[MP];
#pragma unroll
        for (int i = 0; i < MP; i++) acc[i] = 0ull;

        // previous unit, whose accumulators are read back while the MMA works on the current one
        bool pv = false, pv_stage_end = false, pv_seg_end = false;
        uint32_t pv_sl = 0, pv_par = 0, pv_xs = 0, pv_ts = 0, pv_slot = 0, pv_tile = 0, pv_ka = 0, pv_kb = 0;
        float pv_d0 = 0.f, pv_d1 = 0.f;
        uint32_t seg_ka = 0;  // first unit (within the tile) of the running segment
        bool ok = true;

        auto readout = [&]() {
            if (!mbar_wait(&d_full[pv_sl], pv_par, &abort_flag, a.status, ST_WAIT_MMA_TIMEOUT, wdq)) {
                ok = false;
                return;
            }
            tc_fence_after();
            uint32_t d[32];
            tmem_ld_32x32(lane_base + pv_sl * kVtSlotCols + 32, d);
            tmem_ld_wait();
            if (MLXN_DBG(c) & 1u) return;
            const uint64_t dd0 = pack2(pv_d0 * 16777216.0f, pv_d0 * 16777216.0f), dn0 = pack2(-kOff * pv_d0, -kOff * pv_d0);
            const uint64_t dd1 = pack2(pv_d1 * 16777216.0f, pv_d1 * 16777216.0f), dn1 = pack2(-kOff * pv_d1, -kOff * pv_d1);
#pragma unroll
            for (int i = 0; i < MP; i++) {
                uint32_t x0, x1, x2, x3, s0, s1;
                lds64(pv_xs + i * 8, x0, x1);          // block sums of the two blocks, rows 2i and 2i+1
                lds64(pv_xs + 32 + i * 8, x2, x3);
                lds64(pv_ts + i * 8, s0, s1);           // the half's scale for rows 2i and 2i+1
                const uint64_t sa = fadd2(pack2u(d[2 * i], d[2 * i + 1]), pack2u(d[8 + 2 * i], d[8 + 2 * i + 1]));
                const uint64_t sb = fadd2(pack2u(d[16 + 2 * i], d[16 + 2 * i + 1]), pack2u(d[24 + 2 * i], d[24 + 2 * i + 1]));
                uint64_t tsum = ffma2(dn0, pack2u(x0, x1), 0ull);
                tsum = ffma2(dd0, sa, tsum);
                tsum = ffma2(dn1, pack2u(x2, x3), tsum);
                tsum = ffma2(dd1, sb, tsum);
                acc[i] = ffma2(pack2u(s0, s1), tsum, acc[i]);
            }
        };
        // A barrier among the convert warps that gives up with the rest of the CTA instead of hanging:
        // every warp arrives once, everybody waits for the phase.
        uint32_t fin_ph = 0;
        auto sync_bounded = [&](uint64_t *bar, uint32_t ph) -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar);
            return mbar_wait(bar, ph, &abort_flag, a.status, ST_WAIT_EMPTY_TIMEOUT, 0xFFFFFFFFu);
        };
        // sums the four groups' accumulators of the finished segment and writes the tile's rows out
        auto finalize = [&]() {
            if (g != 0) {
#pragma unroll
                for (int i = 0; i < MP; i++) {
                    float lo, hi;
                    unpack2(acc[i], lo, hi);
                    red[((g - 1) * 2 * MP + 2 * i) * kVtRows + row] = lo;
                    red[((g - 1) * 2 * MP + 2 * i + 1) * kVtRows + row] = hi;
                }
            }
            if (!sync_bounded(&fin_all[0], fin_ph)) { ok = false; return; }
            if (g == 0) {
                float tot[2 * MP];
#pragma unroll
                for (int i = 0; i < MP; i++) unpack2(acc[i], tot[2 * i], tot[2 * i + 1]);
#pragma unroll
                for (int gg = 0; gg < kVtGroups - 1; gg++)
#pragma unroll
                    for (int i = 0; i < 2 * MP; i++) tot[i] += red[(gg * 2 * MP + i) * kVtRows + row];
                const uint32_t grow = pv_tile * kVtRows + ((T == GT_Q6_K && c.pairs) ? (row < kVtRows / 2 ? 2 * row : 2 * (row - kVtRows / 2) + 1) : row);
                const bool full = pv_ka == 0 && pv_kb == c.upt;
                const size_t ycol = (size_t)a.y_col0 + grow;
                const uint32_t ld = qmv_ld(a);
                if (full) {
                    if (grow < a.n)
#pragma unroll
                        for (int i = 0; i < 2 * MP; i++)
                            if ((uint32_t)i < a.m) {
                                a.y[(size_t)i * ld + ycol] = tot[i];
                                for (uint32_t pr = 0; pr < a.n_peer; pr++) a.y_peer[pr][(size_t)i * ld + ycol] = tot[i];
                            }
                } else if (grow < a.n) {
                    // the tile's K range is shared with other CTAs: add into the rows the packing kernel zeroed
#pragma unroll
                    for (int i = 0; i < 2 * MP; i++)
                        if ((uint32_t)i < a.m) {
                            atomicAdd(&a.y[(size_t)i * ld + ycol], tot[i]);
                            for (uint32_t pr = 0; pr < a.n_peer; pr++) atomicAdd(&a.y_peer[pr][(size_t)i * ld + ycol], tot[i]);
                        }
                }
            }
            if (!sync_bounded(&fin_all[1], fin_ph)) { ok = false; return; }
            fin_ph ^= 1u;
#pragma unroll
            for (int i = 0; i < MP; i++) acc[i] = 0ull;
        };
        auto retire_prev = [&]() {
            readout();
            if (!ok) return;
            if (pv_stage_end) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[pv_slot]);
            }
            if (pv_seg_end) finalize();
        };

        uint32_t uc = 0;
        VtWalk st;
        for (st.init(u0, u1, c.upt, c.cu, c.nslots); ok && !st.done(); st.next()) {
            const uint32_t slot = st.slot;
            if (!mbar_wait(&raw_full[slot], st.ph, &abort_flag, a.status, ST_WAIT_FULL_TIMEOUT, wdq)) break;
            if (st.kun == 0 || st.sidx == 0) seg_ka = st.kun;
            const uint32_t sl_base = smem_base + slot * c.slot_bytes;
            for (uint32_t ul = 0; ok && ul < st.cnt; ul++) {
#pragma unroll
                for (uint32_t n = 0; n < (uint32_t)SS; n++, uc++) {   // uc counts this group's sub-steps
                    if (!ok) break;
                    const uint32_t p = uc & 1u, sl = 2 * g + p;
                    float d0, d1;
                    // the slot's previous contents were consumed: its accumulators were read back two sub-steps ago
                    if constexpr (T == GT_Q6_K) {
                        uint32_t r[16];
                        // (pair mode: odd weight rows, stage rows 64-127 = lane quarters 2 and 3, start 8 bytes further
                        //  into their 16-byte chunk: four steps on in the lead-in sequence)
                        const uint32_t p8 = (st.kun + ul + ((c.pairs && q4 >= 2) ? 4u : 0u)) & 7u;
                        vt_extract_q6k_p(p8, sl_base + c.raw_off + row * c.row_stride, n, g, r, d0, d1);
                        tmem_st_32x32_x16(lane_base + sl * kVtSlotCols, r);
                    } else {
                        uint32_t r[32];
                        vt_extract_g<T>(g, sl_base + c.raw_off + row * c.row_stride + ul * UB, r, d0, d1);
                        tmem_st_32x32_x32(lane_base + sl * kVtSlotCols, r);
                    }
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_full[sl]);
                    if (pv) retire_prev();
                    pv = true;
                    pv_sl = sl;
                    pv_par = (uc >> 1) & 1u;
                    pv_d0 = d0;
                    pv_d1 = d1;
                    // sums of x for the sub-step's two scale groups, and the scale of its half of the unit
                    const uint32_t ss = T == GT_Q6_K ? 4 * n + g : g;
                    pv_xs = sl_base + c.xs_off + ul * AUX + 2 * ss * 32;
                    pv_ts = sl_base + c.xs_off + ul * AUX + (AUX - 64) + (T == GT_Q6_K ? n : (g >> 1)) * 32;
                    pv_slot = slot;
                    pv_stage_end = ul + 1 == st.cnt && n + 1 == (uint32_t)SS;
                    pv_seg_end = pv_stage_end && st.seg_end;
                    pv_tile = st.tile;
                    pv_ka = seg_ka;
                    pv_kb = st.kun + st.cnt;
                }
            }
        }
        if (ok && pv) retire_prev();
    }
    if (abort_flag) {  // let copies in flight land before the CTA's shared memory is released
        for (int i = 0; i < 200; i++) __nanosleep(5000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kVtCvtWarps + 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kVtTmemCols);
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static bool vt_have_encoder();
bool qmv_tc_supported(int ggml_type, const QmvArgs &a) {
    if (ggml_type != GT_Q4_0 && ggml_type != GT_Q8_0 && ggml_type != GT_Q6_K) return false;
    if (ggml_type == GT_Q6_K) {
        // rows of 210-byte super-blocks: every row on a 16-byte boundary (k % 2048 == 0), or every other row with the
        // rows between 8 bytes past one (k % 2048 == 1024: pairs of rows become the tensor map's rows; n even)
        const uint32_t rem = a.k % 2048;
        if (!(rem == 0 || (rem == 1024 && a.n % 2 == 0 && !exp_env("MLXN_VT_NO_PAIRS")))) return false;
    }
    if (a.ids || a.nprob != 1 || a.m < 1 || a.m > 8) return false;
    if (a.k % kVtUnitK != 0 || a.k == 0 || a.n == 0 || a.k / kVtUnitK > (uint32_t)kVtMaxUnits) return false;
    if ((uint64_t)a.m * a.n >= (1ull << 32)) return false;
    if (((uintptr_t)a.w & 15u) || ((uintptr_t)a.x & 15u)) return false;
    return vt_have_encoder();
}

static inline size_t vt_align(size_t v, size_t al) { return (v + al - 1) / al * al; }

// Scratch layout: packed activation tiles | per-unit block sums and scales.
size_t qmv_tc_scratch_bytes(const QmvArgs &a) {
    return vt_align((size_t)(a.k / 64) * 2048, 1024) + vt_align((size_t)(a.k / kVtUnitK) * 576, 1024);
}

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        (void)cudaGetLastError();
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

static bool vt_have_encoder() { return encode_tiled_fn() != nullptr; }

template <int T, int MP>
static cudaError_t launch_vt(const QmvArgs &a, const VtCfg &c, const VtScratch &sc, const CUtensorMap &wmap, uint32_t grid,
                             size_t smem, cudaStream_t st) {
    static size_t attr_smem[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (smem > attr_smem[dev]) {
        cudaError_t e = cudaFuncSetAttribute(qmv_tc_kernel<T, MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_smem[dev] = smem;
    }
    return launch_overlapped(qmv_tc_kernel<T, MP>, dim3(grid), dim3(kVtThreads), smem, st, a, c, sc, wmap);
}

template <int T>
static cudaError_t launch_vt_t(const QmvArgs &a, uint8_t *scratch, uint32_t *flags, int sm_count, cudaStream_t st, int *launches) {
    constexpr int UB = VtTraits<T>::UB;
    VtCfg c{};
    {
        const char *dbg = exp_env("MLXN_VT_DEBUG");
        c.debug = dbg ? (uint32_t)atoi(dbg) : 0u;
    }
    c.tiles = (a.n + kVtRows - 1) / kVtRows;
    c.upt = a.k / kVtUnitK;
    c.total_units = c.tiles * c.upt;
    // cu odd: the rows of a stage sit cu * UB bytes apart, an odd multiple of 16 bytes, so that the 16-byte reads
    // of eight consecutive rows fall into eight different bank groups
    c.cu = T == GT_Q4_0 ? 3u : 1u;
    if (const char *e = exp_env("MLXN_VT_CU")) {  // experiment switch
        const uint32_t v = (uint32_t)atoi(e);
        if (T != GT_Q6_K && v >= 1 && v <= 5 && v * UB / 4 <= 256) c.cu = v;
    }
    c.row_stride = T == GT_Q6_K ? (uint32_t)kVtQ6Box : c.cu * UB;
    c.xs_off = c.cu * 4 * 2048;
    c.raw_off = (uint32_t)vt_align(c.xs_off + c.cu * VtTraits<T>::AUX, 128);
    c.slot_bytes = (uint32_t)vt_align(c.raw_off + (size_t)kVtRows * c.row_stride, 1024);
    const uint32_t limit = 208 * 1024;
    c.nslots = limit / c.slot_bytes;
    if (c.nslots > (uint32_t)kVtMaxSlots) c.nslots = kVtMaxSlots;
    if (const char *e = exp_env("MLXN_VT_SLOTS")) {  // experiment switch
        const uint32_t v = (uint32_t)atoi(e);
        if (v >= 2 && v <= c.nslots) c.nslots = v;
    }
    if (c.nslots < 2) return cudaErrorInvalidConfiguration;
    const size_t smem = (size_t)c.nslots * c.slot_bytes + 1024;
    uint32_t grid = (uint32_t)sm_count;
    if (grid > (uint32_t)kVtMaxCtas) grid = kVtMaxCtas;
    if (grid > c.total_units) grid = c.total_units;

    VtScratch sc{};
    size_t off = 0;
    sc.xpack = scratch + off;
    off += vt_align((size_t)(a.k / 64) * 2048, 1024);
    sc.aux = scratch + off;
    (void)flags;

    // the weight matrix as a 2-D tensor of 32-bit words: [n rows][row_bytes / 4], box = 128 rows x cu units
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return cudaErrorNotSupported;
    const uint32_t row_bytes = (a.k / BlockTraits<T>::QK) * BlockTraits<T>::BYTES;
    alignas(64) CUtensorMap wmap;
    c.row_bytes = row_bytes;
    c.pairs = (T == GT_Q6_K && row_bytes % 16 != 0) ? 1u : 0u;
    {
        const cuuint64_t gdim[2] = {c.pairs ? row_bytes / 2 : row_bytes / 4, c.pairs ? a.n / 2 : a.n};
        const cuuint64_t gstride[1] = {c.pairs ? 2ull * row_bytes : row_bytes};
        const cuuint32_t box[2] = {c.row_stride / 4, (cuuint32_t)(c.pairs ? kVtRows / 2 : kVtRows)};
        const cuuint32_t estr[2] = {1, 1};
        if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t *>(a.w), gdim, gstride, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    cudaError_t e = launch_overlapped(qmv_tc_pack_kernel, dim3(c.upt, (2 * a.m + 3) / 4), dim3(128), 0, st, a, (int)T, sc, c.debug);
    (*launches)++;
    if (e != cudaSuccess) return e;
    (*launches)++;
    if (a.m <= 2) return launch_vt<T, 1>(a, c, sc, wmap, grid, smem, st);
    if (a.m <= 4) return launch_vt<T, 2>(a, c, sc, wmap, grid, smem, st);
    return launch_vt<T, 4>(a, c, sc, wmap, grid, smem, st);
}

// Row-sharded form: copies this rank's columns of the result into the other ranks' result buffers.  The mat-vec
// kernel adds split tiles up with atomics, which are slow on peer memory; a plain copy of the finished columns is not.
__global__ void __launch_bounds__(256) qmv_publish_kernel(const QmvArgs a) {
    grid_dependency_wait();  // the mat-vec kernel ahead has finished
    allow_dependents();
    const uint32_t total = a.m * a.n, ld = qmv_ld(a);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const uint32_t t = i / a.n, col = i - t * a.n;
        const size_t off = (size_t)t * ld + a.y_col0 + col;
        const float v = a.y[off];
        for (uint32_t pr = 0; pr < a.n_peer; pr++) a.y_peer[pr][off] = v;
    }
}

// `pub_st` / `pub_ev` (optional): for the row-sharded form, run the copy to the peers on a stream of its own behind an
// event instead of on `st`.  (Measured on two GPUs: slower than leaving it on `st`, where it is a programmatic
// dependent of the mat-vec kernel; the runtime passes null.)
cudaError_t launch_qmv_tc(int ggml_type, const QmvArgs &a, uint8_t *scratch, uint32_t *flags, int sm_count, cudaStream_t st,
                          cudaStream_t pub_st, cudaEvent_t pub_ev, int *launches) {
    QmvArgs loc = a;
    loc.n_peer = 0;  // the mat-vec itself writes this rank's buffer only
    cudaError_t e;
    switch (ggml_type) {
    case GT_Q4_0: e = launch_vt_t<GT_Q4_0>(loc, scratch, flags, sm_count, st, launches); break;
    case GT_Q8_0: e = launch_vt_t<GT_Q8_0>(loc, scratch, flags, sm_count, st, launches); break;
    case GT_Q6_K: e = launch_vt_t<GT_Q6_K>(loc, scratch, flags, sm_count, st, launches); break;
    default: return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess || a.n_peer == 0) return e;
    const uint32_t total = a.m * a.n;
    uint32_t blocks = (total + 255) / 256;
    if (blocks > 64) blocks = 64;
    (*launches)++;
    if (!pub_st) return launch_overlapped(qmv_publish_kernel, dim3(blocks), dim3(256), 0, st, a);
    if ((e = cudaEventRecord(pub_ev, st)) != cudaSuccess) return e;
    if ((e = cudaStreamWaitEvent(pub_st, pub_ev, 0)) != cudaSuccess) return e;
    qmv_publish_kernel<<<blocks, 256, 0, pub_st>>>(a);
    return cudaGetLastError();
}

}  // namespace mlxn
