// Register-level mat-vec for 1..8 activation rows (decode): y[m, n] = x[m, k] . W[n, k]^T with W in GGML blocks.
//
// Replaces upstream kernel_mul_mv_{q4_0,q8_0,q6_K}_f32 (src/shaders/quantized_matmul_ggml.metal:104-330), and for a
// handful of (token, slot) rows kernel_mul_mv_id_* and its fused SwiGLU form (src/shaders/quantized_matmul_id_ggml.metal).
// The operation is bound by the weight stream, so the kernel is organised around these things:
//
//  * One launch, no scratch memory, no atomics on results.  The activations are split into f16 hi + lo halves inside
//    the kernel (per block of 32 / scale group of 16, pre-scaled by a power of two so that both halves stay f16
//    normals whatever the magnitudes), and every output element is written exactly once by one CTA, so results are
//    bit-reproducible and there is nothing to zero or to combine afterwards.
//  * The multiply-adds run on the tensor cores from registers (mma.sync m16n8k16, f16 x f16 -> f32).  The weights
//    enter as *exact integers*: the raw 4/6/8-bit codes written as f16 subnormals (n * 2^-24; about one bit operation
//    per pair of codes, no conversion instruction).  A 16-row weight tile is the A operand.  The 8 columns of B are
//    (activation row, f16 half): column 2 r holds the hi halves of activation row r, column 2 r + 1 the lo halves, so
//    one multiply yields both partial sums of up to four activation rows (two "sets" for five to eight).  The codes
//    are unsigned; the bias (8, 32, 128) times the block's activation sum is added with the block's scale.
//  * The weights arrive through a shared-memory ring filled by 2-D tensor-map copies (TMA) of R rows x one K stage,
//    with an L2 evict-first hint (they pass once); the activations are re-read by every item and carry evict-last.
//    There is no producer warp: thread 0 fills the ring at the start and afterwards the warp that is the last of the
//    eight to release a slot issues the copy of the stage that gets the slot next.  A CTA is 8 warps, 128 registers
//    and about 112 KB of shared memory, two per SM.  Launched as a programmatic dependent, the next mat-vec in the
//    stream fills its ring with weights while the one ahead is still running.
//  * Q4_0 / Q8_0 blocks are worked on in pairs: the even block of a pair starts on a 4-byte boundary, lanes 1..3 read
//    whole words of its codes and lane 0 the two half words at either end, which sit in the words that also hold the
//    pair's two f16 scales (so with one activation row the scales cost no load).  All shared-memory offsets inside a
//    stage are compile-time constants of the instructions.
//  * One launch carries up to 16 mat-vecs of the same block type (MwBatch): conflict-free neighbours of an encoder
//    share one work list cut into chunks of equal numbers of stages.  Optionally (dep_mask) mat-vecs that depend on one
//    another ride in one cooperative launch with a bounded barrier across the grid between them.
//
// Work split: an item is R = 16 * TPW weight rows over all of K; inside a CTA the eight warps split every stage along
// K (Q4_0 / Q8_0: warp w owns blocks KB w .. KB w + KB - 1 of the stage's 8 KB; Q6_K: one (super-block parity, half,
// 16-column strip) of the stage's 2 KB super-blocks), each keeping TPW accumulator tiles; at the end of an item the
// eight partial sums per output are added in a fixed order through shared memory.
//
// Supported: Q4_0 / Q8_0 with k % 256 == 0, Q6_K with k % 512 == 0; weight rows that start on 16-byte boundaries
// (Q6_K also rows of 16 j + 8 bytes, in pairs).  Everything else takes the other mat-vec kernels.
#include "tensor_map.cuh"

#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace mlxn {

constexpr int kMwWarps = 8;                         // consumer warps
constexpr int kMwThreads = kMwWarps * 32;
constexpr int kMwMaxSlots = 12;

// A "unit" is what one warp multiplies per tile and K step: one block of 32 (Q4_0 / Q8_0: two MMAs, one scale)
// or one quarter of a Q6_K super-block (one half nh, one 16-column strip js: four MMAs, four scale groups).
// UBYTES: bytes of a stage per row and per unit-of-every-warp (8 blocks, or 2 super-blocks).  OFFSET: code bias.
// NG: scale groups (accumulator starts) per unit.  NM: MMAs per unit (each wants 4 activation values per lane).
template <int T> struct MwTraits;
template <> struct MwTraits<GT_Q4_0> { static constexpr int UK = 256, UBYTES = 144, OFFSET = 8, NG = 1, NM = 2; };
template <> struct MwTraits<GT_Q8_0> { static constexpr int UK = 256, UBYTES = 272, OFFSET = 128, NG = 1, NM = 2; };
template <> struct MwTraits<GT_Q6_K> { static constexpr int UK = 512, UBYTES = 420, OFFSET = 32, NG = 4, NM = 4; };
// Q4_K: a unit is one PAIR of 32-value sub-blocks of a super-block (32 bytes: low nibbles = the first sub-block, high
// nibbles = the second; four MMAs, two scale groups).  The codes carry no bias; the sub-block's minimum dmin * m is
// subtracted through the activation sum (OFFSET 1 is the weight of that sum).
template <> struct MwTraits<GT_Q4_K> { static constexpr int UK = 512, UBYTES = 288, OFFSET = 1, NG = 2, NM = 4; };
// Q5_K: as Q4_K with a fifth code bit per value from the super-block's 32 qh bytes (176-byte super-blocks); both
// sub-blocks' codes are brought down to plain 5-bit values, so neither needs its activations rescaled.
template <> struct MwTraits<GT_Q5_K> { static constexpr int UK = 512, UBYTES = 352, OFFSET = 1, NG = 2, NM = 4; };

// Shared-memory bytes per row of a stage of KB units per warp: the stage's bytes plus the up to 12 bytes between
// the 16-byte boundary the copy starts at and the stage's first byte (Q6_K), rounded up to an ODD multiple of 16,
// so that the 32-bit reads of eight consecutive rows fall into distinct banks.
// A tensor copy is at most 256 elements (2048 bytes) wide: a longer stage row arrives as two copies, the first half of
// the stage's K range for warps 0..3 and the second for warps 4..7, each into its own R x PITCH region of the slot.
__host__ __device__ constexpr uint32_t mw_halves(int ggml_type, int kb) {
    return (ggml_type == GT_Q4_0 ? 144u : ggml_type == GT_Q8_0 ? 272u : ggml_type == GT_Q4_K ? 288u : ggml_type == GT_Q5_K ? 352u : 420u) * (uint32_t)kb + 12u > 2048u ? 2u : 1u;
}
__host__ __device__ constexpr uint32_t mw_pitch(int ggml_type, int kb) {
    const uint32_t raw = (ggml_type == GT_Q4_0 ? 144u : ggml_type == GT_Q8_0 ? 272u : ggml_type == GT_Q4_K ? 288u : ggml_type == GT_Q5_K ? 352u : 420u) * (uint32_t)kb / mw_halves(ggml_type, kb);
    const uint32_t lead = ggml_type == GT_Q6_K ? (kb == 1 ? 12u : 8u) : 0u;
    const uint32_t c = (raw + lead + 15u) / 16u;
    return 16u * (c | 1u);
}

constexpr int kMwMaxProbs = 16;    // mat-vecs one launch can carry
constexpr int kMwMaxGrid = 320;    // CTAs of a launch (two per SM)

// One mat-vec of a launch.  A launch carries up to kMwMaxProbs mat-vecs that have no buffer conflicts with one
// another (same block type and kernel configuration); their row groups form one list of work items.
struct MwProb {
    const float *x;
    const float *x2;      // fused SwiGLU: the activations are silu(x) * x2 (nullptr: x as it is)
    const uint32_t *ids;  // expert-routed: the weights are those of expert ids[id_idx] of the stacked tensor (3-D map)
    uint32_t id_idx;
    float *y;
    uint32_t n, k, m;
    uint32_t spi;         // stages per item = k / (KB * UK)
    uint32_t item0;       // index of the problem's first item in the launch's item list
    uint32_t y_ld, y_col0;
    uint32_t n_peer;      // row-sharded form (see QmvArgs): the other ranks' result buffers
    float *y_peer[kMaxPeers];
};
struct MwBatch {
    MwProb p[kMwMaxProbs];
    uint32_t nprob;
    uint32_t early_weights;   // no problem's weights were written by a kernel of this process (see QmvArgs)
    uint32_t *status;
    uint32_t nitems;          // items of all problems
    // Dependent form (dep_mask != 0; a cooperative launch): bit p set = problem p starts only after every CTA has
    // finished all the problems before it.  Every problem's items are then spread over all CTAs (CTA c takes
    // items [c I / G, (c + 1) I / G) of a problem with I items), and the weights of the problems ahead keep streaming
    // into the ring while a CTA waits.  bar[p] counts the CTAs that are done with the problems before p; bar[31] the
    // CTAs that have left (the last one zeroes the block for the next launch).
    uint32_t dep_mask;
    uint32_t *bar;
    uint32_t routed;          // some problem is expert-routed: the expert ids are read once the kernels ahead are done
    // CTA c works on items [cta_begin[c], cta_begin[c + 1]): contiguous chunks of (nearly) equal numbers of stages
    uint32_t cta_begin[kMwMaxGrid + 1];
};
struct MwMaps {
    CUtensorMap m[kMwMaxProbs];
};

struct MwCfg {
#ifdef MLXN_EXPERIMENTS
    uint32_t debug;       // 1: consumers only wait and release (no arithmetic); 2: no copies (arithmetic on stale data);
                          // 4: no activation conversion; 8: no Q6_K scale table
#endif
    uint32_t nslots;      // ring depth
    uint32_t xst_off;     // shared-memory offsets behind the ring
    uint32_t ptab_off;
    uint32_t red_off;
};

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// Loads at a compile-time offset from a register address (the offset travels in the instruction: no address arithmetic)
template <uint32_t OFF> __device__ __forceinline__ uint32_t lds32i(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}
template <uint32_t OFF> __device__ __forceinline__ uint32_t lds_u16i(uint32_t addr) {
    uint32_t v;
    asm volatile("{ .reg .u16 t; ld.shared.u16 t, [%1+%2]; cvt.u32.u16 %0, t; }" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}
template <uint32_t OFF> __device__ __forceinline__ void lds64i(uint32_t addr, uint32_t &a, uint32_t &b) {
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2+%3];" : "=r"(a), "=r"(b) : "r"(addr), "n"(OFF));
}
template <uint32_t OFF> __device__ __forceinline__ void lds128i(uint32_t addr, uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d) {
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr), "n"(OFF));
}
// The f16 in the low / high half of a 32-bit word, as f32
__device__ __forceinline__ float f16lo_to_float(uint32_t w) {
    float f;
    asm("{ .reg .f16 l, h; mov.b32 {l, h}, %1; cvt.f32.f16 %0, l; }" : "=f"(f) : "r"(w));
    return f;
}
__device__ __forceinline__ float f16hi_to_float(uint32_t w) {
    float f;
    asm("{ .reg .f16 l, h; mov.b32 {l, h}, %1; cvt.f32.f16 %0, h; }" : "=f"(f) : "r"(w));
    return f;
}
// f(integral_constant<int, I>) for I = 0 .. N - 1: loop bodies whose shared-memory offsets must be compile-time constants
template <int I, int N, class F> __device__ __forceinline__ void static_for(F &&f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<I + 1, N>(f);
    }
}

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.b32 [%0], {%1,%2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t a) {
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(a) : "memory");
}

// D = A (16 x 16, row) * B (16 x 8, col) + C, f16 operands, f32 accumulate.  Lane (g = lane / 4, t = lane % 4):
// a0 = A[g][2t, 2t+1], a1 = A[g+8][2t, 2t+1], a2 = A[g][2t+8, 2t+9], a3 = A[g+8][2t+8, 2t+9];
// b0 = B[2t, 2t+1][g], b1 = B[2t+8, 2t+9][g]; c0 = C[g][2t], c1 = C[g][2t+1], c2 = C[g+8][2t], c3 = C[g+8][2t+1].
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1, const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

__device__ __forceinline__ uint32_t h2_bits(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// Four activation values (scaled) -> the B registers of one MMA: hi halves (e0, e2), (e1, e3) and the f16 residues.
// The pairing follows the code extraction: a 32-bit word of four codes (c0..c3) becomes the A registers (c0, c2)
// and (c1, c3).
__device__ __forceinline__ void split4(float e0, float e1, float e2, float e3, uint32_t &bh0, uint32_t &bh1, uint32_t &bl0,
                                       uint32_t &bl1) {
    const __half2 h02 = __floats2half2_rn(e0, e2), h13 = __floats2half2_rn(e1, e3);
    const float2 f02 = __half22float2(h02), f13 = __half22float2(h13);
    bh0 = *reinterpret_cast<const uint32_t *>(&h02);
    bh1 = *reinterpret_cast<const uint32_t *>(&h13);
    bl0 = h2_bits(e0 - f02.x, e2 - f02.y);
    bl1 = h2_bits(e1 - f13.x, e3 - f13.y);
}

// Power of two that brings `amax` into [2^13, 2^14), and its inverse; 1 for an all-zero or non-finite run.
__device__ __forceinline__ void pow2_scale(float amax, float &s, float &inv) {
    s = 1.f;
    inv = 1.f;
    if (amax > 0.f && amax < 3.0e38f) {
        int e = 13 + 127 - (int)((__float_as_uint(amax) >> 23) & 0xffu);
        e = max(-100, min(100, e));
        s = __uint_as_float((uint32_t)(e + 127) << 23);
        inv = __uint_as_float((uint32_t)(127 - e) << 23);
    }
}

// Which elements of its block (Q4_0 / Q8_0) lane t multiplies in MMA `h` (0, 1) of the block, as two pairs of
// consecutive elements.  The blocks of a row are worked on in pairs (even, odd index inside the stage): the even
// block starts on a 4-byte boundary, so its codes (2 bytes in) straddle the 32-bit words.  There lanes t = 1..3 take
// whole words and lane 0 the two half words at either end of the codes (which sit in the words that also hold the
// pair's two f16 scales).  The odd block's codes are word-aligned.  `mis` = the even block.
__device__ __forceinline__ void mw_pairs(int ggml_type, bool mis, uint32_t t, uint32_t h, uint32_t &p0, uint32_t &p1) {
    if (ggml_type == GT_Q8_0) {
        if (!mis) { p0 = 16 * h + 4 * t; p1 = p0 + 2; }
        else if (h == 0) { p0 = t ? 4 * t - 2 : 0; p1 = t ? 4 * t : 30; }
        else { p0 = 14 + 4 * t; p1 = 16 + 4 * t; }
    } else {  // Q4_0: byte c holds element c (low nibble, MMA 0) and 16 + c (high nibble, MMA 1)
        if (!mis) { p0 = 4 * t; p1 = 4 * t + 2; }
        else { p0 = t ? 4 * t - 2 : 0; p1 = t ? 4 * t : 14; }
        p0 += 16 * h;
        p1 += 16 * h;
    }
}

// A pair of blocks (even, odd index inside the stage; 2 x 32 values) against the warp's TPW tiles.
// `base` = shared address of the pair in row g of the stage + 4 t; `base2`: lanes 1..3 the same, lane 0 the word that
// holds the last two codes of the even block (and the odd block's scale); `sel`: the byte permute that joins lane 0's
// two half words (identity in the other lanes); `rbs`: the pair's address in row g (scales, more than one activation
// row only: with one, the scales are needed in lane 0 alone, which has them in the words it reads anyway).
//
// The 8 columns of an MMA are (activation row, f16 half): column 2 r holds the hi halves of activation row r (of the
// set's four), column 2 r + 1 the lo halves, so ONE multiply gives both partial sums and lane t ends up with those of
// activation row t: (hi, lo) for weight row g and (hi, lo) for weight row g + 8.  NS = 2 sets for 5..8 activation rows.
// bf0 / bf1: the B registers of the two blocks' MMAs [set][MMA of the block][2]; cc: -offset sum(x), cs: inverse
// activation pre-scale of this lane's activation row [set][block] (the codes enter unsigned, so every block owes
// scale x cc).  All other rows are compile-time offsets from these addresses.
template <int T, int TPW, int MP, int NS, uint32_t PITCH, uint32_t IOFF>
__device__ __forceinline__ void mw_pair_tiles(uint32_t base, uint32_t base2, uint32_t rbs, uint32_t sel,
                                              const uint32_t (&bf0)[NS][2][2], const uint32_t (&bf1)[NS][2][2],
                                              const float (&cc)[NS][2], const float (&cs)[NS][2], float (&acc)[TPW][NS][4]) {
    const float zz[4] = {0.f, 0.f, 0.f, 0.f};
    constexpr uint32_t BB = T == GT_Q8_0 ? 34u : 18u;
    static_for<0, TPW>([&](auto J) {
        constexpr uint32_t j = decltype(J)::value;
        uint32_t w0[2], w1[2], w2[2], w3[2];   // [row g, row g + 8]
        float d0[2], d1[2];
        static_for<0, 2>([&](auto H) {
            constexpr uint32_t h = decltype(H)::value, OFF = (16 * j + 8 * h) * PITCH + IOFF;
            const uint32_t s0 = lds32i<OFF>(base), s1 = lds32i<OFF>(base2);
            w0[h] = __byte_perm(s0, s1, sel);
            if constexpr (T == GT_Q8_0) {
                w1[h] = lds32i<OFF + 16>(base);
                w2[h] = lds32i<OFF + 36>(base);
                w3[h] = lds32i<OFF + 52>(base);
            } else {
                w1[h] = lds32i<OFF + 20>(base);
                w2[h] = w3[h] = 0;
            }
            if constexpr (MP == 1) {
                d0[h] = f16lo_to_float(s0);
                d1[h] = f16hi_to_float(s1);
            } else {
                d0[h] = f16lo_to_float(lds_u16i<OFF>(rbs));
                d1[h] = f16lo_to_float(lds_u16i<OFF + BB>(rbs));
            }
        });
        uint32_t a[4][4];   // the A registers of the pair's four MMAs
        if constexpr (T == GT_Q8_0) {
            // codes + 128 as f16 subnormals: bytes 0, 2 and bytes 1, 3 of the word, each into the low byte of a half
            auto un = [&](uint32_t (&r)[4], uint32_t wg, uint32_t wg8) {
                const uint32_t x0 = wg ^ 0x80808080u, x1 = wg8 ^ 0x80808080u;
                r[0] = __byte_perm(x0, 0u, 0x4240); r[1] = __byte_perm(x1, 0u, 0x4240);
                r[2] = __byte_perm(x0, 0u, 0x4341); r[3] = __byte_perm(x1, 0u, 0x4341);
            };
            un(a[0], w0[0], w0[1]);
            un(a[1], w1[0], w1[1]);
            un(a[2], w2[0], w2[1]);
            un(a[3], w3[0], w3[1]);
        } else {
            // low nibbles: elements c0..c3 of the word's four bytes; high nibbles (x 16): 16 + c
            auto un = [&](uint32_t (&lo)[4], uint32_t (&hi)[4], uint32_t wg, uint32_t wg8) {
                lo[0] = wg & 0x000F000Fu; lo[2] = (wg >> 8) & 0x000F000Fu;
                lo[1] = wg8 & 0x000F000Fu; lo[3] = (wg8 >> 8) & 0x000F000Fu;
                hi[0] = wg & 0x00F000F0u; hi[2] = (wg >> 8) & 0x00F000F0u;
                hi[1] = wg8 & 0x00F000F0u; hi[3] = (wg8 >> 8) & 0x00F000F0u;
            };
            un(a[0], a[1], w0[0], w0[1]);
            un(a[2], a[3], w1[0], w1[1]);
        }
#pragma unroll
        for (int ns = 0; ns < NS; ns++) {
            float e0[4], e1[4];
            mma16816(e0, a[0][0], a[0][1], a[0][2], a[0][3], bf0[ns][0][0], bf0[ns][0][1], zz);
            mma16816(e1, a[2][0], a[2][1], a[2][2], a[2][3], bf1[ns][0][0], bf1[ns][0][1], zz);
            mma16816(e0, a[1][0], a[1][1], a[1][2], a[1][3], bf0[ns][1][0], bf0[ns][1][1], e0);
            mma16816(e1, a[3][0], a[3][1], a[3][2], a[3][3], bf1[ns][1][0], bf1[ns][1][1], e1);
            const float t00 = d0[0] * cs[ns][0], t01 = d0[1] * cs[ns][0], t10 = d1[0] * cs[ns][1], t11 = d1[1] * cs[ns][1];
            acc[j][ns][0] = fmaf(t00, e0[0], fmaf(d0[0], cc[ns][0], acc[j][ns][0]));
            acc[j][ns][1] = fmaf(t00, e0[1], acc[j][ns][1]);
            acc[j][ns][2] = fmaf(t01, e0[2], fmaf(d0[1], cc[ns][0], acc[j][ns][2]));
            acc[j][ns][3] = fmaf(t01, e0[3], acc[j][ns][3]);
            acc[j][ns][0] = fmaf(t10, e1[0], fmaf(d1[0], cc[ns][1], acc[j][ns][0]));
            acc[j][ns][1] = fmaf(t10, e1[1], acc[j][ns][1]);
            acc[j][ns][2] = fmaf(t11, e1[2], fmaf(d1[1], cc[ns][1], acc[j][ns][2]));
            acc[j][ns][3] = fmaf(t11, e1[3], acc[j][ns][3]);
        }
    });
}

// TPW: 16-row tiles per warp.  KB: units per warp and stage.  MP: activation rows carried (1, 2, 4 or 8, >= m).
// PAIR (Q6_K rows of 16 j + 8 bytes, e.g. k = 5120: only every other row starts on a 16-byte boundary): the tensor
// map's rows are PAIRS of weight rows; a stage is two copies of R / 2 map rows, the even weight rows into stage rows
// [0, R / 2) and the odd ones into [R / 2, R), each from the 16-byte boundary below its first byte (the odd rows'
// data therefore starts 8 bytes further into its chunk than the even rows').
template <int T, int TPW, int KB, int MP, bool PAIR>
__global__ void __launch_bounds__(kMwThreads, 2)
    qmv_mma_kernel(const __grid_constant__ MwBatch bt, const MwCfg c, const __grid_constant__ MwMaps maps) {
    using TR = MwTraits<T>;
    constexpr int R = 16 * TPW, NG = TR::NG, NM = TR::NM;
    constexpr int NS = MP > 4 ? 2 : 1;                       // sets of four activation rows
    constexpr uint32_t PITCH = mw_pitch(T, KB);
    constexpr uint32_t SBYTES = (uint32_t)TR::UBYTES * KB;   // bytes of a stage per row
    constexpr uint32_t SK = (uint32_t)TR::UK * KB;           // K values per stage
    constexpr uint32_t HV = mw_halves(T, KB);                // copies (K halves) per stage
    static_assert(HV == 1 || T != GT_Q6_K, "a Q6_K stage row fits one copy");
    constexpr uint32_t STAGE = HV * (uint32_t)R * PITCH;     // bytes per ring slot (a multiple of 256)
    // activation conversion: one "piece" = the four values a lane feeds to one MMA; a warp has KB * MP * NM * 4 of
    // them per stage, spread over its 32 lanes in NPASS passes
    constexpr int PIECES = KB * MP * NM * 4;
    // ... a stage with fewer than 32 pieces shares a conversion pass with the stages after it (NB stages per batch)
    constexpr int NB = PIECES >= 32 ? 1 : 32 / PIECES;
    constexpr int NPASS = (NB * PIECES + 31) / 32;
    constexpr int CCN = KB * MP * NG;                        // (ci, cs) pairs per stage
    constexpr uint32_t XCC = (uint32_t)NB * PIECES * 16;     // offset of the (ci, cs) table behind the pieces
    constexpr uint32_t XST = (XCC + (uint32_t)NB * CCN * 8 + 15u) & ~15u;   // the pieces are read 16 bytes at a time
    constexpr float kOff = -(float)TR::OFFSET / 16777216.0f;

    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);   // (tensor copies land on 128-byte boundaries)
    __shared__ __align__(8) uint64_t full[kMwMaxSlots], fin[2];
    __shared__ uint32_t rel[kMwMaxSlots];   // warps that have released the slot (counts up; a round is over at a multiple of 8)
    // this CTA's items [s_lo, s_hi) of every problem (counted from the problem's first item) and the number of the
    // CTA's first stage of the problem (s_q0[nprob]: all its stages)
    __shared__ uint32_t s_lo[kMwMaxProbs], s_hi[kMwMaxProbs], s_q0[kMwMaxProbs + 1];
    __shared__ uint32_t s_exp[kMwMaxProbs];   // expert of every routed problem
    __shared__ __align__(8) uint64_t gbar;  // dependent launches: warp 0 tells the others that the grid barrier is through
    __shared__ volatile uint32_t abort_flag;

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g0 = bt.cta_begin[blockIdx.x], g1 = bt.cta_begin[blockIdx.x + 1];   // this CTA's items

    if (tid == 0) {
        abort_flag = 0;
        for (uint32_t s = 0; s < c.nslots; s++) {
            mbar_init(&full[s], 1);
            rel[s] = 0;
        }
        mbar_init(&fin[0], kMwWarps);
        mbar_init(&fin[1], kMwWarps);
        mbar_init(&gbar, 1);
        mbar_init_fence();
    }
    if (tid >= 32 && tid < 32 + bt.nprob) {
        const uint32_t p2 = tid - 32;
        const uint32_t b = bt.p[p2].item0, e = p2 + 1 < bt.nprob ? bt.p[p2 + 1].item0 : bt.nitems;
        if (bt.dep_mask) {   // every problem's items spread over all CTAs
            s_lo[p2] = (uint32_t)(((uint64_t)blockIdx.x * (e - b)) / gridDim.x);
            s_hi[p2] = (uint32_t)(((uint64_t)(blockIdx.x + 1) * (e - b)) / gridDim.x);
        } else {             // one contiguous chunk of the launch's item list
            s_lo[p2] = max(g0, b) - b;
            s_hi[p2] = max(min(g1, e), max(g0, b)) - b;
        }
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t q = 0;
        for (uint32_t p2 = 0; p2 < bt.nprob; p2++) {
            s_q0[p2] = q;
            q += (s_hi[p2] - s_lo[p2]) * bt.p[p2].spi;
        }
        s_q0[bt.nprob] = q;
    }
    __syncthreads();
    allow_dependents();   // the next overlapped launch may become resident and fetch its weights

    const uint32_t smem_base = smem_u32(smem);
    // L2: the weights pass through once (first to go); the activations are read again by every item (last to go)
    uint64_t pol_w, pol_x;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol_w));
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol_x));

    // The tensor copy (R rows x one stage) of the CTA's stage number q into ring slot `slot`.  There is no producer
    // warp: thread 0 fills the ring at the start, and afterwards the warp that is the last to release a slot starts
    // the copy of the stage that uses the slot next.
    auto issue = [&](uint32_t q, uint32_t slot) {
        if (q >= s_q0[bt.nprob]) return;
        uint32_t p = 0;
        while (q >= s_q0[p + 1]) p++;
        const uint32_t spi = bt.p[p].spi, qq = q - s_q0[p];
        const uint32_t item = s_lo[p] + qq / spi, s = qq % spi;
#ifdef MLXN_EXPERIMENTS
        if (c.debug & 2u) {
            mbar_arrive(&full[slot]);
            return;
        }
#endif
        mbar_expect_tx(&full[slot], STAGE);
        // coordinates in 8-byte elements; rows past n and bytes past the end of a row arrive as zeros
        if constexpr (PAIR) {
            const uint32_t row_bytes = (bt.p[p].k / 256u) * 210u;
            const uint32_t xe = ((s * SBYTES) & ~15u) >> 3, xo = ((row_bytes + s * SBYTES) & ~15u) >> 3;
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
                ::"r"(smem_base + slot * STAGE), "l"(&maps.m[p]), "r"(xe), "r"(item * (uint32_t)(R / 2)), "r"(smem_u32(&full[slot])), "l"(pol_w)
                : "memory");
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
                ::"r"(smem_base + slot * STAGE + (R / 2) * PITCH), "l"(&maps.m[p]), "r"(xo), "r"(item * (uint32_t)(R / 2)),
                  "r"(smem_u32(&full[slot])), "l"(pol_w)
                : "memory");
        } else {
#pragma unroll
            for (uint32_t hv = 0; hv < HV; hv++) {
                const uint32_t x0 = ((s * SBYTES + hv * (SBYTES / HV)) & ~15u) >> 3;
                if (bt.p[p].ids) {   // [expert][row][bytes]: an expert id past the table reads as zeros
                    asm volatile(
                        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
                        ::"r"(smem_base + slot * STAGE + hv * (uint32_t)R * PITCH), "l"(&maps.m[p]), "r"(x0), "r"(item * (uint32_t)R),
                          "r"(s_exp[p]), "r"(smem_u32(&full[slot])), "l"(pol_w)
                        : "memory");
                    continue;
                }
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
                    ::"r"(smem_base + slot * STAGE + hv * (uint32_t)R * PITCH), "l"(&maps.m[p]), "r"(x0), "r"(item * (uint32_t)R),
                      "r"(smem_u32(&full[slot])), "l"(pol_w)
                    : "memory");
            }
        }
    };
    if (bt.routed) {
        grid_dependency_wait();   // the expert ids belong to the kernels ahead
        if (tid < bt.nprob) s_exp[tid] = bt.p[tid].ids ? __ldcg(bt.p[tid].ids + bt.p[tid].id_idx) : 0u;
        __syncthreads();
    }
    if (tid == 0) {
        if (!bt.early_weights) grid_dependency_wait();
        for (uint32_t q = 0; q < c.nslots; q++) issue(q, q);
    }

    {
        // ======================= consumers =======================
        const uint32_t g = lane >> 2, t = lane & 3u, w = warp;
        const uint32_t xst = smem_base + c.xst_off + w * XST;   // this warp's converted activations
        const uint32_t xcc = xst + XCC;
        const uint32_t ptab = smem_base + c.ptab_off + w * (R * 16 * KB);
        const uint32_t red = smem_base + c.red_off;

        // ---- geometry of the warp's units inside a stage ----
        // Q4_0 / Q8_0: blocks KB w .. KB w + KB - 1 of the stage's 8 KB; block b starts BB * b bytes into the row
        constexpr uint32_t BB = T == GT_Q8_0 ? 34u : 18u;
        // Q6_K: quarter (nh, js) of the super-blocks sp, sp + 2, ...; super-block sb starts lead + 210 sb bytes in
        const uint32_t sp = w >> 2, nh = (w >> 1) & 1u, js = w & 1u;
        const uint32_t q6A = 64 * nh + 16 * js + 4 * t, q6H = 128 + 32 * nh + 16 * js + 4 * t, q6S = 192 + 8 * nh + js;

        // ---- activation pieces this lane converts: batch piece bp = lane + 32 pass = so PIECES + pc ----
        // (so: stage of the batch)
        // Q4_0 / Q8_0: pc = ((i MP + r) NM + h) 4 + tt (unit i, activation row r, MMA h, quad lane tt);
        // Q6_K:        pc = ((i MP + r) 4 + q) 4 + tt (scale group q)
        uint32_t xrel0[NPASS], xrel1[NPASS], xrow[NPASS], xso[NPASS];   // element offsets inside a stage; activation row
        bool xin[NPASS];
#pragma unroll
        for (int p = 0; p < NPASS; p++) {
            const uint32_t bp = lane + 32 * p, pc = bp % PIECES;
            xso[p] = bp / PIECES;
            const uint32_t tt = pc & 3u, hq = (pc >> 2) % NM, ir = (pc >> 2) / NM;
            const uint32_t i = ir / MP;
            xrow[p] = ir % MP;
            xin[p] = bp < (uint32_t)(NB * PIECES);
            if constexpr (T == GT_Q6_K) {
                const uint32_t sb = sp + 2 * i;
                xrel0[p] = 256 * sb + 128 * nh + 32 * hq + 16 * js + 4 * tt;
                xrel1[p] = xrel0[p] + 2;
            } else if constexpr (T == GT_Q4_K || T == GT_Q5_K) {
                // MMA hq of the unit: sub-block hq / 2 of the pair (low / high nibbles), its elements 16 (hq % 2) + 4 tt ...
                const uint32_t sb = sp + 2 * i;
                xrel0[p] = 256 * sb + 64 * (w & 3u) + 32 * (hq >> 1) + 16 * (hq & 1u) + 4 * tt;
                xrel1[p] = xrel0[p] + 2;
            } else {
                const uint32_t b = KB * w + i;
                uint32_t p0, p1;
                mw_pairs(T, (b & 1u) == 0, tt, hq, p0, p1);
                xrel0[p] = 32 * b + p0;
                xrel1[p] = 32 * b + p1;
            }
        }
        // the problem being worked on
        uint32_t cur = 0xFFFFFFFFu, spi = 1, pm = 0, pk = 0;
        const float *xsrc0[NPASS], *xsrc1[NPASS];
        bool xok[NPASS];
        ptrdiff_t x2d = 0;   // fused SwiGLU: where the second operand sits relative to the first (elements)
        bool has2 = false;
        auto set_problem = [&](uint32_t p) {
            cur = p;
            spi = bt.p[p].spi;
            pm = bt.p[p].m;
            pk = bt.p[p].k;
            has2 = bt.p[p].x2 != nullptr;
            x2d = has2 ? bt.p[p].x2 - bt.p[p].x : 0;
#pragma unroll
            for (int q = 0; q < NPASS; q++) {
                xok[q] = xin[q] && xrow[q] < pm;
                const float *row = bt.p[p].x + (size_t)(xok[q] ? xrow[q] : 0) * bt.p[p].k;
                xsrc0[q] = row + xrel0[q];
                xsrc1[q] = row + xrel1[q];
            }
        };
        float xr[NPASS][4];
        // `s0` = K stage (inside the item) of the batch's first stage; every item starts at K = 0 again
        auto load_x = [&](uint32_t s0) {
#pragma unroll
            for (int p = 0; p < NPASS; p++) {
                uint32_t ks = s0 + xso[p];
                while (ks >= spi) ks -= spi;
                float2 v0 = make_float2(0.f, 0.f), v1 = v0;
                if (xok[p] && ks * SK + xrel0[p] < pk) {   // (the last stage of a row may reach past K: zeros there)
                    asm volatile("ld.global.cg.L2::cache_hint.v2.f32 {%0, %1}, [%2], %3;" : "=f"(v0.x), "=f"(v0.y) : "l"(xsrc0[p] + (size_t)ks * SK), "l"(pol_x));
                    asm volatile("ld.global.cg.L2::cache_hint.v2.f32 {%0, %1}, [%2], %3;" : "=f"(v1.x), "=f"(v1.y) : "l"(xsrc1[p] + (size_t)ks * SK), "l"(pol_x));
                }
                if (has2 && xok[p] && ks * SK + xrel0[p] < pk) {   // silu(gate) * up, as src/shaders/silu_mul.metal:17-30
                    float2 u0, u1;
                    asm volatile("ld.global.cg.L2::cache_hint.v2.f32 {%0, %1}, [%2], %3;" : "=f"(u0.x), "=f"(u0.y) : "l"(xsrc0[p] + (size_t)ks * SK + x2d), "l"(pol_x));
                    asm volatile("ld.global.cg.L2::cache_hint.v2.f32 {%0, %1}, [%2], %3;" : "=f"(u1.x), "=f"(u1.y) : "l"(xsrc1[p] + (size_t)ks * SK + x2d), "l"(pol_x));
                    v0.x = v0.x / (1.0f + expf(-v0.x)) * u0.x;
                    v0.y = v0.y / (1.0f + expf(-v0.y)) * u0.y;
                    v1.x = v1.x / (1.0f + expf(-v1.x)) * u1.x;
                    v1.y = v1.y / (1.0f + expf(-v1.y)) * u1.y;
                }
                xr[p][0] = v0.x; xr[p][1] = v0.y; xr[p][2] = v1.x; xr[p][3] = v1.y;
            }
        };
        // Splits the loaded values into f16 hi + lo and stores the lane's piece; per scale group (the 8 lanes of a
        // block, the 4 of a Q6_K group) also the accumulator start ci = -offset 2^-24 s sum(x) and cs = 1 / s, where
        // s is the power of two that brings the group's largest magnitude into [2^13, 2^14).
        auto convert_x = [&]() {
#pragma unroll
            for (int p = 0; p < NPASS; p++) {
                const uint32_t bp = lane + 32 * p;
                float am = fmaxf(fmaxf(fabsf(xr[p][0]), fabsf(xr[p][1])), fmaxf(fabsf(xr[p][2]), fabsf(xr[p][3])));
                float sum = (xr[p][0] + xr[p][1]) + (xr[p][2] + xr[p][3]);
                constexpr int RED = T == GT_Q6_K ? 2 : 4;   // xor distances 1, 2 (, 4)
#pragma unroll
                for (int o = 1; o <= RED; o <<= 1) {
                    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
                    sum += __shfl_xor_sync(0xffffffffu, sum, o);
                }
                float s, inv;
                pow2_scale(am, s, inv);
                // Q4_0: the high nibbles stay where they are in their byte (16 x the code): their activations / 16
                const float sv = ((T == GT_Q4_0 && ((bp >> 2) & 1u)) || (T == GT_Q4_K && ((bp >> 3) & 1u))) ? s * 0.0625f : s;
                uint32_t f0, f1, f2, f3;
                split4(xr[p][0] * sv, xr[p][1] * sv, xr[p][2] * sv, xr[p][3] * sv, f0, f1, f2, f3);
                if (bp < (uint32_t)(NB * PIECES)) {
                    sts128(xst + bp * 16, f0, f1, f2, f3);
                    // (the pieces of a scale group are consecutive, and PIECES is a multiple of the group size, so
                    //  bp / group size = so CCN + the group's index inside its stage)
                    if constexpr (T == GT_Q6_K) {
                        if ((bp & 3u) == 0) sts64(xcc + (bp >> 2) * 8, __float_as_uint(kOff * sum), __float_as_uint(inv));
                    } else {
                        if ((bp & 7u) == 0) sts64(xcc + (bp >> 3) * 8, __float_as_uint(kOff * sum), __float_as_uint(inv));
                    }
                }
            }
        };

        // Q6_K with one activation row: the bias term of the rows this lane builds the scale table for (row lane + 32 rr)
        float corr[(R + 31) / 32];
#pragma unroll
        for (int rr = 0; rr < (R + 31) / 32; rr++) corr[rr] = 0.f;
        // [tile][set][hi and lo partial sums of weight row g, of weight row g + 8] for activation row t + 4 set
        float acc[TPW][NS][4];
#pragma unroll
        for (int j = 0; j < TPW; j++)
#pragma unroll
            for (int ns = 0; ns < NS; ns++) acc[j][ns][0] = acc[j][ns][1] = acc[j][ns][2] = acc[j][ns][3] = 0.f;

        grid_dependency_wait();   // the activations belong to the kernels ahead until they are done

        uint32_t slot = 0, ph = 0, fin_ph = 0, bi = 0;   // bi: stage inside the conversion batch
        uint32_t qn = 0;                                 // the CTA's stages so far
        uint32_t gb_ph = 0;
        bool ok = true, first_item = true;
        for (uint32_t p = 0; ok && p < bt.nprob; p++) {
        const uint32_t item_lo = s_lo[p], item_hi = s_hi[p];
        if ((bt.dep_mask >> p) & 1u) {
            // The problem reads or overwrites results of the problems before it.  Every CTA reports, once, that its
            // share of those is written (also the CTAs that have no items here), then waits for all the others.
            if (warp == 0) {
                if (!first_item && !mbar_wait(&fin[1], fin_ph ^ 1u, &abort_flag, bt.status, ST_WAIT_EMPTY_TIMEOUT, 0u)) ok = false;
                if (ok && lane == 0) {
                    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(bt.bar + p) : "memory");
                    if (item_hi > item_lo) {   // one thread per CTA watches the counter; the other warps wait in shared memory
                        uint64_t t0 = 0;
                        for (uint32_t polls = 1;; polls++) {
                            uint32_t v;
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bt.bar + p) : "memory");
                            if (v >= gridDim.x) break;
                            __nanosleep(40);
                            if ((polls & 63u) == 0) {
                                if (abort_flag) break;
                                const uint64_t now = global_timer_ns();
                                if (t0 == 0) t0 = now;
                                else if (now - t0 > kWaitLimitNs) {
                                    abort_flag = 1;
                                    if (bt.status) atomicCAS(bt.status, 0u, (uint32_t)ST_WAIT_GRID_TIMEOUT);
                                    break;
                                }
                            }
                        }
                        mbar_arrive(&gbar);
                    }
                }
                __syncwarp();
            }
            if (item_hi > item_lo) {
                if (!mbar_wait(&gbar, gb_ph, &abort_flag, bt.status, ST_WAIT_GRID_TIMEOUT, 0u) || abort_flag) ok = false;
                gb_ph ^= 1u;
            }
        }
        for (uint32_t item = item_lo; ok && item < item_hi; item++) {
            if (p != cur) {   // first item, or the next mat-vec of the launch: its activations from K = 0
                set_problem(p);
                load_x(0);
                bi = 0;
            }
            for (uint32_t s = 0; ok && s < spi; s++) {
#ifdef MLXN_EXPERIMENTS
                if (bi == 0 && !(c.debug & 4u)) {
#else
                if (bi == 0) {
#endif
                    __syncwarp();           // the previous batch's pieces have all been fetched
                    convert_x();
                    __syncwarp();
                    load_x(s + NB);         // the next batch's values, consumed NB stages from now
                }
                const uint32_t xsb = xst + bi * (PIECES * 16), xcb = xcc + bi * (CCN * 8);
                bi = bi + 1 == (uint32_t)NB ? 0u : bi + 1;

                if (!mbar_wait(&full[slot], ph, &abort_flag, bt.status, ST_WAIT_FULL_TIMEOUT, 0u)) {
                    ok = false;
                    break;
                }
                const uint32_t stage = smem_base + slot * STAGE;
#ifdef MLXN_EXPERIMENTS
                if (c.debug & 1u) {
                    __syncwarp();
                    if (lane == 0) {   // the last of the eight warps to let go of the slot starts the copy of the stage that gets it next
                        uint32_t old;
                        asm volatile("atom.acq_rel.cta.shared.add.u32 %0, [%1], 1;" : "=r"(old) : "r"(smem_u32(&rel[slot])) : "memory");
                        if ((old & (uint32_t)(kMwWarps - 1)) == (uint32_t)(kMwWarps - 1)) issue(qn + c.nslots, slot);
                    }
                    qn++;
                    if (++slot == c.nslots) { slot = 0; ph ^= 1u; }
                    continue;
                }
#endif
                uint32_t lead = 0;
                if constexpr (T == GT_Q4_K || T == GT_Q5_K) {
                    constexpr uint32_t SBB = T == GT_Q4_K ? 144u : 176u;   // super-block bytes
                    // (d * sc, d * sc', dmin * m, dmin * m') of the warp's sub-block pair, for every row of the stage (lanes
                    // split the rows); the 6-bit scales and minima are unpacked as in src/gguf/mod.rs:440-452
                    const uint32_t pu = w & 3u;
#pragma unroll
                    for (int i = 0; i < KB; i++) {
#pragma unroll
                        for (int rr = 0; rr < (R + 31) / 32; rr++) {
                            const uint32_t r = lane + 32 * rr;
                            if (r < (uint32_t)R) {
                                const uint32_t rb = stage + r * PITCH + SBB * (sp + 2 * i);
                                const uint32_t dd = lds32(rb);
                                const float d = f16lo_to_float(dd), dmin = f16hi_to_float(dd);
                                const uint32_t s0 = lds32(rb + 4), s1 = lds32(rb + 8), s2 = lds32(rb + 12);   // scales[0..11]
                                uint32_t sc0, sc1, m0, m1;
                                if (pu < 2) {          // sub-blocks j = 2 pu, 2 pu + 1 < 4: sc = s[j] & 63, m = s[j + 4] & 63
                                    const uint32_t a = s0 >> (16 * pu), b = s1 >> (16 * pu);
                                    sc0 = a & 63u; sc1 = (a >> 8) & 63u;
                                    m0 = b & 63u; m1 = (b >> 8) & 63u;
                                } else {               // j >= 4: sc = (s[j + 4] & 15) | (s[j - 4] >> 6) << 4, m = (s[j + 4] >> 4) | (s[j] >> 6) << 4
                                    const uint32_t sh = 16 * (pu - 2);
                                    const uint32_t a = s2 >> sh, lo = s0 >> sh, hi = s1 >> sh;
                                    sc0 = (a & 15u) | (((lo >> 6) & 3u) << 4);
                                    sc1 = ((a >> 8) & 15u) | (((lo >> 14) & 3u) << 4);
                                    m0 = ((a >> 4) & 15u) | (((hi >> 6) & 3u) << 4);
                                    m1 = ((a >> 12) & 15u) | (((hi >> 14) & 3u) << 4);
                                }
                                sts128(ptab + (i * R + r) * 16, __float_as_uint(d * (float)sc0), __float_as_uint(d * (float)sc1),
                                       __float_as_uint(dmin * (float)m0), __float_as_uint(dmin * (float)m1));
                            }
                        }
                    }
                    __syncwarp();
                }
                if constexpr (T == GT_Q6_K) {
                    lead = (s * SBYTES) & 15u;   // a multiple of 4
                    // d * sub-scale of the warp's scale groups, for every row of the stage (lanes split the rows)
#ifdef MLXN_EXPERIMENTS
                    if (!(c.debug & 8u))
#endif
#pragma unroll
                    for (int i = 0; i < KB; i++) {
#pragma unroll
                        for (int rr = 0; rr < (R + 31) / 32; rr++) {
                            const uint32_t r = lane + 32 * rr;
                            if (r < (uint32_t)R) {
                                // (pair mode: logical row r sits in stage row (r & 1) R / 2 + r / 2, odd rows 8 bytes further in)
                                const uint32_t rb = PAIR ? stage + ((r & 1u) * (R / 2) + (r >> 1)) * PITCH + (lead ^ (8u * (r & 1u))) + 210 * (sp + 2 * i)
                                                         : stage + r * PITCH + lead + 210 * (sp + 2 * i);
                                const float d = half_bits_to_float(lds_u16(rb + 208));
                                float p[4];
#pragma unroll
                                for (int q = 0; q < 4; q++) p[q] = d * (float)lds_s8(rb + q6S + 2 * q);
                                if constexpr (MP == 1) {
                                    // one activation row: the groups' inverse pre-scales go into the table, and what the
                                    // row owes for the codes' bias (scale x -32 sum(x), over all groups) into `corr`
#pragma unroll
                                    for (int q = 0; q < 4; q++) {
                                        uint32_t u0, u1;
                                        lds64(xcb + (i * 4 + q) * 8, u0, u1);
                                        corr[rr] = fmaf(p[q], __uint_as_float(u0), corr[rr]);
                                        p[q] *= __uint_as_float(u1);
                                    }
                                }
                                sts128(ptab + (i * R + r) * 16, __float_as_uint(p[0]), __float_as_uint(p[1]), __float_as_uint(p[2]),
                                       __float_as_uint(p[3]));
                            }
                        }
                    }
                    __syncwarp();
                }

                // this lane's converted activations: column g of an MMA = (activation row g / 2, hi or lo half); the rows are
                // wrapped, the columns past 2 m are never looked at.  Its outputs belong to activation row t (+ 4 per set).
                const uint32_t xlane = xsb + ((((g >> 1) & (uint32_t)(MP - 1)) * NM * 4 + t) * 16) + (g & 1u) * 8;
                const uint32_t clane = xcb + (t & (uint32_t)(MP - 1)) * (NG * 8);
                if constexpr (T == GT_Q4_K || T == GT_Q5_K) {
                    constexpr bool Q5 = T == GT_Q5_K;
                    constexpr uint32_t SBB = Q5 ? 176u : 144u, QS0 = Q5 ? 48u : 16u;   // super-block bytes; where its nibbles start
                    // row g of the stage, the warp's first super-block, its pair of sub-blocks: 32 bytes of nibbles
                    // (Q5_K: and the 32 bytes of fifth bits 16 bytes in, bits 2 pu and 2 pu + 1 for the pair's two sub-blocks)
                    const uint32_t pu = w & 3u;
                    const uint32_t pQ = stage + g * PITCH + SBB * sp + QS0 + 32 * pu + 4 * t, pP = ptab + g * 16;
                    const uint32_t pH = stage + g * PITCH + SBB * sp + 16 + 4 * t;
                    const float zz[4] = {0.f, 0.f, 0.f, 0.f};
                    static_for<0, KB>([&](auto IC) {
                        constexpr uint32_t i = decltype(IC)::value;
                        uint32_t bf[NS][4][2];
                        float cc[NS][2], cs[NS][2];
                        static_for<0, NS>([&](auto SC) {
                            constexpr uint32_t ns = decltype(SC)::value;
                            static_for<0, 4>([&](auto QC) {
                                constexpr uint32_t q = decltype(QC)::value;
                                lds64i<(((i * MP + 4 * ns) * 4 + q) * 64)>(xlane, bf[ns][q][0], bf[ns][q][1]);
                            });
                            static_for<0, 2>([&](auto QC) {
                                constexpr uint32_t q = decltype(QC)::value;
                                uint32_t u0, u1;
                                lds64i<(((i * MP + 4 * ns) * 2 + q) * 8)>(clane, u0, u1);
                                cc[ns][q] = __uint_as_float(u0);
                                cs[ns][q] = __uint_as_float(u1);
                            });
                        });
                        static_for<0, TPW>([&](auto JC) {
                            constexpr uint32_t j = decltype(JC)::value;
                            uint32_t w0[2], w1[2], hb0[2] = {0, 0}, hb1[2] = {0, 0}, pv[2][4];
                            static_for<0, 2>([&](auto HC) {
                                constexpr uint32_t h = decltype(HC)::value;
                                constexpr uint32_t off = (16 * j + 8 * h) * PITCH + 2 * SBB * i;   // rows g, g + 8 of tile j
                                w0[h] = lds32i<off>(pQ);
                                w1[h] = lds32i<off + 16>(pQ);
                                if constexpr (Q5) {
                                    hb0[h] = lds32i<off>(pH) >> (2 * pu);
                                    hb1[h] = lds32i<off + 16>(pH) >> (2 * pu);
                                }
                                lds128i<((i * R) + 16 * j + 8 * h) * 16>(pP, pv[h][0], pv[h][1], pv[h][2], pv[h][3]);
                            });
                            uint32_t a[4][4];
                            if constexpr (Q5) {
                                // five-bit codes, one per byte: nibble | fifth bit << 4; then bytes 0, 2 and 1, 3 into halves
                                auto un5 = [&](uint32_t (&lo)[4], uint32_t (&hi)[4], int r0, uint32_t wg, uint32_t hg, uint32_t wg8, uint32_t hg8) {
                                    const uint32_t cA = (wg & 0x0F0F0F0Fu) | ((hg & 0x01010101u) << 4), cB = ((wg >> 4) & 0x0F0F0F0Fu) | ((hg & 0x02020202u) << 3);
                                    const uint32_t dA = (wg8 & 0x0F0F0F0Fu) | ((hg8 & 0x01010101u) << 4), dB = ((wg8 >> 4) & 0x0F0F0F0Fu) | ((hg8 & 0x02020202u) << 3);
                                    (void)r0;
                                    lo[0] = __byte_perm(cA, 0u, 0x4240); lo[2] = __byte_perm(cA, 0u, 0x4341);
                                    lo[1] = __byte_perm(dA, 0u, 0x4240); lo[3] = __byte_perm(dA, 0u, 0x4341);
                                    hi[0] = __byte_perm(cB, 0u, 0x4240); hi[2] = __byte_perm(cB, 0u, 0x4341);
                                    hi[1] = __byte_perm(dB, 0u, 0x4240); hi[3] = __byte_perm(dB, 0u, 0x4341);
                                };
                                un5(a[0], a[2], 0, w0[0], hb0[0], w0[1], hb0[1]);
                                un5(a[1], a[3], 0, w1[0], hb1[0], w1[1], hb1[1]);
                            } else {
                            // low nibbles: first sub-block, elements c0..c3 of the word's bytes; high nibbles (x 16): the second
                            a[0][0] = w0[0] & 0x000F000Fu; a[0][2] = (w0[0] >> 8) & 0x000F000Fu;
                            a[0][1] = w0[1] & 0x000F000Fu; a[0][3] = (w0[1] >> 8) & 0x000F000Fu;
                            a[1][0] = w1[0] & 0x000F000Fu; a[1][2] = (w1[0] >> 8) & 0x000F000Fu;
                            a[1][1] = w1[1] & 0x000F000Fu; a[1][3] = (w1[1] >> 8) & 0x000F000Fu;
                            a[2][0] = w0[0] & 0x00F000F0u; a[2][2] = (w0[0] >> 8) & 0x00F000F0u;
                            a[2][1] = w0[1] & 0x00F000F0u; a[2][3] = (w0[1] >> 8) & 0x00F000F0u;
                            a[3][0] = w1[0] & 0x00F000F0u; a[3][2] = (w1[0] >> 8) & 0x00F000F0u;
                            a[3][1] = w1[1] & 0x00F000F0u; a[3][3] = (w1[1] >> 8) & 0x00F000F0u;
                            }
                            const float pa0 = __uint_as_float(pv[0][0]), pa1 = __uint_as_float(pv[0][1]), ma0 = __uint_as_float(pv[0][2]),
                                        ma1 = __uint_as_float(pv[0][3]);
                            const float pb0 = __uint_as_float(pv[1][0]), pb1 = __uint_as_float(pv[1][1]), mb0 = __uint_as_float(pv[1][2]),
                                        mb1 = __uint_as_float(pv[1][3]);
#pragma unroll
                            for (int ns = 0; ns < NS; ns++) {
                                float e0[4], e1[4];
                                mma16816(e0, a[0][0], a[0][1], a[0][2], a[0][3], bf[ns][0][0], bf[ns][0][1], zz);
                                mma16816(e1, a[2][0], a[2][1], a[2][2], a[2][3], bf[ns][2][0], bf[ns][2][1], zz);
                                mma16816(e0, a[1][0], a[1][1], a[1][2], a[1][3], bf[ns][1][0], bf[ns][1][1], e0);
                                mma16816(e1, a[3][0], a[3][1], a[3][2], a[3][3], bf[ns][3][0], bf[ns][3][1], e1);
                                const float ta0 = pa0 * cs[ns][0], ta1 = pa1 * cs[ns][1], tb0 = pb0 * cs[ns][0], tb1 = pb1 * cs[ns][1];
                                acc[j][ns][0] = fmaf(ta0, e0[0], fmaf(ma0, cc[ns][0], acc[j][ns][0]));
                                acc[j][ns][1] = fmaf(ta0, e0[1], acc[j][ns][1]);
                                acc[j][ns][2] = fmaf(tb0, e0[2], fmaf(mb0, cc[ns][0], acc[j][ns][2]));
                                acc[j][ns][3] = fmaf(tb0, e0[3], acc[j][ns][3]);
                                acc[j][ns][0] = fmaf(ta1, e1[0], fmaf(ma1, cc[ns][1], acc[j][ns][0]));
                                acc[j][ns][1] = fmaf(ta1, e1[1], acc[j][ns][1]);
                                acc[j][ns][2] = fmaf(tb1, e1[2], fmaf(mb1, cc[ns][1], acc[j][ns][2]));
                                acc[j][ns][3] = fmaf(tb1, e1[3], acc[j][ns][3]);
                            }
                        });
                    });
                } else if constexpr (T == GT_Q6_K) {
                    // odd super-blocks start 2 bytes past a 4-byte boundary: their words are read from the boundary below
                    // and shifted by a byte permute (ODD).  The parity is the warp's, so the branch sits outside the loops.
                    auto body = [&](auto ODDC) {
                        constexpr bool ODD = decltype(ODDC)::value;
                        const float zz[4] = {0.f, 0.f, 0.f, 0.f};
                        // row g of the stage, the warp's first super-block
                        const uint32_t u6 = (PAIR ? stage + ((g & 1u) * (R / 2) + (g >> 1)) * PITCH + (lead ^ (8u * (g & 1u)))
                                                  : stage + g * PITCH + lead) + 208 * sp;
                        const uint32_t pA = u6 + q6A, pH = u6 + q6H, pP = ptab + g * 16;
                        static_for<0, KB>([&](auto IC) {
                            constexpr uint32_t i = decltype(IC)::value;
                            uint32_t bf[NS][4][2];
                            float cc[NS][4], cs[NS][4];
                            static_for<0, NS>([&](auto SC) {
                                constexpr uint32_t ns = decltype(SC)::value;
                                static_for<0, 4>([&](auto QC) {
                                    constexpr uint32_t q = decltype(QC)::value;
                                    lds64i<(((i * MP + 4 * ns) * 4 + q) * 64)>(xlane, bf[ns][q][0], bf[ns][q][1]);
                                    if constexpr (MP > 1) {   // (one activation row: pre-scale and bias are in the scale table)
                                        uint32_t u0, u1;
                                        lds64i<(((i * MP + 4 * ns) * 4 + q) * 8)>(clane, u0, u1);
                                        cc[ns][q] = __uint_as_float(u0);
                                        cs[ns][q] = __uint_as_float(u1);
                                    }
                                });
                            });
                            static_for<0, TPW>([&](auto JC) {
                                constexpr uint32_t j = decltype(JC)::value;
                                uint32_t qv[2][4];   // [row g / g + 8][q1..q4]: four 6-bit codes each, one per byte
                                uint32_t pv[2][4];
                                static_for<0, 2>([&](auto HC) {
                                    constexpr uint32_t h = decltype(HC)::value;
                                    constexpr uint32_t off = (PAIR ? 8 * j + 4 * h : 16 * j + 8 * h) * PITCH + 420 * i;   // rows g, g + 8 of tile j
                                    uint32_t A, B, H;
                                    if constexpr (!ODD) {
                                        A = lds32i<off>(pA);
                                        B = lds32i<off + 32>(pA);
                                        H = lds32i<off>(pH);
                                    } else {
                                        A = __byte_perm(lds32i<off>(pA), lds32i<off + 4>(pA), 0x5432);
                                        B = __byte_perm(lds32i<off + 32>(pA), lds32i<off + 36>(pA), 0x5432);
                                        H = __byte_perm(lds32i<off>(pH), lds32i<off + 4>(pH), 0x5432);
                                    }
                                    qv[h][0] = (A & 0x0F0F0F0Fu) | ((H & 0x03030303u) << 4);
                                    qv[h][1] = (B & 0x0F0F0F0Fu) | ((H & 0x0C0C0C0Cu) << 2);
                                    qv[h][2] = ((A >> 4) & 0x0F0F0F0Fu) | (H & 0x30303030u);
                                    qv[h][3] = ((B >> 4) & 0x0F0F0F0Fu) | ((H & 0xC0C0C0C0u) >> 2);
                                    lds128i<((i * R) + 16 * j + 8 * h) * 16>(pP, pv[h][0], pv[h][1], pv[h][2], pv[h][3]);
                                });
#pragma unroll
                                for (int q = 0; q < 4; q++) {
                                    const uint32_t a0 = __byte_perm(qv[0][q], 0u, 0x4240), a2 = __byte_perm(qv[0][q], 0u, 0x4341);
                                    const uint32_t a1 = __byte_perm(qv[1][q], 0u, 0x4240), a3 = __byte_perm(qv[1][q], 0u, 0x4341);
                                    const float pa = __uint_as_float(pv[0][q]), pb = __uint_as_float(pv[1][q]);
#pragma unroll
                                    for (int ns = 0; ns < NS; ns++) {
                                        float d[4];
                                        mma16816(d, a0, a1, a2, a3, bf[ns][q][0], bf[ns][q][1], zz);
                                        if constexpr (MP == 1) {
                                            acc[j][ns][0] = fmaf(pa, d[0], acc[j][ns][0]);
                                            acc[j][ns][1] = fmaf(pa, d[1], acc[j][ns][1]);
                                            acc[j][ns][2] = fmaf(pb, d[2], acc[j][ns][2]);
                                            acc[j][ns][3] = fmaf(pb, d[3], acc[j][ns][3]);
                                            continue;
                                        }
                                        const float ta = pa * cs[ns][q], tb = pb * cs[ns][q];
                                        acc[j][ns][0] = fmaf(ta, d[0], fmaf(pa, cc[ns][q], acc[j][ns][0]));
                                        acc[j][ns][1] = fmaf(ta, d[1], acc[j][ns][1]);
                                        acc[j][ns][2] = fmaf(tb, d[2], fmaf(pb, cc[ns][q], acc[j][ns][2]));
                                        acc[j][ns][3] = fmaf(tb, d[3], acc[j][ns][3]);
                                    }
                                }
                            });
                        });
                    };
                    if (sp) body(std::true_type{});
                    else body(std::false_type{});
                } else {
                    // the warp's blocks KB w .. KB w + KB - 1 of the stage, two at a time (KB is even: the first of a pair
                    // starts on a 4-byte boundary); rows g and g + 8 of tile j sit (16 j + 8 h) PITCH bytes further on
                    const uint32_t rb = stage + (HV == 2 ? (w >> 2) * ((uint32_t)R * PITCH) : 0u) + g * PITCH + BB * KB * (HV == 2 ? (w & 3u) : w);
                    const uint32_t base = rb + 4 * t, base2 = rb + (t ? 4 * t : (T == GT_Q8_0 ? 32u : 16u));
                    const uint32_t sel = t ? 0x3210u : 0x5432u;
                    static_for<0, KB / 2>([&](auto IC) {
                        constexpr uint32_t i = 2 * decltype(IC)::value;
                        uint32_t bf0[NS][2][2], bf1[NS][2][2];
                        float cc[NS][2], cs[NS][2];
                        static_for<0, NS>([&](auto SC) {
                            constexpr uint32_t ns = decltype(SC)::value;
                            static_for<0, 2>([&](auto HC) {
                                constexpr uint32_t h = decltype(HC)::value;
                                lds64i<((i * MP + 4 * ns) * 2 + h) * 64>(xlane, bf0[ns][h][0], bf0[ns][h][1]);
                                lds64i<(((i + 1) * MP + 4 * ns) * 2 + h) * 64>(xlane, bf1[ns][h][0], bf1[ns][h][1]);
                            });
                            uint32_t u0, u1, v0, v1;
                            lds64i<(i * MP + 4 * ns) * 8>(clane, u0, u1);
                            lds64i<((i + 1) * MP + 4 * ns) * 8>(clane, v0, v1);
                            cc[ns][0] = __uint_as_float(u0);
                            cs[ns][0] = __uint_as_float(u1);
                            cc[ns][1] = __uint_as_float(v0);
                            cs[ns][1] = __uint_as_float(v1);
                        });
                        mw_pair_tiles<T, TPW, MP, NS, PITCH, BB * i>(base, base2, rb, sel, bf0, bf1, cc, cs, acc);
                    });
                }
                __syncwarp();
                if (lane == 0) {   // the last of the eight warps to let go of the slot starts the copy of the stage that gets it next
                    uint32_t old;
                    asm volatile("atom.acq_rel.cta.shared.add.u32 %0, [%1], 1;" : "=r"(old) : "r"(smem_u32(&rel[slot])) : "memory");
                    if ((old & (uint32_t)(kMwWarps - 1)) == (uint32_t)(kMwWarps - 1)) issue(qn + c.nslots, slot);
                }
                qn++;
                if (++slot == c.nslots) { slot = 0; ph ^= 1u; }
            }
            if (!ok) break;

            // ---- end of the item: add the eight warps' partial sums in a fixed order and write the rows out ----
            if (!first_item) {   // the previous item's sums have all been read
                if (!mbar_wait(&fin[1], fin_ph ^ 1u, &abort_flag, bt.status, ST_WAIT_EMPTY_TIMEOUT, 0u)) {
                    ok = false;
                    break;
                }
            }
#pragma unroll
            for (int j = 0; j < TPW; j++) {
#pragma unroll
                for (int ns = 0; ns < NS; ns++) {
                    const uint32_t col = t + 4 * ns;
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const uint32_t row = 16 * j + g + 8 * i;
                        if (col < (uint32_t)MP)
                            sts32(red + ((w * MP + col) * R + row) * 4, __float_as_uint((acc[j][ns][2 * i] + acc[j][ns][2 * i + 1]) * 16777216.0f));
                        acc[j][ns][2 * i] = acc[j][ns][2 * i + 1] = 0.f;
                    }
                }
            }
            __syncwarp();
            if constexpr (T == GT_Q6_K && MP == 1) {
                // ... plus the bias term of the rows this lane kept the books for (this warp's share of K)
#pragma unroll
                for (int rr = 0; rr < (R + 31) / 32; rr++) {
                    const uint32_t r = lane + 32 * rr;
                    if (r < (uint32_t)R) {
                        const uint32_t addr = red + (w * R + r) * 4;
                        sts32(addr, __float_as_uint(__uint_as_float(lds32(addr)) + corr[rr] * 16777216.0f));
                    }
                    corr[rr] = 0.f;
                }
                __syncwarp();
            }
            if (lane == 0) mbar_arrive(&fin[0]);
            if (!mbar_wait(&fin[0], fin_ph, &abort_flag, bt.status, ST_WAIT_EMPTY_TIMEOUT, 0u)) {
                ok = false;
                break;
            }
            {
                const MwProb &P = bt.p[p];
                const uint32_t ld = P.y_ld ? P.y_ld : P.n;
                for (uint32_t idx = tid; idx < (uint32_t)R * pm; idx += kMwWarps * 32) {
                    const uint32_t col = idx / R, row = idx % R;
                    float sum = 0.f;
#pragma unroll
                    for (int ww = 0; ww < kMwWarps; ww++) sum += __uint_as_float(lds32(red + ((ww * MP + col) * R + row) * 4));
                    const uint32_t grow = item * R + row;
                    if (grow < P.n) {
                        const size_t off = (size_t)col * ld + P.y_col0 + grow;
                        P.y[off] = sum;
                        for (uint32_t pr = 0; pr < P.n_peer; pr++) P.y_peer[pr][off] = sum;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&fin[1]);
            fin_ph ^= 1u;
            first_item = false;
        }
        }
    }
    if (abort_flag) {  // let copies in flight land before the CTA's shared memory is released
        for (int i = 0; i < 200; i++) __nanosleep(5000);
    }
    if (bt.dep_mask) {
        // the last CTA to leave clears the barrier words for the next launch that uses them (launches that share
        // them are ordered by their stream)
        __syncthreads();
        if (tid == 0) {
            const uint32_t old = atomicAdd(bt.bar + 31, 1u);
            if (old == gridDim.x - 1) {
                for (uint32_t i = 0; i < 32; i++) bt.bar[i] = 0;
                __threadfence();
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static uint32_t mw_uk(int t) { return t == GT_Q6_K ? 512u : 256u; }   // (Q4_K: a last stage of one super-block is fine)

// Q6_K rows of 16 j + 8 bytes with an even row count: pairs of rows start on 16-byte boundaries (see PAIR above)
bool qmv_mma_pair_mode(int ggml_type, const QmvArgs &a) {
    if (ggml_type != GT_Q6_K || a.k % 256 != 0) return false;
    const uint64_t row_bytes = (uint64_t)(a.k / 256) * 210;
    return row_bytes % 16 == 8 && a.n % 2 == 0;
}

bool qmv_mma_supported(int ggml_type, const QmvArgs &a) {
    if (ggml_type != GT_Q4_0 && ggml_type != GT_Q8_0 && ggml_type != GT_Q6_K && ggml_type != GT_Q4_K) return false;
    if (a.ids || a.nprob != 1 || a.m < 1 || a.m > 8) return false;
    if (a.k == 0 || a.n == 0 || a.k % mw_uk(ggml_type) != 0) return false;
    const uint64_t row_bytes = (uint64_t)(a.k / ggml_qk(ggml_type)) * ggml_block_bytes(ggml_type);
    if ((row_bytes % 16 != 0 && !qmv_mma_pair_mode(ggml_type, a)) || row_bytes >= (1ull << 31)) return false;
    if (((uintptr_t)a.w & 15u) || ((uintptr_t)a.x & 15u)) return false;
    if ((uint64_t)a.m * a.n >= (1ull << 32)) return false;
    return encode_tiled_fn() != nullptr;
}

// The expert-routed form: one problem per (token, slot) row (m = 1, `ids` and `id_index` set).  The stacked weights are
// addressed through a 3-D map [expert][row][bytes], so rows and experts must start on 16-byte boundaries.
bool qmv_mma_supported_routed(int ggml_type, const QmvArgs &a) {
    if (ggml_type != GT_Q4_0 && ggml_type != GT_Q8_0 && ggml_type != GT_Q6_K && ggml_type != GT_Q4_K && ggml_type != GT_Q5_K) return false;
    if (!a.ids || a.m != 1 || a.k == 0 || a.n == 0 || a.n_experts == 0 || a.k % mw_uk(ggml_type) != 0) return false;
    const uint64_t row_bytes = (uint64_t)(a.k / ggml_qk(ggml_type)) * ggml_block_bytes(ggml_type);
    if (row_bytes % 16 != 0 || row_bytes >= (1ull << 31) || a.expert_stride % 16 != 0 || a.expert_stride < row_bytes * a.n) return false;
    if (((uintptr_t)a.w & 15u) || ((uintptr_t)a.x & 15u) || ((uintptr_t)a.x2 & 15u)) return false;
    return encode_tiled_fn() != nullptr;
}

static inline size_t mw_align(size_t v, size_t al) { return (v + al - 1) / al * al; }

template <int T, int TPW, int KB, int MP, bool PAIR>
static cudaError_t launch_mw(const QmvArgs *ops, int nops, int sm_count, int ctas_per_sm, cudaStream_t st) {
    using TR = MwTraits<T>;
    constexpr uint32_t R = 16 * TPW, PITCH = mw_pitch(T, KB), STAGE = mw_halves(T, KB) * R * PITCH;
    constexpr uint32_t PIECES = KB * MP * TR::NM * 4, NB = PIECES >= 32 ? 1 : 32 / PIECES;
    constexpr uint32_t XST = (NB * PIECES * 16 + NB * KB * MP * TR::NG * 8 + 15u) & ~15u;   // as in the kernel
    MwCfg c{};
#ifdef MLXN_EXPERIMENTS
    if (const char *e = getenv("MLXN_MW_DEBUG")) c.debug = (uint32_t)atoi(e);
#endif
    const size_t xst_bytes = mw_align((size_t)kMwWarps * XST, 128);
    const size_t ptab_bytes = (T == GT_Q6_K || T == GT_Q4_K || T == GT_Q5_K) ? (size_t)kMwWarps * R * 16 * KB : 0;
    const size_t red_bytes = (size_t)kMwWarps * MP * R * 4;
    const size_t tail = xst_bytes + ptab_bytes + red_bytes;
    // two CTAs per SM: 228 KB, less 1 KB per CTA for the system and the kernel's few hundred bytes of static storage
    const size_t budget = 115200;
    uint32_t nslots = (uint32_t)((budget - tail - 128) / STAGE);
    if (nslots > (uint32_t)kMwMaxSlots) nslots = kMwMaxSlots;
    if (nslots < 2) return cudaErrorInvalidConfiguration;
    c.nslots = nslots;
    c.xst_off = nslots * STAGE;
    c.ptab_off = c.xst_off + (uint32_t)xst_bytes;
    c.red_off = c.ptab_off + (uint32_t)ptab_bytes;
    const size_t smem = (size_t)c.red_off + red_bytes + 128;

    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return cudaErrorNotSupported;
    if (nops < 1 || nops > kMwMaxProbs) return cudaErrorInvalidValue;
    static thread_local MwBatch bt;      // too large for the stack of a deep call chain; one launch at a time per thread
    alignas(64) static thread_local MwMaps maps;
    bt.nprob = (uint32_t)nops;
    bt.early_weights = 1;
    bt.routed = 0;
    bt.status = ops[0].status;
    uint64_t total_stages = 0;
    uint32_t items = 0;
    for (int i = 0; i < nops; i++) {
        const QmvArgs &a = ops[i];
        MwProb &P = bt.p[i];
        P.x = a.x;
        P.x2 = a.x2;
        P.ids = a.ids;
        P.id_idx = a.id_index;
        if (a.ids) bt.routed = 1;
        P.y = a.y;
        P.n = a.n;
        P.k = a.k;
        P.m = a.m;
        P.spi = (a.k + TR::UK * KB - 1) / (TR::UK * KB);   // the last stage may reach past K: the copy fills zeros
        P.item0 = items;
        P.y_ld = a.y_ld;
        P.y_col0 = a.y_col0;
        P.n_peer = a.n_peer;
        for (uint32_t q = 0; q < (uint32_t)kMaxPeers; q++) P.y_peer[q] = q < a.n_peer ? a.y_peer[q] : nullptr;
        const uint32_t its = (a.n + R - 1) / R;
        items += its;
        total_stages += (uint64_t)its * P.spi;
        if (!a.early_weights || a.ids) bt.early_weights = 0;
        const uint32_t row_bytes = (a.k / BlockTraits<T>::QK) * BlockTraits<T>::BYTES;
        // the weight matrix as [n rows][row_bytes / 8] 8-byte elements; box = R rows x PITCH bytes
        // (pair mode: [n / 2 row pairs][2 row_bytes / 8], box = R / 2 pairs x PITCH bytes)
        const cuuint64_t gdim[2] = {PAIR ? row_bytes / 4 : row_bytes / 8, PAIR ? a.n / 2 : a.n};
        const cuuint64_t gstride[1] = {PAIR ? 2ull * row_bytes : row_bytes};
        const cuuint32_t box[2] = {(cuuint32_t)(PITCH / 8), (cuuint32_t)(PAIR ? R / 2 : R)};
        const cuuint32_t estr[2] = {1, 1};
        if (a.ids) {
            // the stacked experts as [n_experts][n rows][row_bytes / 8]; box = 1 expert x R rows x PITCH bytes
            if (PAIR) return cudaErrorInvalidValue;
            const cuuint64_t gdim3[3] = {row_bytes / 8, a.n, a.n_experts};
            const cuuint64_t gstride3[2] = {row_bytes, a.expert_stride};
            const cuuint32_t box3[3] = {(cuuint32_t)(PITCH / 8), (cuuint32_t)R, 1};
            const cuuint32_t estr3[3] = {1, 1, 1};
            if (enc(&maps.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<uint8_t *>(a.w), gdim3, gstride3, box3, estr3,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return cudaErrorInvalidValue;
            continue;
        }
        if (enc(&maps.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t *>(a.w), gdim, gstride, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    bt.nitems = items;
    bt.dep_mask = 0;
    bt.bar = ops[0].grid_bar;
    uint32_t max_items = 0;
    for (int i = 0; i < nops; i++) {
        if (i > 0 && ops[i].after_earlier) bt.dep_mask |= 1u << i;
        const uint32_t its = (ops[i].n + R - 1) / R;
        if (its > max_items) max_items = its;
    }
    if (bt.dep_mask && !bt.bar) return cudaErrorInvalidValue;
    for (int i = nops; i < kMwMaxProbs; i++) {
        bt.p[i] = MwProb{};
        bt.p[i].item0 = items;
        maps.m[i] = maps.m[0];
    }
    uint32_t grid = (uint32_t)(sm_count * ctas_per_sm);
    if (grid > (uint32_t)kMwMaxGrid) grid = kMwMaxGrid;
    if (grid > (bt.dep_mask ? max_items : items)) grid = bt.dep_mask ? max_items : items;
    // contiguous chunks of items holding (nearly) the same number of stages each: CTA c starts at the first item whose
    // stages begin at or after c / grid of all the launch's stages
    {
        uint32_t pi = 0;
        uint64_t before = 0;   // stages of the problems ahead of pi
        for (uint32_t cta = 0; cta <= grid; cta++) {
            const uint64_t target = total_stages * cta / grid;
            while (pi + 1 < (uint32_t)nops) {
                const uint64_t its = bt.p[pi + 1].item0 - bt.p[pi].item0;
                if (before + its * bt.p[pi].spi > target) break;
                before += its * bt.p[pi].spi;
                pi++;
            }
            const uint64_t its_p = (pi + 1 < (uint32_t)nops ? bt.p[pi + 1].item0 : items) - bt.p[pi].item0;
            uint64_t in = (target - before + bt.p[pi].spi - 1) / bt.p[pi].spi;
            if (in > its_p) in = its_p;
            bt.cta_begin[cta] = bt.p[pi].item0 + (uint32_t)in;
        }
        bt.cta_begin[0] = 0;
        bt.cta_begin[grid] = items;
        for (uint32_t cta = grid + 1; cta <= (uint32_t)kMwMaxGrid; cta++) bt.cta_begin[cta] = items;
    }
    static size_t attr_smem[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (smem > attr_smem[dev]) {
        cudaError_t e = cudaFuncSetAttribute(qmv_mma_kernel<T, TPW, KB, MP, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_smem[dev] = smem;
    }
    if (bt.dep_mask)   // its CTAs wait on one another: all of them resident at once, or the launch is refused
        return launch_cooperative(qmv_mma_kernel<T, TPW, KB, MP, PAIR>, dim3(grid), dim3(kMwThreads), smem, st, bt, c, maps);
    return launch_overlapped(qmv_mma_kernel<T, TPW, KB, MP, PAIR>, dim3(grid), dim3(kMwThreads), smem, st, bt, c, maps);
}

// (TPW, KB): a warp works on TPW x KB tile-units per stage.  Few weight rows -> narrow row groups and long K stages.
// Q4_0 / Q8_0 blocks are worked on in pairs (KB even).  The activation split costs MP x KB per stage and warp whatever
// TPW is, so many activation rows want a small KB.
template <int T, int MP, bool PAIR>
static cudaError_t launch_mw_m(const QmvArgs *ops, int nops, int sm_count, int ctas_per_sm, int tpw, cudaStream_t st) {
    if constexpr (T == GT_Q6_K || T == GT_Q4_K || T == GT_Q5_K) {
        if (tpw >= 4 || MP == 8) return launch_mw<T, 4, 1, MP, PAIR>(ops, nops, sm_count, ctas_per_sm, st);
        if constexpr (MP <= 4) {
            if (tpw >= 2 || MP == 4) return launch_mw<T, 2, 2, MP, PAIR>(ops, nops, sm_count, ctas_per_sm, st);
        }
        if constexpr (MP <= 2) return launch_mw<T, 1, 4, MP, PAIR>(ops, nops, sm_count, ctas_per_sm, st);
    } else {
        if constexpr (MP == 8) return launch_mw<T, 2, 2, MP, PAIR>(ops, nops, sm_count, ctas_per_sm, st);
        if constexpr (MP <= 4) {
            if (tpw >= 4) return launch_mw<T, 4, 2, MP, PAIR>(ops, nops, sm_count, ctas_per_sm, st);
            if (tpw >= 2) return launch_mw<T, 2, 4, MP, PAIR>(ops, nops, sm_count, ctas_per_sm, st);
        }
        if constexpr (MP == 4) return launch_mw<T, 1, 4, MP, PAIR>(ops, nops, sm_count, ctas_per_sm, st);
        if constexpr (MP <= 2) return launch_mw<T, 1, 8, MP, PAIR>(ops, nops, sm_count, ctas_per_sm, st);
    }
    return cudaErrorInvalidConfiguration;
}

template <int T, bool PAIR>
static cudaError_t launch_mw_p(const QmvArgs *ops, int nops, uint32_t mmax, int sm_count, int ctas_per_sm, int tpw, cudaStream_t st) {
    if (mmax <= 1) return launch_mw_m<T, 1, PAIR>(ops, nops, sm_count, ctas_per_sm, tpw, st);
    if (mmax <= 2) return launch_mw_m<T, 2, PAIR>(ops, nops, sm_count, ctas_per_sm, tpw, st);
    if (mmax <= 4) return launch_mw_m<T, 4, PAIR>(ops, nops, sm_count, ctas_per_sm, tpw, st);
    return launch_mw_m<T, 8, PAIR>(ops, nops, sm_count, ctas_per_sm, tpw, st);
}

template <int T>
static cudaError_t launch_mw_t(const QmvArgs *ops, int nops, uint32_t mmax, int sm_count, int ctas_per_sm, int tpw, cudaStream_t st) {
    if constexpr (T == GT_Q6_K) {
        // all or none of a launch's mat-vecs are in pair mode (the caller batches accordingly)
        const bool pair = qmv_mma_pair_mode(T, ops[0]);
        for (int i = 1; i < nops; i++)
            if (qmv_mma_pair_mode(T, ops[i]) != pair) return cudaErrorInvalidValue;
        if (pair) return launch_mw_p<T, true>(ops, nops, mmax, sm_count, ctas_per_sm, tpw, st);
    }
    return launch_mw_p<T, false>(ops, nops, mmax, sm_count, ctas_per_sm, tpw, st);
}

// Launches `nops` (1..8) mat-vecs of one block type as ONE kernel.  The caller guarantees that no operation reads or
// writes what another one writes.  `ctas_per_sm` (1 or 2) and `tpw` (0: chosen from the row count; 1, 2, 4) are tuning
// knobs of the caller.
cudaError_t launch_qmv_mma(int ggml_type, const QmvArgs *ops, int nops, int sm_count, int ctas_per_sm, int tpw, cudaStream_t st) {
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    if (ctas_per_sm > 2) ctas_per_sm = 2;
    uint32_t mmax = 1;
    for (int i = 0; i < nops; i++)
        if (ops[i].m > mmax) mmax = ops[i].m;
    bool routed = false;
    for (int i = 0; i < nops; i++) routed = routed || ops[i].ids != nullptr;
    if (tpw <= 0 && routed) {
        // Expert-routed rows: one geometry whatever else is in the launch (64-row groups: the smallest K stage of every
        // row class), because the geometry fixes how K is shared among the warps and with it the rounding of a row's sum.
        // A (token, slot) pair's result then does not depend on how many pairs travel with it, which is what makes an
        // expert-parallel layer bit-identical to the single-GPU one.
        tpw = 4;
    }
    if (tpw <= 0) {
        // measured: the largest row group (the activation split is paid once per group) that still gives at least every
        // other CTA slot an item; 16-row groups when even 32-row groups do not
        tpw = 1;
        for (int cand = 4; cand >= 2; cand >>= 1) {
            uint64_t items = 0;
            for (int i = 0; i < nops; i++) items += (ops[i].n + 16u * cand - 1) / (16u * cand);
            if (items >= (uint64_t)sm_count) {
                tpw = cand;
                break;
            }
        }
    }
    switch (ggml_type) {
    case GT_Q4_0: return launch_mw_t<GT_Q4_0>(ops, nops, mmax, sm_count, ctas_per_sm, tpw, st);
    case GT_Q8_0: return launch_mw_t<GT_Q8_0>(ops, nops, mmax, sm_count, ctas_per_sm, tpw, st);
    case GT_Q6_K: return launch_mw_t<GT_Q6_K>(ops, nops, mmax, sm_count, ctas_per_sm, tpw, st);
    case GT_Q4_K: return launch_mw_t<GT_Q4_K>(ops, nops, mmax, sm_count, ctas_per_sm, tpw, st);
    case GT_Q5_K: return launch_mw_t<GT_Q5_K>(ops, nops, mmax, sm_count, ctas_per_sm, tpw, st);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace mlxn
