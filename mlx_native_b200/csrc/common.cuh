// Shared declarations for the sm_100a kernels of the GGML block-quantized matmul path.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include <cstdlib>

namespace mlxn {

// Experiment switches — environment variables that re-configure a kernel or switch parts of it off, for ablations —
// exist only in builds made with -DMLXN_EXPERIMENTS.  The shipped library does not look at them, and the kernels'
// debug masks are the constant 0 there, so their tests compile away.
#ifdef MLXN_EXPERIMENTS
inline const char *exp_env(const char *name) { return getenv(name); }
#define MLXN_DBG(c) ((c).debug)
#else
inline const char *exp_env(const char *) { return nullptr; }
#define MLXN_DBG(c) 0u
#endif

// GGML type codes (same numbering as mlxn_ggml_type in include/mlxn_b200.h).
enum : int { GT_F32 = 0, GT_F16 = 1, GT_Q4_0 = 2, GT_Q8_0 = 3, GT_Q4_K = 4, GT_Q5_K = 5, GT_Q6_K = 6, GT_I16 = 7 };

// Block geometry (upstream src/shaders/quantized_matmul_ggml.metal:49-67).
template <int T> struct BlockTraits;
template <> struct BlockTraits<GT_Q4_0> { static constexpr int QK = 32, BYTES = 18; };
template <> struct BlockTraits<GT_Q8_0> { static constexpr int QK = 32, BYTES = 34; };
template <> struct BlockTraits<GT_Q6_K> { static constexpr int QK = 256, BYTES = 210; };
template <> struct BlockTraits<GT_Q4_K> { static constexpr int QK = 256, BYTES = 144; };
template <> struct BlockTraits<GT_Q5_K> { static constexpr int QK = 256, BYTES = 176; };

// Q4_K (src/gguf/mod.rs:440-452): the 6-bit (scale, min) pair of sub-block j from the block's 12 packed bytes.
__host__ __device__ inline void q4k_scale_min(uint32_t j, const uint8_t *scales, uint32_t &sc, uint32_t &mn) {
    if (j < 4) {
        sc = scales[j] & 63u;
        mn = scales[j + 4] & 63u;
    } else {
        sc = (scales[j + 4] & 0x0Fu) | ((uint32_t)(scales[j - 4] >> 6) << 4);
        mn = (uint32_t)(scales[j + 4] >> 4) | ((uint32_t)(scales[j] >> 6) << 4);
    }
}

__host__ __device__ inline uint32_t ggml_qk(int t) {
    switch (t) {
    case GT_F32: case GT_F16: case GT_I16: return 1;
    case GT_Q4_0: case GT_Q8_0: return 32;
    default: return 256;
    }
}
__host__ __device__ inline uint32_t ggml_block_bytes(int t) {
    switch (t) {
    case GT_F32: return 4;
    case GT_F16: case GT_I16: return 2;
    case GT_Q4_0: return 18;
    case GT_Q8_0: return 34;
    case GT_Q4_K: return 144;
    case GT_Q5_K: return 176;
    default: return 210;
    }
}

// Device status word written by kernels whose bounded waits gave up.  0 = ok.
enum : uint32_t { ST_OK = 0, ST_WAIT_FULL_TIMEOUT = 1, ST_WAIT_EMPTY_TIMEOUT = 2, ST_WAIT_MMA_TIMEOUT = 3,
                  ST_WAIT_TMEM_TIMEOUT = 4, ST_BAD_ARGUMENT = 5, ST_WAIT_PEER_TIMEOUT = 6, ST_WAIT_GRID_TIMEOUT = 7 };

// Arguments shared by the mat-vec kernels (dense and expert-routed).
struct QmvArgs {
    const uint8_t *w;       // weight blocks; expert e starts at w + e*expert_stride
    const float *x;         // activations [n_x_rows, k]
    float *y;               // outputs [n_out_rows, n]
    const uint32_t *ids;    // expert id per output row group (nullptr for the dense form)
    uint32_t n, k;          // weight rows, reduction length
    uint32_t m;             // dense: activation rows sharing the weights; routed: 1
    uint32_t nprob;         // dense: 1; routed: n_tokens*top_k independent mat-vecs
    uint32_t top_k;         // routed: activation row of problem p is p / top_k
    uint32_t n_experts;
    uint64_t expert_stride; // bytes
    uint32_t *status;       // device status word
    uint32_t early_weights; // 1: no kernel of this process wrote the weights, so they may be fetched before the
                            // kernels ahead in the stream have finished (see launch_overlapped)
    // Row-sharded form (dense only): this rank holds n of the n_total weight rows; output row t lives at
    // y[t * y_ld + y_col0 ..] and every result is also stored to the same place in the other ranks' output
    // buffers (peer memory), so that each rank ends up with the whole [m, n_total] result without a collective.
    uint32_t y_ld;          // elements between output rows (0: n)
    uint32_t y_col0;        // first output column of this rank
    uint32_t n_peer;        // other ranks' buffers in y_peer
    float *y_peer[7];
    // Batched launches of the register-level kernel only: this mat-vec reads or overwrites what a mat-vec earlier in
    // the same launch writes, so it starts after all of them have finished (a barrier across the grid).
    uint32_t after_earlier;
    uint32_t *grid_bar;     // 32 zeroed words of device memory for those barriers (one launch at a time uses them)
    // Register-level kernel, expert-routed form: one QmvArgs per (token, slot) row with m = 1, `ids` set and the
    // row's expert read from ids[id_index]; `x` / `y` already point at the row's activations and results.
    uint32_t id_index;
    // ... and its fused SwiGLU form: the activations are silu(x) * x2 (src/shaders/quantized_matmul_id_ggml.metal:231-319)
    const float *x2;
};
constexpr int kMaxPeers = 7;
__host__ __device__ inline uint32_t qmv_ld(const QmvArgs &a) { return a.y_ld ? a.y_ld : a.n; }

// Arguments of the mat-mat kernels (dense and grouped-by-expert).
struct QmmArgs {
    const uint8_t *w;
    const float *x;          // [m, k] (dense) or [n_tokens, k] (routed)
    float *y;                // [m, n] or [n_tokens*top_k, n]
    uint32_t m, n, k;
    // routed form (hids == nullptr for dense)
    const uint32_t *htpe;    // [n_experts] rows routed to each expert
    const int32_t *hids;     // [n_experts, hids_stride] entries token*top_k+slot
    uint32_t hids_stride;
    uint32_t top_k;
    uint32_t n_experts;
    uint32_t total_rows;     // n_tokens*top_k
    uint64_t expert_stride;
    const uint32_t *tiles;   // optional compact tile list built by the bucketing kernel
    uint32_t *status;
    // Row-sharded dense form (tensor-core kernel only): this rank holds n of the y_ld weight rows; output row o lives
    // at y[o * y_ld + y_col0 ..] and every finished tile is also stored to the same place in the other ranks' result
    // buffers (peer memory), as for the mat-vec (see QmvArgs).  y_ld == 0: a plain [m, n] result.
    uint32_t y_ld, y_col0, n_peer;
    float *y_peer[7];
    // bf16 "perm021" activations (dense tensor-core form only; src/ops/quantized_matmul_ggml.rs:573-742): x[row][kk] is
    // read from a bf16 array laid out [k / head_dim heads][m rows][head_dim] — the attention output before its permute —
    // and cast bf16 -> f32 -> f16 while it is packed.  nullptr: the f32 array `x`.
    const uint16_t *x_bf16;
    uint32_t head_dim;
    // Fused MoE layer (routed tensor-core form): what an earlier call of the same layer has left in the scratch area and
    // this call takes over instead of building it again (bit 0: the tile list, bit 1: the packed activations), and the
    // second operand of a SwiGLU formed while packing: activations = silu(x) * x2 (src/shaders/silu_mul.metal:17-30).
    uint32_t reuse;
    const float *x2;
};
__host__ __device__ inline uint32_t qmm_ld(const QmmArgs &a) { return a.y_ld ? a.y_ld : a.n; }

// ---- overlapped launches -------------------------------------------------------------------------
// A kernel launched with launch_overlapped may be scheduled while the kernel ahead of it in the stream is still
// running: its blocks set themselves up (barriers, tensor memory, the first weight copies) and then call
// grid_dependency_wait(), which returns once every kernel ahead has completed and its writes are visible.
// Nothing a predecessor may have written is read before that call.  allow_dependents() lets the *next*
// overlapped launch start in the same way.  Launched after anything else (copies, ordinary kernels) it
// behaves like an ordinary launch.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                     Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// The same for a kernel whose blocks wait on one another: all blocks of the grid are resident at the same time
// (the launch fails with cudaErrorCooperativeLaunchTooLarge if they cannot be).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cooperative(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                      Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// ---- small device helpers ---------------------------------------------------------------------
__device__ __forceinline__ float half_bits_to_float(uint32_t h16) {
    return __half2float(__ushort_as_half((unsigned short)h16));
}

// 2-byte-aligned little-endian loads (GGML blocks are only 2-byte aligned).
__device__ __forceinline__ uint32_t ld_u16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }
__device__ __forceinline__ uint32_t ld_u32_2(const uint8_t *p) {
    const uint16_t *q = reinterpret_cast<const uint16_t *>(p);
    return (uint32_t)q[0] | ((uint32_t)q[1] << 16);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Exact dequantisation of one element group, shared by the simple mat-vec and the mat-mat staging.
// Q4_0: value = d*(nibble-8); Q8_0: d*q; Q6_K: (d*scale)*q  (all exact in f32).

}  // namespace mlxn
