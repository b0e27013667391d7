// Routing and glue kernels around the expert-routed matmul.
//
//   moe_map0           replaces kernel_mul_mm_id_map0_ne20_{1,8} (src/shaders/quantized_matmul_id_mm.metal:242-301):
//                      per-expert count `htpe[e]` and list `hids[e, :]` of token*top_k+slot entries in
//                      ascending token order (stable), for any top_k.
//   moe_softmax_topk   replaces moe_softmax_topk_f32 (src/shaders/moe_softmax_topk.metal:27-148).
//   silu_mul           replaces silu_mul_f32 (src/shaders/silu_mul.metal:17-30).
//   moe_weighted_reduce replaces moe_weighted_reduce_f32 (src/shaders/moe_weighted_reduce.metal:33-66).
#include "common.cuh"

namespace mlxn {

constexpr uint32_t kNotLocal = 0xFFFFFFFFu;   // id of a (token, slot) pair whose expert lives on another rank

// One CTA of eight warps per expert.  The CTA stages the id table through shared memory a chunk of tokens at a time
// (one coalesced pass, transposed to [slot][token] so that the scan reads without bank conflicts); warp w takes the
// w-th eighth of the chunk's tokens.  Every lane evaluates the upstream selector for its token (sum of (slot+1) over
// slots whose id, truncated to 16 bits, equals the expert); pass 1 counts each warp's hits, a prefix over the eight
// counts gives each warp its first position, pass 2 writes the entries (ballot + popcount inside the warp), so the
// list order is the scan order.  grid n_experts, 256 threads.
constexpr uint32_t kMap0Entries = 4096;   // id entries staged per chunk (8 KB + padding)
// An id >= n_experts belongs to no bucket (it is staged as 0xFFFF, which is no expert because n_experts <= 65535).  So
// that the grouped route agrees with the mat-vec route, which writes a zero row for such a pair, CTA 0 zeroes the
// pair's output row (`y`, n floats; optional) -- except for the id 0xFFFFFFFF, the "expert of another rank" mark of the
// expert-sharded form, whose rows nobody reads and which is far too frequent there to pay for.
__global__ void __launch_bounds__(256) moe_map0_kernel(const uint32_t *ids, uint32_t n_tokens, uint32_t top_k,
                                                       uint32_t n_experts, uint32_t hids_stride, uint32_t *htpe,
                                                       int32_t *hids, float *y, uint32_t n) {
    __shared__ uint16_t stage[kMap0Entries + 2 * 64 + 64];
    __shared__ uint32_t warp_hits[8];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t e = blockIdx.x;
    if (e >= n_experts) return;
    int32_t *row = hids + (size_t)e * hids_stride;
    const uint16_t e16 = (uint16_t)(e & 0xFFFFu);
    uint32_t n_all = 0;    // entries written so far (kept in step by every thread)
    if (top_k > 64) {      // a chunk of 32 tokens would not fit the stage: one warp scans the table in place
        if (warp != 0) return;
        for (uint32_t t0 = 0; t0 < n_tokens; t0 += 32) {
            const uint32_t t = t0 + lane;
            int sel = 0;
            if (t < n_tokens)
                for (uint32_t sl = 0; sl < top_k; sl++)
                    sel += (ids[(size_t)t * top_k + sl] == e) ? (int)(sl + 1) : 0;
            const uint32_t hit = __ballot_sync(0xffffffffu, sel > 0);
            if (sel > 0) {
                const uint32_t pos = n_all + __popc(hit & ((1u << lane) - 1u));
                if (pos < hids_stride) row[pos] = (int32_t)(t * top_k) + sel - 1;
            }
            n_all += __popc(hit);
        }
        if (lane == 0) htpe[e] = n_all;
        return;
    }
    // tokens per chunk: a multiple of 256 when it fits (32 per warp and round), at least 32
    uint32_t chunk = (kMap0Entries / top_k) & ~31u;
    if (chunk < 32) chunk = 32;
    const uint32_t pitch = chunk + 2;   // 16-bit entries: +2 moves each slot's row by one 32-bit bank
    for (uint32_t c0 = 0; c0 < n_tokens; c0 += chunk) {
        const uint32_t ct = min(chunk, n_tokens - c0);
        __syncthreads();   // the previous chunk has been scanned, warp_hits consumed
        for (uint32_t i = threadIdx.x; i < ct * top_k; i += 256) {
            const uint32_t t = i / top_k, sl = i - t * top_k;
            const uint32_t id = ids[(size_t)c0 * top_k + i];
            stage[sl * pitch + t] = id < n_experts ? (uint16_t)id : (uint16_t)0xFFFFu;
            if (e == 0 && y && id >= n_experts && id != 0xFFFFFFFFu) {
                float *yr = y + ((size_t)c0 * top_k + i) * n;
                for (uint32_t j = 0; j < n; j++) yr[j] = 0.f;
            }
        }
        __syncthreads();
        // warp w scans the 32-token groups [g_lo, g_hi) of the chunk
        const uint32_t groups = (ct + 31) / 32;
        const uint32_t g_lo = warp * groups / 8, g_hi = (warp + 1) * groups / 8;
        auto selector = [&](uint32_t t) -> int {
            int sel = 0;
            if (t < ct)
                for (uint32_t sl = 0; sl < top_k; sl++) sel += (stage[sl * pitch + t] == e16) ? (int)(sl + 1) : 0;
            return sel;
        };
        uint32_t mine = 0;
        for (uint32_t g = g_lo; g < g_hi; g++) mine += __popc(__ballot_sync(0xffffffffu, selector(32 * g + lane) > 0));
        if (lane == 0) warp_hits[warp] = mine;
        __syncthreads();
        uint32_t base = n_all, total = 0;
        for (uint32_t w = 0; w < 8; w++) {
            if (w < warp) base += warp_hits[w];
            total += warp_hits[w];
        }
        for (uint32_t g = g_lo; g < g_hi; g++) {
            const uint32_t t = 32 * g + lane;
            const int sel = selector(t);
            const uint32_t hit = __ballot_sync(0xffffffffu, sel > 0);
            if (sel > 0) {
                const uint32_t pos = base + __popc(hit & ((1u << lane) - 1u));
                if (pos < hids_stride) row[pos] = (int32_t)((c0 + t) * top_k) + sel - 1;
            }
            base += __popc(hit);
        }
        n_all += total;
    }
    if (threadIdx.x == 0) htpe[e] = n_all;
}

cudaError_t launch_moe_map0(const uint32_t *ids, uint32_t n_tokens, uint32_t top_k, uint32_t n_experts,
                            uint32_t hids_stride, uint32_t *htpe, int32_t *hids, float *y, uint32_t n, cudaStream_t st) {
    moe_map0_kernel<<<n_experts, 256, 0, st>>>(ids, n_tokens, top_k, n_experts, hids_stride, htpe, hids, y, n);
    return cudaGetLastError();
}

// One CTA of tg = min(n_experts, 128) threads per token, same reduction trees as upstream so that
// the probabilities (and therefore the selected ids) match its arithmetic.
// dynamic shared memory: (2*tg + n_experts + 128) words.
__global__ void moe_softmax_topk_kernel(const float *logits, uint32_t n_tokens, uint32_t n_experts, uint32_t top_k,
                                        uint32_t *out_ids, float *out_w) {
    extern __shared__ float sh[];
    const uint32_t tg = blockDim.x, tid = threadIdx.x, tok = blockIdx.x;
    if (tok >= n_tokens) return;
    float *tg_max = sh, *tg_sum = sh + tg, *prob = sh + 2 * tg;
    const float *lg = logits + (size_t)tok * n_experts;
    float mx = -INFINITY;
    for (uint32_t e = tid; e < n_experts; e += tg) {
        const float v = lg[e];
        if (v > mx) mx = v;
    }
    tg_max[tid] = mx;
    __syncthreads();
    for (uint32_t stride = tg / 2; stride > 0; stride >>= 1) {
        if (tid < stride && tg_max[tid + stride] > tg_max[tid]) tg_max[tid] = tg_max[tid + stride];
        __syncthreads();
    }
    const float gmax = tg_max[0];
    float ls = 0.0f;
    for (uint32_t e = tid; e < n_experts; e += tg) {
        const float ev = expf(lg[e] - gmax);
        prob[e] = ev;
        ls += ev;
    }
    tg_sum[tid] = ls;
    __syncthreads();
    for (uint32_t stride = tg / 2; stride > 0; stride >>= 1) {
        if (tid < stride) tg_sum[tid] += tg_sum[tid + stride];
        __syncthreads();
    }
    const float gsum = tg_sum[0];
    bool any_nan = false;
    for (uint32_t e = tid; e < n_experts; e += tg) {
        const float p = prob[e] / gsum;
        prob[e] = p;
        any_nan |= p != p;
    }
    // Selection.  Upstream keeps a sorted top-k list in one thread (insertion with strict comparisons: of two equal
    // probabilities the lower expert index comes first).  The same list falls out of ranking every expert against
    // all others in parallel: rank(e) = #{j : p_j > p_e, or p_j == p_e and j < e}; rank < top_k is its slot.
    float *top_v = prob + n_experts;            // top_k <= 64 slots each
    uint32_t *top_i = reinterpret_cast<uint32_t *>(prob + n_experts + 64);
    if (__syncthreads_or(any_nan)) {
        // NaN probabilities have no order; keep the one-thread insertion for that (garbage-in) case
        if (tid == 0) {
            for (uint32_t k = 0; k < top_k; k++) {
                top_v[k] = -INFINITY;
                top_i[k] = 0;
            }
            for (uint32_t e = 0; e < n_experts; e++) {
                const float p = prob[e];
                if (p <= top_v[top_k - 1]) continue;
                uint32_t ins = top_k - 1;
                while (ins > 0 && p > top_v[ins - 1]) ins--;
                for (uint32_t k = top_k - 1; k > ins; k--) {
                    top_v[k] = top_v[k - 1];
                    top_i[k] = top_i[k - 1];
                }
                top_v[ins] = p;
                top_i[ins] = e;
            }
        }
    } else {
        for (uint32_t k = n_experts + tid; k < top_k; k += tg) {  // more slots than experts: the rest stay empty
            top_v[k] = -INFINITY;
            top_i[k] = 0;
        }
        for (uint32_t e = tid; e < n_experts; e += tg) {
            const float p = prob[e];
            uint32_t rank = 0;
            for (uint32_t j = 0; j < n_experts; j++) {
                const float q = prob[j];
                rank += (q > p || (q == p && j < e)) ? 1u : 0u;
            }
            if (rank < top_k) {
                top_v[rank] = p;
                top_i[rank] = e;
            }
        }
    }
    __syncthreads();
    float ts = 0.0f;
    for (uint32_t k = 0; k < top_k; k++) ts += top_v[k];   // slot order, as upstream sums them
    const float inv = ts > 1e-9f ? 1.0f / ts : 1.0f;
    for (uint32_t k = tid; k < top_k; k += tg) {
        out_ids[(size_t)tok * top_k + k] = top_i[k];
        out_w[(size_t)tok * top_k + k] = top_v[k] * inv;
    }
}

cudaError_t launch_moe_softmax_topk(const float *logits, uint32_t n_tokens, uint32_t n_experts, uint32_t top_k,
                                    uint32_t *out_ids, float *out_w, cudaStream_t st) {
    const uint32_t tg = n_experts < 128 ? n_experts : 128;
    const size_t smem = (2 * (size_t)tg + n_experts + 128) * sizeof(float);
    moe_softmax_topk_kernel<<<n_tokens, tg, smem, st>>>(logits, n_tokens, n_experts, top_k, out_ids, out_w);
    return cudaGetLastError();
}

__device__ __forceinline__ float silu_mul_one(float g, float u) { return g / (1.0f + expf(-g)) * u; }

__global__ void silu_mul_kernel(const float *gate, const float *up, float *out, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = silu_mul_one(gate[i], up[i]);
}

// Four elements per thread with 16-byte accesses (all three arrays 16-byte aligned); grid-stride.
__global__ void __launch_bounds__(256) silu_mul_vec4_kernel(const float4 *gate, const float4 *up, float4 *out, uint32_t n4) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) {
        const float4 g = __ldg(gate + i), u = __ldg(up + i);
        out[i] = make_float4(silu_mul_one(g.x, u.x), silu_mul_one(g.y, u.y), silu_mul_one(g.z, u.z), silu_mul_one(g.w, u.w));
    }
}

cudaError_t launch_silu_mul(const float *gate, const float *up, float *out, uint32_t n, cudaStream_t st) {
    const uint32_t n4 = n / 4;
    if (n4 && ((((uintptr_t)gate | (uintptr_t)up | (uintptr_t)out) & 15u) == 0)) {
        uint32_t blocks = (n4 + 255) / 256;
        if (blocks > 148 * 8) blocks = 148 * 8;
        silu_mul_vec4_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const float4 *>(gate), reinterpret_cast<const float4 *>(up),
                                                     reinterpret_cast<float4 *>(out), n4);
        if (n % 4) silu_mul_kernel<<<1, 32, 0, st>>>(gate + 4 * n4, up + 4 * n4, out + 4 * n4, n % 4);
        return cudaGetLastError();
    }
    silu_mul_kernel<<<(n + 255) / 256, 256, 0, st>>>(gate, up, out, n);
    return cudaGetLastError();
}

// `local_ids` (optional, expert-sharded form): slots whose entry is kNotLocal belong to another rank's experts;
// their rows of y were never written here and are not read.
__global__ void moe_weighted_reduce_kernel(const float *w, const float *y, const float *sh_logit, const float *y_shared,
                                           const float *residual, const uint32_t *local_ids, float *out,
                                           uint32_t n_tokens, uint32_t top_k, uint32_t h) {
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (c >= h || t >= n_tokens) return;
    float acc = 0.0f;
    for (uint32_t k = 0; k < top_k; k++) {
        const size_t slot = (size_t)t * top_k + k;
        if (local_ids && local_ids[slot] == kNotLocal) continue;
        acc += w[slot] * y[slot * h + c];
    }
    if (y_shared) {
        const float gate = sh_logit ? 1.0f / (1.0f + expf(-sh_logit[t])) : 1.0f;
        acc += gate * y_shared[(size_t)t * h + c];
    }
    if (residual) acc += residual[(size_t)t * h + c];
    out[(size_t)t * h + c] = acc;
}

cudaError_t launch_moe_weighted_reduce(const float *w, const float *y, const float *sh_logit, const float *y_shared,
                                       const float *residual, const uint32_t *local_ids, float *out, uint32_t n_tokens,
                                       uint32_t top_k, uint32_t h, cudaStream_t st) {
    dim3 grid((h + 255) / 256, n_tokens);
    moe_weighted_reduce_kernel<<<grid, 256, 0, st>>>(w, y, sh_logit, y_shared, residual, local_ids, out, n_tokens, top_k, h);
    return cudaGetLastError();
}

// Expert-sharded routing: this rank owns the experts [lo, lo + count).  Global ids become local ones (id - lo);
// entries of other ranks' experts become kNotLocal, which every routed kernel treats as "no expert" (no tile is
// built for it; the mat-vec form writes a zero row).
__global__ void moe_expert_shard_route_kernel(const uint32_t *ids, uint32_t *local_ids, uint32_t n, uint32_t lo,
                                              uint32_t count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t id = ids[i];
    local_ids[i] = (id >= lo && id - lo < count) ? id - lo : kNotLocal;
}

cudaError_t launch_moe_expert_shard_route(const uint32_t *ids, uint32_t *local_ids, uint32_t n, uint32_t lo, uint32_t count,
                                          cudaStream_t st) {
    moe_expert_shard_route_kernel<<<(n + 255) / 256, 256, 0, st>>>(ids, local_ids, n, lo, count);
    return cudaGetLastError();
}

}  // namespace mlxn
