/*
 * mlxn_b200 — C ABI of the B200 (sm_100a) implementation of mlx-native's GGML
 * block-quantized matmul path.
 *
 * Every entry point replaces one piece of the upstream Rust API; the upstream
 * location (path inside the mlx-native repository, file:line) is cited beside
 * it.  All functions return an mlxn_status; on failure a human-readable
 * message (the upstream error text where one exists) is available from
 * mlxn_last_error_message() on the calling thread.  No function panics or
 * aborts.  Handles are opaque and reference counted where the upstream type is
 * `Clone`.
 *
 * Threading: devices and buffers may be shared between threads; an encoder and
 * a registry are used by one thread at a time (as upstream: src/encoder.rs:593-607,
 * src/kernel_registry.rs:31-36).
 *
 * There is no CPU fallback: every compute entry point launches CUDA kernels and
 * fails with MLXN_DEVICE_NOT_FOUND when no CUDA device is usable.
 */
#ifndef MLXN_B200_H
#define MLXN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes: one per upstream MlxError variant that this path can raise (src/error.rs:21-84) */
typedef enum mlxn_status {
    MLXN_OK = 0,
    MLXN_DEVICE_NOT_FOUND = 1,        /* MlxError::DeviceNotFound */
    MLXN_COMMAND_BUFFER_ERROR = 2,    /* MlxError::CommandBufferError (is_transient() == true) */
    MLXN_KERNEL_NOT_FOUND = 3,        /* MlxError::KernelNotFound */
    MLXN_BUFFER_ALLOCATION_ERROR = 4, /* MlxError::BufferAllocationError */
    MLXN_INVALID_ARGUMENT = 5,        /* MlxError::InvalidArgument */
    MLXN_UNSUPPORTED_DTYPE = 6        /* MlxError::UnsupportedDtype */
} mlxn_status;

/* Message of the last failing call on this thread ("" if none).  Valid until the next failing call. */
const char *mlxn_last_error_message(void);
/* Upstream MlxError::is_transient (src/error.rs:87-89). */
int mlxn_status_is_transient(int status);

/* ---- element types: upstream DType (src/dtypes.rs:7-51) */
typedef enum mlxn_dtype {
    MLXN_F32 = 0, MLXN_F16 = 1, MLXN_BF16 = 2, MLXN_U8 = 3, MLXN_U16 = 4, MLXN_U32 = 5, MLXN_I32 = 6
} mlxn_dtype;
size_t mlxn_dtype_size(int dtype);       /* DType::size_of; 0 for an unknown code */
const char *mlxn_dtype_name(int dtype);  /* DType::name */

/* ---- GGML block types: upstream GgmlType (src/ops/quantized_matmul_ggml.rs:48-100) */
typedef enum mlxn_ggml_type {
    MLXN_GGML_F32 = 0, MLXN_GGML_F16 = 1, MLXN_GGML_Q4_0 = 2, MLXN_GGML_Q8_0 = 3,
    MLXN_GGML_Q4_K = 4, MLXN_GGML_Q5_K = 5, MLXN_GGML_Q6_K = 6, MLXN_GGML_I16 = 7
} mlxn_ggml_type;
uint32_t mlxn_ggml_block_values(int ggml_type); /* GgmlType::block_values (:79-90) */
uint32_t mlxn_ggml_block_bytes(int ggml_type);  /* GgmlType::block_bytes  (:93-104) */

/* Routing thresholds (src/ops/quantized_matmul_ggml.rs:180, src/ops/quantized_matmul_id_ggml.rs:397). */
#define MLXN_MM_ROUTING_THRESHOLD 8u
#define MLXN_MM_ID_ROUTING_THRESHOLD 32u
/* The expert-routed threshold in force: the constant above unless the environment variable
 * HF2Q_MM_ID_ROUTING_THRESHOLD overrides it (src/ops/quantized_matmul_id_ggml.rs:406-423). */
uint32_t mlxn_mm_id_routing_threshold(void);

typedef struct mlxn_device mlxn_device;     /* MlxDevice      src/device.rs:22-26 */
typedef struct mlxn_buffer mlxn_buffer;     /* MlxBuffer      src/buffer.rs:63-66 */
typedef struct mlxn_pool mlxn_pool;         /* MlxBufferPool  src/buffer_pool.rs:53-67 */
typedef struct mlxn_encoder mlxn_encoder;   /* CommandEncoder src/encoder.rs:507-591 */
typedef struct mlxn_registry mlxn_registry; /* KernelRegistry src/kernel_registry.rs:37-44 */
typedef struct mlxn_graph mlxn_graph;       /* a captured, replayable encoder (CUDA graph) */

/* ---- device ------------------------------------------------------------------------------ */
/* MlxDevice::new (src/device.rs:36-72).  ordinal < 0 selects the current CUDA device. */
int mlxn_device_create(int ordinal, mlxn_device **out);
void mlxn_device_destroy(mlxn_device *dev);
/* MlxDevice::name (src/device.rs:222).  The string lives as long as the device. */
const char *mlxn_device_name(const mlxn_device *dev);
int mlxn_device_ordinal(const mlxn_device *dev);
int mlxn_device_sm_count(const mlxn_device *dev);

/* ---- buffers ----------------------------------------------------------------------------- */
/* MlxDevice::alloc_buffer (src/device.rs:130-194): zero-filled device memory; byte_len == 0 is
 * MLXN_INVALID_ARGUMENT; an allocation failure is MLXN_BUFFER_ALLOCATION_ERROR. */
int mlxn_buffer_alloc(mlxn_device *dev, size_t byte_len, int dtype, const size_t *shape, size_t rank,
                      mlxn_buffer **out);
/* MlxBuffer::from_raw (src/buffer.rs:122): adopt device memory owned by the caller (for example a
 * tensor of another library).  The memory is not freed when the handle is released. */
int mlxn_buffer_wrap(mlxn_device *dev, void *device_ptr, size_t byte_len, int dtype, const size_t *shape,
                     size_t rank, mlxn_buffer **out);
/* MlxBuffer::slice_view (src/buffer.rs:187-197): a handle onto [byte_offset, byte_offset +
 * n_elements*size_of(dtype)) of the same storage.  Out of range is MLXN_INVALID_ARGUMENT (upstream panics). */
int mlxn_buffer_slice_view(mlxn_buffer *buf, uint64_t byte_offset, size_t n_elements, mlxn_buffer **out);
/* Clone / Drop of the upstream handle. */
void mlxn_buffer_retain(mlxn_buffer *buf);
void mlxn_buffer_release(mlxn_buffer *buf);
int mlxn_buffer_dtype(const mlxn_buffer *buf);            /* src/buffer.rs:209 */
size_t mlxn_buffer_rank(const mlxn_buffer *buf);          /* src/buffer.rs:215 */
size_t mlxn_buffer_shape(const mlxn_buffer *buf, size_t axis);
size_t mlxn_buffer_byte_len(const mlxn_buffer *buf);      /* src/buffer.rs:221 (length of this view) */
size_t mlxn_buffer_element_count(const mlxn_buffer *buf); /* src/buffer.rs:227 */
uint64_t mlxn_buffer_byte_offset(const mlxn_buffer *buf); /* src/buffer.rs:253 */
/* MlxBuffer::contents_ptr (src/buffer.rs:238): here a DEVICE address (HBM), not host-readable. */
void *mlxn_buffer_device_ptr(const mlxn_buffer *buf);
/* MlxBuffer::as_mut_slice (src/buffer.rs:324-348) / as_slice (:294-317).  Upstream memory is unified;
 * here each storage lazily gets a pinned host shadow.  host_map(write=1) returns the shadow and marks it
 * newer than HBM; the next operation that binds the buffer uploads it on the encoder's stream.
 * host_map(write=0) first waits for the last encoder that wrote the buffer and downloads it if HBM is
 * newer.  The pointer addresses this view's first byte and stays valid until the storage is freed. */
int mlxn_buffer_host_map(mlxn_buffer *buf, int write, void **host_ptr);
/* Synchronous copies for callers that keep their own host arrays. */
int mlxn_buffer_upload(mlxn_buffer *buf, const void *src, size_t byte_len, size_t dst_offset);
int mlxn_buffer_download(mlxn_buffer *buf, void *dst, size_t byte_len, size_t src_offset);

/* ---- pool: MlxBufferPool (src/buffer_pool.rs:78-378), power-of-two buckets ------------------ */
int mlxn_pool_create(mlxn_pool **out);
void mlxn_pool_destroy(mlxn_pool *pool);
int mlxn_pool_alloc(mlxn_pool *pool, mlxn_device *dev, size_t byte_len, int dtype, const size_t *shape,
                    size_t rank, mlxn_buffer **out);                 /* :97-112 */
/* alloc_batch (:114-135): `count` buffers in one call, all or nothing: on failure the buffers this call took go
 * back to the pool and out[] holds no handle.  `shapes` concatenates the requests' shapes, ranks[i] entries each
 * (both may be NULL: no shapes). */
int mlxn_pool_alloc_batch(mlxn_pool *pool, mlxn_device *dev, size_t count, const size_t *byte_lens, const int *dtypes,
                          const size_t *shapes, const size_t *ranks, mlxn_buffer **out);
int mlxn_pool_release(mlxn_pool *pool, mlxn_buffer *buf);            /* :218-222 (consumes the handle) */
void mlxn_pool_reset(mlxn_pool *pool);                               /* :248-252 */
int mlxn_pool_register_existing(mlxn_pool *pool, mlxn_device *dev, mlxn_buffer *buf); /* :306-357 (no-op on CUDA) */
size_t mlxn_pool_free_count(const mlxn_pool *pool);                  /* :359 */
size_t mlxn_pool_free_bytes(const mlxn_pool *pool);                  /* :364 */
size_t mlxn_pool_in_use_count(const mlxn_pool *pool);                /* :372 */
void mlxn_pool_clear(mlxn_pool *pool);                               /* :378 */

/* ---- kernel registry: KernelRegistry (src/kernel_registry.rs:49, 667-720, 870-880) ----------
 * Kernels are compiled ahead of time; the registry is a name table with the upstream kernel names
 * ("kernel_mul_mv_q4_0_f32", "kernel_mul_mm_id_map0_ne20_8", ...).  get_pipeline resolves a name
 * (MLXN_KERNEL_NOT_FOUND if unknown) and records it as cached. */
int mlxn_registry_create(mlxn_registry **out);
void mlxn_registry_destroy(mlxn_registry *reg);
int mlxn_registry_get_pipeline(mlxn_registry *reg, mlxn_device *dev, const char *name);
int mlxn_registry_is_cached(const mlxn_registry *reg, const char *name);
size_t mlxn_registry_cached_count(const mlxn_registry *reg);
size_t mlxn_registry_source_count(const mlxn_registry *reg);

/* ---- command encoder: CommandEncoder (src/encoder.rs) --------------------------------------
 * Upstream encodes with MTLDispatchTypeConcurrent: dispatches may overlap unless memory_barrier() separates them
 * (src/encoder.rs:837-853), and its tracked mode inserts that barrier itself where the buffers of a new dispatch
 * conflict with the running group (src/graph.rs:1494-1530).  The same holds here: an encoder owns two CUDA stream
 * "lanes"; an operation none of whose buffers conflicts (read-after-write, write-after-read, write-after-write,
 * or an input whose host view still has to be uploaded) with the operations encoded since the last barrier goes
 * to the other lane and may overlap them; a conflict, memory_barrier(), commit, a capture boundary and
 * mlxn_encoder_stream() join the lanes first.  Results are therefore those of encode order. */
int mlxn_encoder_create(mlxn_device *dev, mlxn_encoder **out);       /* MlxDevice::command_encoder src/device.rs:86-88 */
void mlxn_encoder_destroy(mlxn_encoder *enc);                        /* Drop: waits for submitted work */
int mlxn_encoder_memory_barrier(mlxn_encoder *enc);                  /* src/encoder.rs:886-906 */
int mlxn_encoder_commit(mlxn_encoder *enc);                          /* src/encoder.rs:2022 */
int mlxn_encoder_wait_until_completed(mlxn_encoder *enc);            /* src/encoder.rs:2038 */
int mlxn_encoder_commit_and_wait(mlxn_encoder *enc);                 /* src/encoder.rs:1852-1879 */
/* commit_wait_with_gpu_time (src/encoder.rs:2001-2014): device time of the committed work in seconds. */
int mlxn_encoder_commit_wait_with_gpu_time(mlxn_encoder *enc, double *gpu_seconds);
/* The encoder's cudaStream_t (lane 0), after it has been made to wait for the other lane: work the caller
 * enqueues on it runs behind everything encoded so far.  NULL on failure. */
void *mlxn_encoder_stream(mlxn_encoder *enc);
/* commit_labeled / commit_and_wait_labeled (src/encoder.rs:1893-1935): as commit / commit_and_wait; with the
 * environment variable MLX_PROFILE_CB=1 the command buffer's device time is printed to stderr under `label`
 * when its wait returns (upstream's per-command-buffer profile, src/encoder.rs:1882-1935). */
int mlxn_encoder_commit_labeled(mlxn_encoder *enc, const char *label);
int mlxn_encoder_commit_and_wait_labeled(mlxn_encoder *enc, const char *label);
/* The profile table (src/kernel_profile.rs): command buffers and device nanoseconds recorded under `label`. */
int mlxn_profile_cb_get(const char *label, uint64_t *count, uint64_t *nanoseconds);
void mlxn_profile_cb_reset(void);
/* Replay support for launch-bound decode loops: everything encoded between begin and end is recorded
 * into a CUDA graph instead of being run; graph_launch replays it on the encoder's stream.
 * Lifetimes: the graph keeps a reference to every buffer its operations bind, owns the scratch arenas its
 * kernels use (eager work on the same encoder never shares or frees them) and shares the recording encoder's
 * status block, so it stays valid after that encoder is destroyed; it replays only on the encoder that recorded
 * it (or on the pooled successor that inherited its status block), other encoders get MLXN_INVALID_ARGUMENT.
 * A host view of an input whose upload is part of the graph may be rewritten right after graph_launch: the
 * write waits until the replay has read the view. */
int mlxn_encoder_begin_capture(mlxn_encoder *enc);
int mlxn_encoder_end_capture(mlxn_encoder *enc, mlxn_graph **out);
int mlxn_graph_launch(mlxn_graph *graph, mlxn_encoder *enc);
void mlxn_graph_destroy(mlxn_graph *graph);

/* Global counters (src/encoder.rs:271-330). */
uint64_t mlxn_dispatch_count(void);
uint64_t mlxn_sync_count(void);
uint64_t mlxn_cmd_buf_count(void);
uint64_t mlxn_barrier_count(void);
void mlxn_reset_counters(void);
/* Number of CUDA kernels this library has launched since reset_counters (dispatch_count counts
 * operations; one operation may launch several kernels). */
uint64_t mlxn_kernel_launch_count(void);

/* ---- the hot path -------------------------------------------------------------------------- */
/* GgmlQuantizedMatmulParams (src/ops/quantized_matmul_ggml.rs:183-194) */
typedef struct mlxn_qmm_params {
    uint32_t m, n, k;
    uint32_t ggml_type; /* mlxn_ggml_type */
} mlxn_qmm_params;

/* GgmlQuantizedMatmulIdParams (src/ops/quantized_matmul_id_ggml.rs:44-61) */
typedef struct mlxn_qmm_id_params {
    uint32_t n_tokens, top_k, n, k, n_experts;
    uint32_t ggml_type; /* mlxn_ggml_type */
    uint64_t expert_stride;
} mlxn_qmm_id_params;

/* quantized_matmul_ggml (src/ops/quantized_matmul_ggml.rs:267-361):
 * output[m,n] f32 = input[m,k] f32 * dequant(weight[n][k/QK] blocks)^T.  Same validation, same messages.
 * m <= 8 (or k < 32) runs the fused dequant-dot mat-vec kernels, larger m the tensor-core mat-mat. */
int mlxn_quantized_matmul_ggml(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input,
                               mlxn_buffer *weight, mlxn_buffer *output, const mlxn_qmm_params *params);
/* GgmlQuantizedMatmulPerm021Params (src/ops/quantized_matmul_ggml.rs:612-625). */
typedef struct mlxn_qmm_perm021_params {
    uint32_t m, n, k;      /* k = n_heads * head_dim */
    uint32_t head_dim;     /* a positive multiple of 32 */
    uint32_t ggml_type;    /* MLXN_GGML_Q4_0 or MLXN_GGML_Q6_K */
} mlxn_qmm_perm021_params;
/* quantized_matmul_mm_tensor_perm021 (src/ops/quantized_matmul_ggml.rs:640-742; kernel
 * src/shaders/quantized_matmul_mm_tensor.metal:411-598): the tensor-core mat-mat whose activations are the
 * attention output where it lies, bf16 [n_heads, seq_len = m, head_dim], cast bf16 -> f32 -> f16 as upstream does
 * (:520-539).  weight: [n, k] blocks; output: f32 [m, n].  Always the mat-mat route, at any m. */
int mlxn_quantized_matmul_mm_tensor_perm021(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev,
                                            mlxn_buffer *input_bf16, mlxn_buffer *weight, mlxn_buffer *output,
                                            const mlxn_qmm_perm021_params *params);
/* dispatch_mm_for_test (src/ops/quantized_matmul_ggml.rs:371-402): force the mat-mat path at any m. */
int mlxn_dispatch_mm_for_test(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input,
                              mlxn_buffer *weight, mlxn_buffer *output, const mlxn_qmm_params *params);

/* quantized_matmul_id_ggml (src/ops/quantized_matmul_id_ggml.rs:163-276):
 * output[t*top_k+s, :] = dequant(weight[ids[t*top_k+s]]) * input[t].  The mat-mat route allocates its
 * routing scratch per call, as upstream does. */
int mlxn_quantized_matmul_id_ggml(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input,
                                  mlxn_buffer *weight, mlxn_buffer *ids, mlxn_buffer *output,
                                  const mlxn_qmm_id_params *params);
/* quantized_matmul_id_swiglu_q4_0 (src/ops/quantized_matmul_id_ggml.rs:551-670; kernel
 * src/shaders/quantized_matmul_id_ggml.metal:231-319), here for Q4_0, Q8_0 and Q6_K: the fused SwiGLU + expert-routed
 * mat-vec of the MoE down projection.  gate, up: f32 [n_tokens * top_k, k], one row per (token, slot) pair;
 * output[r, :] = W[ids[r]] . (silu(gate[r, :]) * up[r, :]).  The activations are formed while they are loaded: there
 * is no separate SwiGLU launch and no [rows, k] intermediate in memory. */
int mlxn_quantized_matmul_id_swiglu(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *gate,
                                    mlxn_buffer *up, mlxn_buffer *weight, mlxn_buffer *ids, mlxn_buffer *output,
                                    const mlxn_qmm_id_params *params);
/* The expert half of a MoE FFN layer as one call (no upstream counterpart; upstream's callers encode
 * quantized_matmul_id_ggml for gate and up, silu_mul, and quantized_matmul_id_ggml with n_tokens * top_k rows and
 * top_k = 1 for down, e.g. benches/bench_mul_mm_id_qwen36_ffn.rs).  Results are those of that chain, bit for bit.
 *   x f32 [n_tokens, hidden]; ids u32 [n_tokens * top_k]; gate_w / up_w: stacked [n_experts][ffn][hidden / QK] blocks;
 *   down_w: [n_experts][hidden][ffn / QK] blocks; gate_out, up_out f32 [n_tokens * top_k, ffn] (intermediates the caller
 *   provides); down_out f32 [n_tokens * top_k, hidden], one row per (token, slot) pair, to be reduced with
 *   mlxn_moe_weighted_reduce.
 * More than HF2Q_MM_ID_ROUTING_THRESHOLD tokens: the pairs are bucketed once, the tile list is built once, x is packed
 * once for gate and up, and silu(gate) * up is formed while the down projection's operand is packed (seven launches
 * instead of thirteen).  Fewer tokens: the routed mat-vecs and the fused SwiGLU mat-vec.  What up_out holds afterwards
 * depends on the route (the up projection, or silu(gate) * up where the stand-alone SwiGLU ran over it).
 * A pair whose id names no expert gets a zero row in down_out; its rows of gate_out / up_out are unspecified. */
typedef struct mlxn_moe_ffn_params {
    uint32_t n_tokens, top_k, hidden, ffn, n_experts;
    uint32_t gate_type, up_type, down_type;           /* mlxn_ggml_type */
    uint64_t gate_stride, up_stride, down_stride;     /* bytes from one expert's matrix to the next */
} mlxn_moe_ffn_params;
int mlxn_moe_ffn_layer(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *x, mlxn_buffer *ids,
                       mlxn_buffer *gate_w, mlxn_buffer *up_w, mlxn_buffer *down_w, mlxn_buffer *gate_out,
                       mlxn_buffer *up_out, mlxn_buffer *down_out, const mlxn_moe_ffn_params *params);
/* quantized_matmul_id_ggml_pooled (src/ops/quantized_matmul_id_ggml.rs:288-389) with the caller-owned
 * IdMmScratch {htpe, hids} (:672-719) and its capacities (check_capacity :704-718). */
int mlxn_quantized_matmul_id_ggml_pooled(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev,
                                         mlxn_buffer *input, mlxn_buffer *weight, mlxn_buffer *ids,
                                         mlxn_buffer *output, mlxn_buffer *htpe, mlxn_buffer *hids,
                                         uint32_t n_experts_cap, uint32_t n_tokens_cap,
                                         const mlxn_qmm_id_params *params);
/* dispatch_id_mm_for_test (src/ops/quantized_matmul_id_ggml.rs:902-1129): forced two-stage route
 * (bucket by expert, then grouped mat-mat) with explicit scratch.  htpe: u32[n_experts];
 * hids: i32[n_experts, n_tokens]; both are left holding the bucketing result. */
int mlxn_dispatch_id_mm_for_test(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input,
                                 mlxn_buffer *weight, mlxn_buffer *ids, mlxn_buffer *htpe, mlxn_buffer *hids,
                                 mlxn_buffer *output, const mlxn_qmm_id_params *params);
/* GgmlIdMmDispatchParams::htpe_bytes / hids_bytes (src/ops/quantized_matmul_id_ggml.rs:850-879). */
size_t mlxn_id_mm_htpe_bytes(const mlxn_qmm_id_params *params);
size_t mlxn_id_mm_hids_bytes(const mlxn_qmm_id_params *params);

/* ---- MoE glue around the expert-routed matmul ------------------------------------------------ */
/* moe_softmax_topk (src/ops/moe_softmax_topk.rs:112-128, src/shaders/moe_softmax_topk.metal:27-148):
 * logits f32 [n_tokens, n_experts] -> ids u32 [n_tokens*top_k], weights f32 [n_tokens*top_k]. */
int mlxn_moe_softmax_topk(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *logits,
                          mlxn_buffer *out_ids, mlxn_buffer *out_weights, uint32_t n_tokens,
                          uint32_t n_experts, uint32_t top_k);
/* silu_mul (src/ops/silu_mul.rs, src/shaders/silu_mul.metal:17-30): out = gate/(1+exp(-gate)) * up. */
int mlxn_silu_mul(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *gate, mlxn_buffer *up,
                  mlxn_buffer *out, uint32_t n);
/* moe_weighted_reduce (src/ops/moe_weighted_reduce.rs, src/shaders/moe_weighted_reduce.metal:33-66):
 * out[t,h] = sum_k w[t,k] * y[t*top_k+k, h] (+ sigmoid(sh_logit[t]) * y_shared[t,h]) (+ residual[t,h]).
 * y_shared/sh_logit and residual may be NULL. */
int mlxn_moe_weighted_reduce(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *expert_w,
                             mlxn_buffer *y_expert, mlxn_buffer *sh_logit, mlxn_buffer *y_shared,
                             mlxn_buffer *residual, mlxn_buffer *out, uint32_t n_tokens, uint32_t top_k,
                             uint32_t h);

/* ---- expert-sharded MoE (no counterpart in the reference: it runs on one GPU) ------------------------
 * Rank r of g holds the experts [r E/g, (r+1) E/g) (a contiguous byte range of the stacked expert weights at
 * `expert_stride`).  Activations and the router's ids/weights are replicated, so "dispatch" is a local filter:
 * mlxn_moe_expert_shard_route turns the global ids into local ones (id - expert_lo) and marks the pairs of
 * other ranks' experts with 0xFFFFFFFF, which mlxn_quantized_matmul_id_ggml treats as "no expert" (n_experts
 * in its params is the local count).  mlxn_moe_weighted_reduce_local sums this rank's pairs only; the ranks'
 * partial results are then added up by one all-reduce (the combine step). */
int mlxn_moe_expert_shard_route(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *ids,
                                mlxn_buffer *local_ids, uint32_t n_pairs, uint32_t expert_lo, uint32_t expert_count);
int mlxn_moe_weighted_reduce_local(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *expert_w,
                                   mlxn_buffer *y_expert, mlxn_buffer *local_ids, mlxn_buffer *out, uint32_t n_tokens,
                                   uint32_t top_k, uint32_t h);

/* ---- mat-mat without any allocation (no counterpart in the reference) ------------------------------
 * For callers that cannot allocate device memory when they need the product: a serving process whose own
 * allocator has claimed all of HBM, a latency-critical loop that must stay off the driver's allocation
 * path, or a plug-in that only ever receives pointers.  Same result as mlxn_dispatch_mm_for_test (the
 * tensor-core mat-mat at any m), but the packed f16 activations go into a fixed 16 MiB array compiled into
 * the library instead of the encoder's arena, and inputs/outputs are plain device pointers on `cuda_stream`
 * (a cudaStream_t; NULL = the default stream).  Nothing is allocated or freed, on the host or the device.
 * Limits and rules:
 *  - the packed activations, ceil(m/NT)*NT * ceil(k/64)*64 * 2 bytes, must fit in
 *    mlxn_noalloc_scratch_limit() bytes (m*k up to about 8M elements); larger calls are refused with
 *    MLXN_INVALID_ARGUMENT and a message naming both sizes;
 *  - dense Q4_0 / Q8_0 / Q6_K only; K a multiple of 32;
 *  - the call works on the CURRENT device: `cuda_stream` and the three pointers must belong to it (a stream of
 *    another device is refused with MLXN_INVALID_ARGUMENT where the runtime can tell);
 *  - the first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
 *    current) — make that first call outside any stream capture;
 *  - all calls on a device share the one array: two calls whose kernels overlap on the GPU (different
 *    streams) race; the array keeps the last call's tiles, and every call rewrites all the tiles it reads;
 *  - a kernel wait that gives up is not reported (there is no status word without an allocation). */
size_t mlxn_noalloc_scratch_limit(void);
int mlxn_quantized_matmul_ggml_mm_noalloc(void *cuda_stream, const void *input_dev, const void *weight_dev,
                                          void *output_dev, const mlxn_qmm_params *params);

/* Row-sharded matmul for tensor parallelism (no upstream counterpart: upstream is single-GPU).  This rank holds
 * params->n of the n_total weight rows, rows [col0, col0 + n) of the full matrix.  `output` is this rank's full
 * result buffer, f32 [m, n_total]; the kernels store their columns there AND at the same place in the other ranks'
 * result buffers (`peer_outputs`: device addresses mapped into this process, e.g. CUDA IPC or symmetric memory; at
 * most 7), so that every rank holds the whole result once all ranks' kernels have finished, without a collective
 * launch.  m <= 8 takes the mat-vec kernels (the register-level one stores to the peers from its own epilogue: one
 * launch per call), larger m the tensor-core mat-mat, whose epilogue sends each finished tile to the peers while the
 * other tiles are still being computed.  The caller orders ranks (a barrier between this call and the first use of
 * the full result, and between that use and the next call that writes the buffers). */
int mlxn_quantized_matmul_ggml_sharded(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input,
                                       mlxn_buffer *weight, mlxn_buffer *output, const mlxn_qmm_params *params,
                                       uint32_t n_total, uint32_t col0, void *const *peer_outputs, uint32_t n_peers);

/* Cross-rank barrier for the row-sharded and expert-sharded forms (one process per GPU; no upstream counterpart).
 * Every rank owns a zero-initialised flag array uint32[world] in memory its peers can store to (symmetric or IPC
 * memory); flag_ptrs[r] is rank r's array as mapped into this process.  The call enqueues, behind everything encoded
 * so far, a kernel that publishes `epoch` (which the caller raises by one per barrier) to every rank and waits until
 * every rank's epoch has arrived here: what the ranks stored to one another before the barrier is visible after it.
 * The wait is bounded by `limit_us` (1..10000000): when it runs out the next commit reports MLXN_COMMAND_BUFFER_ERROR
 * ("gave up waiting for another rank") and the GPU stays usable.  world <= 32.  Plain peer loads and stores only. */
int mlxn_peer_barrier(mlxn_encoder *enc, uint32_t rank, uint32_t world, void *const *flag_ptrs, uint32_t epoch,
                      uint32_t limit_us);

/* ---- tuning and introspection (no upstream counterpart) -------------------------------------- */
/* Selects kernel variants for cross-checks: key/value pairs
 *   "qmv" = auto | mma | tc | stream | simple   (auto: per shape and m, the fastest of the register-level tensor-core
 *           kernel "mma" and the tensor-memory kernel "tc", the streaming SIMT kernel for shapes neither takes;
 *           mma, stream and simple give bit-reproducible results, tc may differ in the last bit from run to run),
 *   "qmm" = tc | simt,
 *   "qmv_mma_ctas" = 1 | 2 (CTAs per SM of the mma kernel), "qmv_mma_tpw" = 0 | 1 | 2 | 4 (its row-group size; 0 = auto).
 * Unknown keys are MLXN_INVALID_ARGUMENT.  The defaults are the fast paths. */
int mlxn_set_option(const char *key, const char *value);
/* Exercises the give-up path of the kernels' bounded waits: enqueues a one-CTA kernel that waits `limit_us`
 * microseconds (1..100000) on a barrier nothing arrives at, records "wait for data timed out" in the encoder's
 * status word and returns normally.  The next commit_and_wait reports MLXN_COMMAND_BUFFER_ERROR; the encoder and
 * the device stay usable (src/encoder.rs:1867-1878 is the upstream path that surfaces a failed command buffer). */
int mlxn_debug_wait_probe(mlxn_encoder *enc, uint32_t limit_us);
/* Name of the kernel variant the last operation on this thread launched (for tests and profiles). */
const char *mlxn_last_kernel_name(void);

#ifdef __cplusplus
}
#endif
#endif /* MLXN_B200_H */
