// CUDA runtime layer and C ABI of the library: device, buffers (HBM + lazily created pinned host
// shadow), power-of-two buffer pool, kernel-name registry, stream-backed command encoder with CUDA
// graph capture, global counters, and the host-side dispatchers of the quantized matmul path.
// The dispatchers mirror upstream src/ops/quantized_matmul_ggml.rs and
// src/ops/quantized_matmul_id_ggml.rs: same validation order, same messages, same routing rules.
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "../../include/mlxn_b200.h"
#include "common.cuh"
#include "ptx.cuh"

namespace mlxn {
cudaError_t launch_qmv(int ggml_type, const QmvArgs &a, bool want_stream, int sm_count, cudaStream_t st,
                       const char **kname);
bool qmv_tc_supported(int ggml_type, const QmvArgs &a);
size_t qmv_tc_scratch_bytes(const QmvArgs &a);
cudaError_t launch_qmv_tc(int ggml_type, const QmvArgs &a, uint8_t *scratch, uint32_t *flags, int sm_count, cudaStream_t st,
                          cudaStream_t pub_st, cudaEvent_t pub_ev, int *launches);
bool qmv_mma_supported(int ggml_type, const QmvArgs &a);
bool qmv_mma_supported_routed(int ggml_type, const QmvArgs &a);
bool qmv_stream_available(int ggml_type, const QmvArgs &a, int sm_count);
constexpr size_t kMvBatchMax = 16;   // mat-vecs one launch of the register-level kernel carries (kMwMaxProbs)
bool qmv_mma_pair_mode(int ggml_type, const QmvArgs &a);
cudaError_t launch_qmv_mma(int ggml_type, const QmvArgs *ops, int nops, int sm_count, int ctas_per_sm, int tpw, cudaStream_t st);
cudaError_t launch_qmm_tc(int ggml_type, const QmmArgs &a, bool routed, uint32_t nt, uint8_t *scratch, cudaStream_t st,
                          int *launches);
cudaError_t launch_qmm_simt(int ggml_type, const QmmArgs &a, bool routed, uint32_t max_rows, cudaStream_t st);
size_t qmm_tc_scratch_bytes(const QmmArgs &a, uint32_t nt, bool routed);
uint32_t qmm_tc_pick_nt(int ggml_type, uint32_t rows, uint32_t n, int sm_count, bool routed);
bool qmm_tc_supported(const QmmArgs &a);
cudaError_t launch_moe_map0(const uint32_t *ids, uint32_t n_tokens, uint32_t top_k, uint32_t n_experts,
                            uint32_t hids_stride, uint32_t *htpe, int32_t *hids, float *y, uint32_t n, cudaStream_t st);
cudaError_t launch_moe_softmax_topk(const float *logits, uint32_t n_tokens, uint32_t n_experts, uint32_t top_k,
                                    uint32_t *out_ids, float *out_w, cudaStream_t st);
cudaError_t launch_silu_mul(const float *gate, const float *up, float *out, uint32_t n, cudaStream_t st);
cudaError_t launch_moe_weighted_reduce(const float *w, const float *y, const float *sh_logit, const float *y_shared,
                                       const float *residual, const uint32_t *local_ids, float *out, uint32_t n_tokens,
                                       uint32_t top_k, uint32_t h, cudaStream_t st);
cudaError_t launch_moe_expert_shard_route(const uint32_t *ids, uint32_t *local_ids, uint32_t n, uint32_t lo, uint32_t count,
                                          cudaStream_t st);
}  // namespace mlxn

using namespace mlxn;

// ------------------------------------------------------------------------------------------------
// errors, counters, options
// ------------------------------------------------------------------------------------------------
static thread_local std::string g_last_error;
static thread_local const char *g_last_kernel = "";

static int fail(int status, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return status;
}
static int cuda_fail(cudaError_t e, const char *what) {
    cudaGetLastError();  // clear the runtime's sticky "last error" so later launches are not blamed for it
    return fail(MLXN_COMMAND_BUFFER_ERROR, "Command buffer error: %s: %s", what, cudaGetErrorString(e));
}
#define CUDA_TRY(expr, what)                          \
    do {                                              \
        cudaError_t _e = (expr);                      \
        if (_e != cudaSuccess) return cuda_fail(_e, what); \
    } while (0)

// error reporting for entry points that live in other translation units
int mlxn_detail_fail(int status, const char *msg) { return fail(status, "%s", msg); }
void mlxn_detail_count_launches(int launches);

static std::atomic<uint64_t> g_dispatch{0}, g_sync{0}, g_cmd_buf{0}, g_barrier{0}, g_launches{0};

void mlxn_detail_count_launches(int launches) {
    g_launches.fetch_add((uint64_t)launches);
    g_dispatch.fetch_add(1);
    g_last_kernel = "qmm_tc";
}

static std::atomic<int> g_opt_qmv{-1}, g_opt_qmm{-1};  // -1 unset; qmv: 0 simple, 1 stream, 2 tc, 3 auto, 4 mma; qmm: 0 simt, 1 tc
static std::atomic<int> g_opt_mma_ctas{2}, g_opt_mma_tpw{0};   // tuning knobs of the register-level mat-vec
static std::atomic<int> g_opt_mv_batch{1};                     // coalesce conflict-free mat-vecs into one launch
// ... and mat-vecs that depend on one another (barriers inside the launch).  Off by default: measured on B200 a barrier
// across the grid costs about a microsecond more than the overlapped launch of a separate kernel.
static std::atomic<int> g_opt_mv_chain{0};
static int opt_qmv() {
    int v = g_opt_qmv.load();
    if (v < 0) {
        const char *e = getenv("MLXN_QMV");
        v = (e && strcmp(e, "simple") == 0) ? 0 : (e && strcmp(e, "stream") == 0) ? 1 : (e && strcmp(e, "tc") == 0) ? 2
            : (e && strcmp(e, "mma") == 0) ? 4 : 3;
        g_opt_qmv = v;
    }
    return v;
}
static bool opt_qmv_stream() { return opt_qmv() >= 1; }
static bool opt_qmm_tc() {
    int v = g_opt_qmm.load();
    if (v < 0) {
        const char *e = getenv("MLXN_QMM");
        v = (e && strcmp(e, "simt") == 0) ? 0 : 1;
        g_opt_qmm = v;
    }
    return v == 1;
}

// ------------------------------------------------------------------------------------------------
// handle types
// ------------------------------------------------------------------------------------------------
struct mlxn_device {
    int ordinal;
    int sm_count;
    std::string name;
};

struct Storage {
    std::atomic<int> refs{1};
    int ordinal = 0;
    void *dptr = nullptr;
    size_t bytes = 0;
    bool owned = true;
    void *host = nullptr;      // pinned shadow, created on first host_map
    bool host_newer = false;   // shadow holds data not yet uploaded
    bool dev_newer = false;    // HBM holds data not yet reflected in the shadow
    cudaStream_t last_stream = nullptr;  // stream of the last operation that touched the storage
    bool has_last = false;
    bool kernel_written = false;  // some operation of this library has used the storage as an output
    struct mlxn_encoder *pend_enc = nullptr;  // encoder holding a not-yet-launched mat-vec that uses the storage
    std::mutex mu;
};

static void storage_release(Storage *s) {
    if (s->refs.fetch_sub(1) == 1) {
        int prev = 0;
        cudaGetDevice(&prev);
        cudaSetDevice(s->ordinal);
        if (s->owned && s->dptr) cudaFree(s->dptr);
        if (s->host) cudaFreeHost(s->host);
        cudaSetDevice(prev);
        delete s;
    }
}

struct mlxn_buffer {
    std::atomic<int> refs{1};
    Storage *st = nullptr;
    size_t offset = 0;
    size_t len = 0;
    int dtype = MLXN_U8;
    std::vector<size_t> shape;
    uint8_t *dev() const { return static_cast<uint8_t *>(st->dptr) + offset; }
};

struct mlxn_pool {
    std::map<size_t, std::vector<Storage *>> free_list;
    std::vector<std::pair<size_t, Storage *>> in_use;
};

struct mlxn_registry {
    std::set<std::string> cached;
};

// Device status words (see ST_* in common.cuh).  Ref-counted: the kernels of a captured graph keep writing to the
// block of the encoder that recorded them, so the block must outlive that encoder for as long as the graph exists.
struct StatusBlock {
    std::atomic<int> refs{1};
    int ordinal = 0;
    uint32_t *dev = nullptr;
};
static void status_block_release(StatusBlock *sb) {
    if (sb && sb->refs.fetch_sub(1) == 1) {
        int prev = 0;
        cudaGetDevice(&prev);
        cudaSetDevice(sb->ordinal);
        cudaFree(sb->dev);
        cudaSetDevice(prev);
        delete sb;
    }
}

struct mlxn_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t launches = 0;  // kernels recorded in the graph
    uint64_t dispatches = 0;
    // Host views and replays: the upload of an input whose host view was dirty at capture time is part of the
    // graph (it reads the pinned shadow again at every replay); outputs become "newer on the device" at every replay.
    std::vector<mlxn_buffer *> uploads, outputs;  // hold a reference each
    std::vector<bool> fetched;                    // per output: the graph copies it back to its host shadow itself
    std::vector<bool> covered;                    // per output: its storage is fetched by one of the graph's copies
    // What the recorded kernels address besides the caller's buffers belongs to the graph: the scratch arenas that
    // were in use while it was recorded (freed when the graph is destroyed) and the recording encoder's status block.
    int ordinal = 0;
    std::vector<std::pair<void *, size_t>> scratch;
    StatusBlock *sb = nullptr;
};

// Scratch arenas outlive their encoder: short-lived encoders (one per command buffer, as upstream uses them) would
// otherwise pay a cudaMalloc / cudaFree pair, which synchronises the device, for every mat-vec they encode.
struct ScratchBlock {
    int ordinal;
    void *ptr;
    size_t bytes;
};
static std::mutex g_scratch_mu;
static std::vector<ScratchBlock> g_scratch_free;
static void *scratch_take(int ordinal, size_t want, size_t *got) {
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    int best = -1;
    for (int i = 0; i < (int)g_scratch_free.size(); i++)
        if (g_scratch_free[i].ordinal == ordinal && g_scratch_free[i].bytes >= want &&
            (best < 0 || g_scratch_free[i].bytes < g_scratch_free[best].bytes))
            best = i;
    if (best < 0) return nullptr;
    void *p = g_scratch_free[best].ptr;
    *got = g_scratch_free[best].bytes;
    g_scratch_free.erase(g_scratch_free.begin() + best);
    return p;
}
static void scratch_give(int ordinal, void *p, size_t bytes) {  // the caller has made sure no kernel still uses p
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    if (g_scratch_free.size() >= 16) {
        cudaFree(p);
        return;
    }
    g_scratch_free.push_back({ordinal, p, bytes});
}

constexpr size_t kStatusBlockBytes = 8192;
// The reference encodes with MTLDispatchTypeConcurrent: dispatches may overlap on the GPU unless a
// memory_barrier() separates them (src/encoder.rs:837-853), and its tracked-dispatch mode inserts the barrier
// itself when the buffers of a new dispatch conflict with the current group (src/graph.rs:1494-1530).  Here a
// "concurrent group" is spread over kLanes CUDA streams: an operation whose buffers do not conflict with the
// group goes to the next lane, so that its kernels start on each SM as the previous operation's CTAs leave it
// (launch latency and the tail of the previous kernel are hidden); a conflict, or an explicit barrier, joins the
// lanes first.  Lane 0 is the encoder's own stream; commits, captures and graph launches happen there.
constexpr int kLanes = 2;
struct mlxn_encoder {
    mlxn_device *dev = nullptr;
    int ordinal = 0;  // of dev (kept by value: an idle pooled encoder may outlive the device handle)
    cudaStream_t lanes[kLanes] = {};
    cudaStream_t stream = nullptr;   // lane of the operation being encoded (lanes[cur_lane])
    int cur_lane = 0;
    bool lane_busy[kLanes] = {};     // lane has work of the current group that lane 0 has not been made to wait for
    cudaEvent_t ev_fork = nullptr, ev_join[kLanes] = {};
    cudaStream_t aux = nullptr;      // side work that nothing in the group waits for (copies of results to peer GPUs)
    cudaEvent_t ev_aux = nullptr, ev_aux_join = nullptr;
    bool aux_busy = false;
    // byte ranges of storages the current group reads / writes (views of one storage that do not overlap are independent)
    struct Span {
        const void *st;
        size_t lo, hi;
    };
    std::vector<Span> grp_reads, grp_writes;
    // inputs whose host shadow was uploaded inside the group (the whole storage is copied), with the lane the copy went
    // to: a write for the other lanes, but an operation that runs on the same lane comes after the copy anyway
    std::vector<std::pair<const void *, int>> grp_uploads;
    bool grp_open = false;           // ev_fork marks the start of the current group
    cudaEvent_t ev_start = nullptr, ev_end = nullptr;
    bool started = false, committed = false, capturing = false;
    uint64_t cap_launch0 = 0, cap_dispatch0 = 0;
    std::vector<mlxn_buffer *> retained;
    uint8_t *scratch_lane[kLanes] = {};
    size_t scratch_lane_bytes[kLanes] = {};
    std::vector<std::pair<void *, size_t>> retired;  // outgrown scratch arenas, handed back after the next wait
    std::vector<mlxn_buffer *> cap_uploads, cap_outputs;  // see mlxn_graph; filled while a capture is open
    // arenas set aside while a capture is open (the capture draws fresh ones, which the graph then owns)
    uint8_t *saved_scratch[kLanes] = {};
    size_t saved_scratch_bytes[kLanes] = {};
    std::vector<std::pair<void *, size_t>> cap_retired;   // arenas outgrown during the capture: also the graph's
    StatusBlock *sb = nullptr;
    uint32_t *status_dev = nullptr;   // == sb->dev
    // Mat-vecs of the current concurrent group that have been encoded but not launched: the reference dispatches the
    // operations of a group concurrently; here up to 8 of them (same block type, same activation-row class) leave as
    // ONE kernel whose CTAs share the work of all of them.  Launched by the first thing that ends the group.
    std::vector<QmvArgs> pend;
    int pend_type = 0, pend_lane = 0;
    uint32_t pend_mp = 0;
    bool pend_pair = false;
    bool grp_pend_only = false;       // every operation of the current group is in `pend` (none has been launched yet)
    uint32_t *status_host = nullptr;  // pinned
};

// ------------------------------------------------------------------------------------------------
// small helpers
// ------------------------------------------------------------------------------------------------
extern "C" const char *mlxn_last_error_message(void) { return g_last_error.c_str(); }
extern "C" int mlxn_status_is_transient(int status) { return status == MLXN_COMMAND_BUFFER_ERROR; }
extern "C" const char *mlxn_last_kernel_name(void) { return g_last_kernel; }

extern "C" size_t mlxn_dtype_size(int dtype) {
    switch (dtype) {
    case MLXN_F32: case MLXN_U32: case MLXN_I32: return 4;
    case MLXN_F16: case MLXN_BF16: case MLXN_U16: return 2;
    case MLXN_U8: return 1;
    default: return 0;
    }
}
extern "C" const char *mlxn_dtype_name(int dtype) {
    static const char *names[] = {"f32", "f16", "bf16", "u8", "u16", "u32", "i32"};
    return (dtype >= 0 && dtype <= MLXN_I32) ? names[dtype] : "?";
}
extern "C" uint32_t mlxn_ggml_block_values(int t) { return (t >= 0 && t <= MLXN_GGML_I16) ? ggml_qk(t) : 0; }
extern "C" uint32_t mlxn_ggml_block_bytes(int t) { return (t >= 0 && t <= MLXN_GGML_I16) ? ggml_block_bytes(t) : 0; }
static const char *ggml_name(int t) {
    static const char *names[] = {"F32", "F16", "Q4_0", "Q8_0", "Q4_K", "Q5_K", "Q6_K", "I16"};
    return (t >= 0 && t <= MLXN_GGML_I16) ? names[t] : "?";
}

extern "C" uint32_t mlxn_mm_id_routing_threshold(void) {
    static std::once_flag once;
    static uint32_t cached = MLXN_MM_ID_ROUTING_THRESHOLD;
    std::call_once(once, [] {
        const char *e = getenv("HF2Q_MM_ID_ROUTING_THRESHOLD");
        if (e && *e) {
            char *end = nullptr;
            unsigned long v = strtoul(e, &end, 10);
            if (end && *end == 0 && v <= 0xFFFFFFFFul) {
                cached = (uint32_t)v;
                if (getenv("MLX_LOG_TENSOR_PROBE"))
                    fprintf(stderr, "[mlx-native] mm_id_routing_threshold: OVERRIDE via HF2Q_MM_ID_ROUTING_THRESHOLD=%u (default %u)\n",
                            cached, MLXN_MM_ID_ROUTING_THRESHOLD);
            }
        }
    });
    return cached;
}

extern "C" int mlxn_set_option(const char *key, const char *value) {
    if (!key || !value) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: option key/value must not be null");
    if (strcmp(key, "qmv") == 0) {
        if (strcmp(value, "auto") == 0) g_opt_qmv = 3;
        else if (strcmp(value, "tc") == 0) g_opt_qmv = 2;
        else if (strcmp(value, "stream") == 0) g_opt_qmv = 1;
        else if (strcmp(value, "simple") == 0) g_opt_qmv = 0;
        else if (strcmp(value, "mma") == 0) g_opt_qmv = 4;
        else return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: qmv must be 'auto', 'mma', 'tc', 'stream' or 'simple'");
        return MLXN_OK;
    }
    if (strcmp(key, "qmv_batch") == 0) {
        if (strcmp(value, "0") != 0 && strcmp(value, "1") != 0)
            return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: qmv_batch must be '0' or '1'");
        g_opt_mv_batch = value[0] == '1';
        return MLXN_OK;
    }
    if (strcmp(key, "qmv_chain") == 0) {
        if (strcmp(value, "0") != 0 && strcmp(value, "1") != 0)
            return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: qmv_chain must be '0' or '1'");
        g_opt_mv_chain = value[0] == '1';
        return MLXN_OK;
    }
    if (strcmp(key, "qmv_mma_ctas") == 0 || strcmp(key, "qmv_mma_tpw") == 0) {
        const int v = atoi(value);
        const bool ctas = key[8] == 'c';
        if (ctas ? (v < 1 || v > 2) : !(v == 0 || v == 1 || v == 2 || v == 4))
            return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: value '%s' out of range", key, value);
        (ctas ? g_opt_mma_ctas : g_opt_mma_tpw) = v;
        return MLXN_OK;
    }
    if (strcmp(key, "qmm") == 0) {
        if (strcmp(value, "tc") == 0) g_opt_qmm = 1;
        else if (strcmp(value, "simt") == 0) g_opt_qmm = 0;
        else return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: qmm must be 'tc' or 'simt'");
        return MLXN_OK;
    }
    return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: unknown option '%s'", key);
}

extern "C" uint64_t mlxn_dispatch_count(void) { return g_dispatch.load(); }
extern "C" uint64_t mlxn_sync_count(void) { return g_sync.load(); }
extern "C" uint64_t mlxn_cmd_buf_count(void) { return g_cmd_buf.load(); }
extern "C" uint64_t mlxn_barrier_count(void) { return g_barrier.load(); }
extern "C" uint64_t mlxn_kernel_launch_count(void) { return g_launches.load(); }
extern "C" void mlxn_reset_counters(void) {
    g_dispatch = 0;
    g_sync = 0;
    g_cmd_buf = 0;
    g_barrier = 0;
    g_launches = 0;
}

// ------------------------------------------------------------------------------------------------
// device
// ------------------------------------------------------------------------------------------------
extern "C" int mlxn_device_create(int ordinal, mlxn_device **out) {
    if (!out) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: out must not be null");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(MLXN_DEVICE_NOT_FOUND, "No CUDA GPU device found — an NVIDIA B200 (sm_100a) is required");
    }
    if (ordinal < 0) {
        if (cudaGetDevice(&ordinal) != cudaSuccess) ordinal = 0;
    }
    if (ordinal >= count) return fail(MLXN_DEVICE_NOT_FOUND, "No CUDA GPU device with ordinal %d (found %d)", ordinal, count);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, ordinal) != cudaSuccess)
        return fail(MLXN_DEVICE_NOT_FOUND, "No CUDA GPU device found — cannot query device %d", ordinal);
    if (prop.major != 10)
        return fail(MLXN_DEVICE_NOT_FOUND, "Device %d (%s, sm_%d%d) is not a Blackwell sm_100 GPU; this library is built for sm_100a only",
                    ordinal, prop.name, prop.major, prop.minor);
    cudaSetDevice(ordinal);
    auto *d = new mlxn_device{ordinal, prop.multiProcessorCount, prop.name};
    if (getenv("MLX_NATIVE_LOG_INIT")) fprintf(stderr, "[mlx-native] device %d: %s, %d SMs\n", ordinal, prop.name, prop.multiProcessorCount);
    *out = d;
    return MLXN_OK;
}
extern "C" void mlxn_device_destroy(mlxn_device *dev) { delete dev; }
extern "C" const char *mlxn_device_name(const mlxn_device *dev) { return dev ? dev->name.c_str() : ""; }
extern "C" int mlxn_device_ordinal(const mlxn_device *dev) { return dev ? dev->ordinal : -1; }
extern "C" int mlxn_device_sm_count(const mlxn_device *dev) { return dev ? dev->sm_count : 0; }

// ------------------------------------------------------------------------------------------------
// buffers
// ------------------------------------------------------------------------------------------------
static mlxn_buffer *make_buffer(Storage *st, size_t offset, size_t len, int dtype, const size_t *shape, size_t rank) {
    auto *b = new mlxn_buffer();
    b->st = st;
    b->offset = offset;
    b->len = len;
    b->dtype = dtype;
    if (shape) b->shape.assign(shape, shape + rank);
    return b;
}

static int alloc_storage(mlxn_device *dev, size_t byte_len, bool zero, Storage **out) {
    cudaSetDevice(dev->ordinal);
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, byte_len);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(MLXN_BUFFER_ALLOCATION_ERROR, "Failed to allocate device buffer of %zu bytes", byte_len);
    }
    if (zero) {
        e = cudaMemset(p, 0, byte_len);
        if (e != cudaSuccess) {
            cudaFree(p);
            return cuda_fail(e, "zero-fill");
        }
    }
    auto *s = new Storage();
    s->ordinal = dev->ordinal;
    s->dptr = p;
    s->bytes = byte_len;
    *out = s;
    return MLXN_OK;
}

extern "C" int mlxn_buffer_alloc(mlxn_device *dev, size_t byte_len, int dtype, const size_t *shape, size_t rank,
                                 mlxn_buffer **out) {
    if (!dev || !out) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: device and out must not be null");
    if (byte_len == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: Buffer byte length must be > 0");
    if (mlxn_dtype_size(dtype) == 0) return fail(MLXN_UNSUPPORTED_DTYPE, "Unsupported dtype: %d", dtype);
    Storage *s = nullptr;
    int rc = alloc_storage(dev, byte_len, true, &s);
    if (rc) return rc;
    *out = make_buffer(s, 0, byte_len, dtype, shape, rank);
    return MLXN_OK;
}

extern "C" int mlxn_buffer_wrap(mlxn_device *dev, void *device_ptr, size_t byte_len, int dtype, const size_t *shape,
                                size_t rank, mlxn_buffer **out) {
    if (!dev || !out || !device_ptr) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: device, pointer and out must not be null");
    if (byte_len == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: Buffer byte length must be > 0");
    if (mlxn_dtype_size(dtype) == 0) return fail(MLXN_UNSUPPORTED_DTYPE, "Unsupported dtype: %d", dtype);
    auto *s = new Storage();
    s->ordinal = dev->ordinal;
    s->dptr = device_ptr;
    s->bytes = byte_len;
    s->owned = false;
    *out = make_buffer(s, 0, byte_len, dtype, shape, rank);
    return MLXN_OK;
}

extern "C" int mlxn_buffer_slice_view(mlxn_buffer *buf, uint64_t byte_offset, size_t n_elements, mlxn_buffer **out) {
    if (!buf || !out) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: buffer and out must not be null");
    const size_t bytes = n_elements * mlxn_dtype_size(buf->dtype);
    if (byte_offset > buf->len || bytes > buf->len - byte_offset)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: slice_view [%llu, +%zu) exceeds buffer of %zu bytes",
                    (unsigned long long)byte_offset, bytes, buf->len);
    buf->st->refs.fetch_add(1);
    size_t shp = n_elements;
    *out = make_buffer(buf->st, buf->offset + (size_t)byte_offset, bytes, buf->dtype, &shp, 1);
    return MLXN_OK;
}

extern "C" void mlxn_buffer_retain(mlxn_buffer *buf) {
    if (buf) buf->refs.fetch_add(1);
}
extern "C" void mlxn_buffer_release(mlxn_buffer *buf) {
    if (!buf) return;
    if (buf->refs.fetch_sub(1) == 1) {
        storage_release(buf->st);
        delete buf;
    }
}
extern "C" int mlxn_buffer_dtype(const mlxn_buffer *buf) { return buf->dtype; }
extern "C" size_t mlxn_buffer_rank(const mlxn_buffer *buf) { return buf->shape.size(); }
extern "C" size_t mlxn_buffer_shape(const mlxn_buffer *buf, size_t axis) { return axis < buf->shape.size() ? buf->shape[axis] : 0; }
extern "C" size_t mlxn_buffer_byte_len(const mlxn_buffer *buf) { return buf->len; }
extern "C" size_t mlxn_buffer_element_count(const mlxn_buffer *buf) { return buf->len / mlxn_dtype_size(buf->dtype); }
extern "C" uint64_t mlxn_buffer_byte_offset(const mlxn_buffer *buf) { return buf->offset; }
extern "C" void *mlxn_buffer_device_ptr(const mlxn_buffer *buf) { return buf->dev(); }

// wait for whatever touched the storage last (device work or an upload still reading the shadow)
static int encoder_flush_pending(struct mlxn_encoder *e);
static int storage_quiesce(Storage *s) {
    if (s->pend_enc) {   // a mat-vec that uses the storage is still waiting to be launched
        struct mlxn_encoder *pe = s->pend_enc;
        s->mu.unlock();   // the flush takes the storages' locks itself
        const int rc = encoder_flush_pending(pe);
        s->mu.lock();
        if (rc) return rc;
    }
    if (s->has_last) {
        CUDA_TRY(cudaStreamSynchronize(s->last_stream), "stream synchronize");
        s->has_last = false;
    }
    return MLXN_OK;
}

extern "C" int mlxn_buffer_host_map(mlxn_buffer *buf, int write, void **host_ptr) {
    if (!buf || !host_ptr) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: buffer and host_ptr must not be null");
    Storage *s = buf->st;
    std::lock_guard<std::mutex> lk(s->mu);
    cudaSetDevice(s->ordinal);
    int rc = storage_quiesce(s);
    if (rc) return rc;
    if (!s->host) {
        CUDA_TRY(cudaHostAlloc(&s->host, s->bytes, cudaHostAllocDefault), "pinned host allocation");
        s->dev_newer = true;  // HBM holds the (zero-filled or wrapped) contents
    }
    if (s->dev_newer) {
        CUDA_TRY(cudaMemcpy(s->host, s->dptr, s->bytes, cudaMemcpyDeviceToHost), "device-to-host copy");
        s->dev_newer = false;
    }
    if (write) s->host_newer = true;
    *host_ptr = static_cast<uint8_t *>(s->host) + buf->offset;
    return MLXN_OK;
}

extern "C" int mlxn_buffer_upload(mlxn_buffer *buf, const void *src, size_t byte_len, size_t dst_offset) {
    if (!buf || !src) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: buffer and src must not be null");
    if (dst_offset > buf->len || byte_len > buf->len - dst_offset)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: upload of %zu bytes at %zu exceeds buffer of %zu bytes", byte_len, dst_offset, buf->len);
    Storage *s = buf->st;
    std::lock_guard<std::mutex> lk(s->mu);
    cudaSetDevice(s->ordinal);
    int rc = storage_quiesce(s);
    if (rc) return rc;
    if (s->host_newer) {  // flush pending shadow writes first so they are not lost
        CUDA_TRY(cudaMemcpy(s->dptr, s->host, s->bytes, cudaMemcpyHostToDevice), "host-to-device copy");
        s->host_newer = false;
    }
    CUDA_TRY(cudaMemcpy(buf->dev() + dst_offset, src, byte_len, cudaMemcpyHostToDevice), "host-to-device copy");
    if (s->host) s->dev_newer = true;
    return MLXN_OK;
}

extern "C" int mlxn_buffer_download(mlxn_buffer *buf, void *dst, size_t byte_len, size_t src_offset) {
    if (!buf || !dst) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: buffer and dst must not be null");
    if (src_offset > buf->len || byte_len > buf->len - src_offset)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: download of %zu bytes at %zu exceeds buffer of %zu bytes", byte_len, src_offset, buf->len);
    Storage *s = buf->st;
    std::lock_guard<std::mutex> lk(s->mu);
    cudaSetDevice(s->ordinal);
    int rc = storage_quiesce(s);
    if (rc) return rc;
    if (s->host_newer) {
        CUDA_TRY(cudaMemcpy(s->dptr, s->host, s->bytes, cudaMemcpyHostToDevice), "host-to-device copy");
        s->host_newer = false;
    }
    CUDA_TRY(cudaMemcpy(dst, buf->dev() + src_offset, byte_len, cudaMemcpyDeviceToHost), "device-to-host copy");
    return MLXN_OK;
}

// ------------------------------------------------------------------------------------------------
// pool
// ------------------------------------------------------------------------------------------------
static size_t bucket_size(size_t n) {
    size_t b = 1;
    while (b < n) b <<= 1;
    return b;
}
extern "C" int mlxn_pool_create(mlxn_pool **out) {
    if (!out) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: out must not be null");
    *out = new mlxn_pool();
    return MLXN_OK;
}
extern "C" void mlxn_pool_clear(mlxn_pool *pool) {
    if (!pool) return;
    for (auto &kv : pool->free_list)
        for (Storage *s : kv.second) storage_release(s);
    pool->free_list.clear();
}
extern "C" void mlxn_pool_destroy(mlxn_pool *pool) {
    if (!pool) return;
    mlxn_pool_clear(pool);
    for (auto &p : pool->in_use) storage_release(p.second);
    delete pool;
}
extern "C" int mlxn_pool_alloc(mlxn_pool *pool, mlxn_device *dev, size_t byte_len, int dtype, const size_t *shape,
                               size_t rank, mlxn_buffer **out) {
    if (!pool || !dev || !out) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: pool, device and out must not be null");
    if (byte_len == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: Buffer byte length must be > 0");
    if (mlxn_dtype_size(dtype) == 0) return fail(MLXN_UNSUPPORTED_DTYPE, "Unsupported dtype: %d", dtype);
    const size_t bucket = bucket_size(byte_len);
    Storage *s = nullptr;
    auto it = pool->free_list.find(bucket);
    if (it != pool->free_list.end() && !it->second.empty()) {
        s = it->second.back();
        it->second.pop_back();
    } else {
        int rc = alloc_storage(dev, bucket, true, &s);
        if (rc) return rc;
    }
    s->refs.fetch_add(1);  // the pool's own reference (returned to the free list by reset)
    pool->in_use.emplace_back(bucket, s);
    *out = make_buffer(s, 0, bucket, dtype, shape, rank);
    return MLXN_OK;
}
extern "C" int mlxn_pool_release(mlxn_pool *pool, mlxn_buffer *buf) {
    if (!pool || !buf) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: pool and buffer must not be null");
    const size_t bucket = bucket_size(buf->st->bytes);
    buf->st->refs.fetch_add(1);
    pool->free_list[bucket].push_back(buf->st);
    mlxn_buffer_release(buf);
    return MLXN_OK;
}
extern "C" int mlxn_pool_alloc_batch(mlxn_pool *pool, mlxn_device *dev, size_t count, const size_t *byte_lens,
                                     const int *dtypes, const size_t *shapes, const size_t *ranks, mlxn_buffer **out) {
    if (!pool || !dev || !out || (count && (!byte_lens || !dtypes)))
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: pool, device, sizes, dtypes and out must not be null");
    size_t shape_at = 0;
    for (size_t i = 0; i < count; i++) {
        const size_t rank = (shapes && ranks) ? ranks[i] : 0;
        const int rc = mlxn_pool_alloc(pool, dev, byte_lens[i], dtypes[i], rank ? shapes + shape_at : nullptr, rank, &out[i]);
        shape_at += rank;
        if (rc) {
            // all or nothing: what this call handed out goes back to the free lists (the error message stays)
            const std::string msg = g_last_error;
            for (size_t j = 0; j < i; j++) {
                for (size_t u = pool->in_use.size(); u-- > 0;)
                    if (pool->in_use[u].second == out[j]->st) {
                        storage_release(pool->in_use[u].second);
                        pool->in_use.erase(pool->in_use.begin() + u);
                        break;
                    }
                mlxn_pool_release(pool, out[j]);
                out[j] = nullptr;
            }
            g_last_error = msg;
            return rc;
        }
    }
    return MLXN_OK;
}
extern "C" void mlxn_pool_reset(mlxn_pool *pool) {
    if (!pool) return;
    for (auto &p : pool->in_use) pool->free_list[p.first].push_back(p.second);
    pool->in_use.clear();
}
extern "C" int mlxn_pool_register_existing(mlxn_pool *pool, mlxn_device *dev, mlxn_buffer *buf) {
    if (!pool || !dev || !buf) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: pool, device and buffer must not be null");
    if (buf->st->ordinal != dev->ordinal)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: MlxBufferPool cannot register a buffer from a different device");
    return MLXN_OK;  // residency sets have no CUDA counterpart: device memory is always resident
}
extern "C" size_t mlxn_pool_free_count(const mlxn_pool *pool) {
    size_t n = 0;
    for (auto &kv : pool->free_list) n += kv.second.size();
    return n;
}
extern "C" size_t mlxn_pool_free_bytes(const mlxn_pool *pool) {
    size_t n = 0;
    for (auto &kv : pool->free_list) n += kv.first * kv.second.size();
    return n;
}
extern "C" size_t mlxn_pool_in_use_count(const mlxn_pool *pool) { return pool->in_use.size(); }

// ------------------------------------------------------------------------------------------------
// registry
// ------------------------------------------------------------------------------------------------
static const char *const kKernelNames[] = {
    "kernel_mul_mv_q4_0_f32", "kernel_mul_mv_q8_0_f32", "kernel_mul_mv_q6_K_f32",
    "kernel_mul_mm_q4_0_f32", "kernel_mul_mm_q8_0_f32", "kernel_mul_mm_q6_K_f32",
    "kernel_mul_mm_q4_0_tensor_f32", "kernel_mul_mm_q8_0_tensor_f32", "kernel_mul_mm_q6_K_tensor_f32",
    "kernel_mul_mm_q4_0_tensor_bf16_perm021", "kernel_mul_mm_q6_K_tensor_bf16_perm021",
    "kernel_mul_mv_id_q4_0_f32", "kernel_mul_mv_id_q8_0_f32", "kernel_mul_mv_id_q6_K_f32", "kernel_mul_mv_id_q4_0_f32_swiglu",
    "kernel_mul_mm_id_map0_ne20_1", "kernel_mul_mm_id_map0_ne20_8",
    // the bucketing kernel takes any top_k; the values upstream's audit lists as uncovered there
    // (docs/moe-q-perf-audit-2026-04-27.md:79-84) have names of the same pattern here
    "kernel_mul_mm_id_map0_ne20_2", "kernel_mul_mm_id_map0_ne20_4", "kernel_mul_mm_id_map0_ne20_5", "kernel_mul_mm_id_map0_ne20_6",
    "kernel_mul_mm_id_map0_ne20_10", "kernel_mul_mm_id_map0_ne20_16", "kernel_mul_mm_id_map0_ne20_22", "kernel_mul_mm_id_map0_ne20_n",
    "kernel_mul_mm_id_q4_0_f32", "kernel_mul_mm_id_q8_0_f32", "kernel_mul_mm_id_q6_K_f32",
    "kernel_mul_mm_id_q4_0_tensor_f32", "kernel_mul_mm_id_q8_0_tensor_f32", "kernel_mul_mm_id_q6_K_tensor_f32",
    "kernel_mul_mv_id_q5_K_f32",
    "kernel_mul_mv_q4_K_f32", "kernel_mul_mv_id_q4_K_f32", "kernel_mul_mm_id_q4_K_f32", "kernel_mul_mm_id_q4_K_tensor_f32",
    "moe_softmax_topk_f32", "moe_weighted_reduce_f32", "silu_mul_f32",
};
static bool known_kernel(const char *name) {
    for (const char *k : kKernelNames)
        if (strcmp(k, name) == 0) return true;
    return false;
}
extern "C" int mlxn_registry_create(mlxn_registry **out) {
    if (!out) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: out must not be null");
    *out = new mlxn_registry();
    return MLXN_OK;
}
extern "C" void mlxn_registry_destroy(mlxn_registry *reg) { delete reg; }
extern "C" int mlxn_registry_get_pipeline(mlxn_registry *reg, mlxn_device *dev, const char *name) {
    if (!reg || !name) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: registry and name must not be null");
    (void)dev;
    if (!known_kernel(name)) return fail(MLXN_KERNEL_NOT_FOUND, "Kernel not found: %s", name);
    reg->cached.insert(name);
    return MLXN_OK;
}
extern "C" int mlxn_registry_is_cached(const mlxn_registry *reg, const char *name) {
    return reg && name && reg->cached.count(name) ? 1 : 0;
}
extern "C" size_t mlxn_registry_cached_count(const mlxn_registry *reg) { return reg ? reg->cached.size() : 0; }
extern "C" size_t mlxn_registry_source_count(const mlxn_registry *) { return sizeof(kKernelNames) / sizeof(kKernelNames[0]); }

static int touch_kernel(mlxn_registry *reg, mlxn_device *dev, const char *name) {
    if (!reg) return MLXN_OK;
    return mlxn_registry_get_pipeline(reg, dev, name);
}

// ------------------------------------------------------------------------------------------------
// encoder
// ------------------------------------------------------------------------------------------------
// Idle encoders (streams, events, status block, scratch arenas) are kept and handed out again: upstream makes
// one encoder per command buffer, and creating streams and pinned memory for each would cost more than a mat-vec.
static std::mutex g_enc_pool_mu;
static std::vector<mlxn_encoder *> g_enc_pool;

extern "C" int mlxn_encoder_create(mlxn_device *dev, mlxn_encoder **out) {
    if (!dev || !out) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: device and out must not be null");
    cudaSetDevice(dev->ordinal);
    {
        std::lock_guard<std::mutex> lk(g_enc_pool_mu);
        for (size_t i = 0; i < g_enc_pool.size(); i++) {
            if (g_enc_pool[i]->ordinal != dev->ordinal) continue;
            mlxn_encoder *e = g_enc_pool[i];
            g_enc_pool.erase(g_enc_pool.begin() + i);
            e->dev = dev;
            g_cmd_buf.fetch_add(1);
            *out = e;
            return MLXN_OK;
        }
    }
    auto *e = new mlxn_encoder();
    e->dev = dev;
    e->ordinal = dev->ordinal;
    cudaError_t err = cudaSuccess;
    for (int l = 0; l < kLanes && err == cudaSuccess; l++) {
        err = cudaStreamCreateWithFlags(&e->lanes[l], cudaStreamNonBlocking);
        if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e->ev_join[l], cudaEventDisableTiming);
    }
    e->stream = e->lanes[0];
    if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&e->aux, cudaStreamNonBlocking);
    if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e->ev_aux, cudaEventDisableTiming);
    if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e->ev_aux_join, cudaEventDisableTiming);
    if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e->ev_fork, cudaEventDisableTiming);
    if (err == cudaSuccess) err = cudaEventCreate(&e->ev_start);
    if (err == cudaSuccess) err = cudaEventCreate(&e->ev_end);
    // status word, then (256 bytes in) the zero-initialised flag words the tensor-core mat-vec's CTAs hand work over with
    if (err == cudaSuccess) err = cudaMalloc((void **)&e->status_dev, kStatusBlockBytes);
    if (err == cudaSuccess) err = cudaMemset(e->status_dev, 0, kStatusBlockBytes);
    if (err == cudaSuccess) {
        e->sb = new StatusBlock();
        e->sb->ordinal = dev->ordinal;
        e->sb->dev = e->status_dev;
    }
    if (err == cudaSuccess) err = cudaHostAlloc((void **)&e->status_host, 4, cudaHostAllocDefault);
    if (err != cudaSuccess) {
        for (int l = 0; l < kLanes; l++) {
            if (e->lanes[l]) cudaStreamDestroy(e->lanes[l]);
            if (e->ev_join[l]) cudaEventDestroy(e->ev_join[l]);
        }
        if (e->ev_fork) cudaEventDestroy(e->ev_fork);
        if (e->aux) cudaStreamDestroy(e->aux);
        if (e->ev_aux) cudaEventDestroy(e->ev_aux);
        if (e->ev_aux_join) cudaEventDestroy(e->ev_aux_join);
        if (e->ev_start) cudaEventDestroy(e->ev_start);
        if (e->ev_end) cudaEventDestroy(e->ev_end);
        if (e->sb) status_block_release(e->sb);
        else if (e->status_dev) cudaFree(e->status_dev);
        delete e;
        return cuda_fail(err, "encoder creation");
    }
    *e->status_host = 0;
    g_cmd_buf.fetch_add(1);
    *out = e;
    return MLXN_OK;
}

static void encoder_release_retained(mlxn_encoder *e) {
    // called once the stream is idle: storages whose last user was this stream no longer need a wait
    for (mlxn_buffer *b : e->retained) {
        {
            std::lock_guard<std::mutex> lk(b->st->mu);
            bool mine = false;
            for (int l = 0; l < kLanes; l++) mine = mine || b->st->last_stream == e->lanes[l];
            if (b->st->has_last && mine) b->st->has_last = false;
        }
        mlxn_buffer_release(b);
    }
    e->retained.clear();
    for (auto &pr : e->retired) scratch_give(e->ordinal, pr.first, pr.second);
    e->retired.clear();
}

extern "C" void mlxn_encoder_destroy(mlxn_encoder *enc) {
    if (!enc) return;
    cudaSetDevice(enc->ordinal);
    (void)encoder_flush_pending(enc);
    cudaError_t serr = cudaStreamSynchronize(enc->aux);
    for (int l = 0; l < kLanes; l++) {
        cudaError_t e1 = cudaStreamSynchronize(enc->lanes[l]);
        if (e1 != cudaSuccess) serr = e1;
    }
    encoder_release_retained(enc);
    if (serr == cudaSuccess && !enc->capturing) {
        // clean and idle: keep it for the next mlxn_encoder_create on this device
        enc->started = enc->committed = false;
        enc->cur_lane = 0;
        enc->stream = enc->lanes[0];
        for (int l = 0; l < kLanes; l++) enc->lane_busy[l] = false;
        enc->aux_busy = false;
        enc->grp_reads.clear();
        enc->grp_writes.clear();
        enc->grp_uploads.clear();
        enc->grp_open = false;
        if (*enc->status_host != 0) {
            *enc->status_host = 0;
            cudaMemset(enc->status_dev, 0, kStatusBlockBytes);
        }
        std::lock_guard<std::mutex> lk(g_enc_pool_mu);
        if (g_enc_pool.size() < 8) {
            g_enc_pool.push_back(enc);
            return;
        }
    }
    (void)cudaGetLastError();
    for (int l = 0; l < kLanes; l++) {
        if (enc->scratch_lane[l]) scratch_give(enc->ordinal, enc->scratch_lane[l], enc->scratch_lane_bytes[l]);
        if (enc->saved_scratch[l]) scratch_give(enc->ordinal, enc->saved_scratch[l], enc->saved_scratch_bytes[l]);
    }
    for (auto &pr : enc->cap_retired) scratch_give(enc->ordinal, pr.first, pr.second);
    status_block_release(enc->sb);
    cudaFreeHost(enc->status_host);
    cudaEventDestroy(enc->ev_start);
    cudaEventDestroy(enc->ev_end);
    cudaEventDestroy(enc->ev_fork);
    cudaEventDestroy(enc->ev_aux);
    cudaEventDestroy(enc->ev_aux_join);
    cudaStreamDestroy(enc->aux);
    for (int l = 0; l < kLanes; l++) {
        cudaEventDestroy(enc->ev_join[l]);
        cudaStreamDestroy(enc->lanes[l]);
    }
    delete enc;
}

static int encoder_join_lanes(mlxn_encoder *e);
static int encoder_flush_pending(mlxn_encoder *e);
// Lane 0, after it has been made to wait for the other lane: work the caller enqueues on the returned stream runs
// behind everything encoded so far.
extern "C" void *mlxn_encoder_stream(mlxn_encoder *enc) {
    if (!enc) return nullptr;
    cudaSetDevice(enc->ordinal);
    if (!enc->capturing && encoder_join_lanes(enc) != MLXN_OK) return nullptr;
    return (void *)enc->lanes[0];
}

// Ends the current concurrent group: lane 0 waits for every other lane that has work of the group; the next
// operation starts a new group on lane 0.
static uint32_t mv_row_class(uint32_t m) { return m <= 1 ? 1u : m <= 2 ? 2u : m <= 4 ? 4u : 8u; }
static int encoder_scratch_on(mlxn_encoder *e, int lane, size_t bytes, uint8_t **out);
static int encoder_flush_pending(mlxn_encoder *e) {
    if (e->pend.empty()) return MLXN_OK;
    cudaSetDevice(e->ordinal);
    cudaStream_t st = e->lanes[e->pend_lane];
    cudaError_t err = cudaSuccess;
    int launches = 1, rc = MLXN_OK;
    // A mat-vec that ended up alone (the next operation depended on it, or nothing followed) gains nothing from the
    // batched kernel's shared work list; with "auto" it takes the kernel that is fastest for a lone call of its kind.
    e->grp_pend_only = false;   // (what is launched here stays part of the group until the lanes are joined)
    // barrier words of a launch whose mat-vecs depend on one another: one set per lane (launches of a lane are ordered)
    for (QmvArgs &a : e->pend) a.grid_bar = e->status_dev + 1024 + 32 * e->pend_lane;
    const QmvArgs &a0 = e->pend[0];
    // (measured: one or two activation rows stay with this kernel, except one Q6_K row on a small matrix, where the
    //  streaming kernel's short start wins; more rows take the tensor-memory kernel, whose time does not grow with m)
    const bool q6_one_row_small = e->pend_type == GT_Q6_K && a0.m == 1 && (uint64_t)a0.n * a0.k < (1ull << 23);
    const bool lone_other = e->pend.size() == 1 && opt_qmv() == 3 && a0.n_peer == 0 && !a0.ids && e->pend_type != GT_Q4_K &&
                            (q6_one_row_small || a0.m > 2);
    if (lone_other) {
        if (!q6_one_row_small && qmv_tc_supported(e->pend_type, a0)) {
            uint8_t *scratch = nullptr;
            if ((rc = encoder_scratch_on(e, e->pend_lane, qmv_tc_scratch_bytes(a0), &scratch)) == MLXN_OK) {
                launches = 0;
                err = launch_qmv_tc(e->pend_type, a0, scratch, e->status_dev + 64, e->dev->sm_count, st, nullptr, nullptr, &launches);
                g_last_kernel = "qmv_tc";
            }
        } else {
            err = launch_qmv(e->pend_type, a0, true, e->dev->sm_count, st, &g_last_kernel);
        }
    } else {
        err = launch_qmv_mma(e->pend_type, e->pend.data(), (int)e->pend.size(), e->dev->sm_count, g_opt_mma_ctas.load(),
                             g_opt_mma_tpw.load(), st);
        if (err == cudaErrorCooperativeLaunchTooLarge) {
            // the device cannot hold the whole grid at once (it is shared): the chained mat-vecs leave one by one
            (void)cudaGetLastError();
            err = cudaSuccess;
            launches = 0;
            for (QmvArgs &a : e->pend) {
                a.after_earlier = 0;
                if (err == cudaSuccess)
                    err = launch_qmv_mma(e->pend_type, &a, 1, e->dev->sm_count, g_opt_mma_ctas.load(), g_opt_mma_tpw.load(), st);
                launches++;
            }
        }
    }
    e->pend.clear();
    for (mlxn_buffer *b : e->retained) {
        std::lock_guard<std::mutex> lk(b->st->mu);
        if (b->st->pend_enc == e) b->st->pend_enc = nullptr;
    }
    if (rc) return rc;
    if (err != cudaSuccess) return cuda_fail(err, "mat-vec launch");
    g_launches.fetch_add((uint64_t)launches);
    return MLXN_OK;
}

static int encoder_join_lanes(mlxn_encoder *e) {
    {
        const int frc = encoder_flush_pending(e);
        if (frc) return frc;
    }
    for (int l = 1; l < kLanes; l++) {
        if (!e->lane_busy[l]) continue;
        CUDA_TRY(cudaEventRecord(e->ev_join[l], e->lanes[l]), "event record");
        CUDA_TRY(cudaStreamWaitEvent(e->lanes[0], e->ev_join[l], 0), "stream wait");
        e->lane_busy[l] = false;
    }
    if (e->aux_busy) {
        CUDA_TRY(cudaEventRecord(e->ev_aux_join, e->aux), "event record");
        CUDA_TRY(cudaStreamWaitEvent(e->lanes[0], e->ev_aux_join, 0), "stream wait");
        e->aux_busy = false;
    }
    e->grp_reads.clear();
    e->grp_writes.clear();
    e->grp_uploads.clear();
    e->grp_open = false;
    e->cur_lane = 0;
    e->stream = e->lanes[0];
    return MLXN_OK;
}

extern "C" int mlxn_encoder_memory_barrier(mlxn_encoder *enc) {
    if (!enc) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: encoder must not be null");
    g_barrier.fetch_add(1);
    cudaSetDevice(enc->ordinal);
    return encoder_join_lanes(enc);
}

static int encoder_begin_work(mlxn_encoder *e) {
    cudaSetDevice(e->ordinal);
    if (!e->started && !e->capturing) {
        CUDA_TRY(cudaEventRecord(e->ev_start, e->lanes[0]), "event record");
        e->started = true;
        e->committed = false;
    }
    return MLXN_OK;
}

extern "C" int mlxn_encoder_commit(mlxn_encoder *enc) {
    if (!enc) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: encoder must not be null");
    if (enc->capturing) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: commit while a capture is open");
    cudaSetDevice(enc->ordinal);
    int jrc = encoder_join_lanes(enc);
    if (jrc) return jrc;
    if (!enc->started) {
        CUDA_TRY(cudaEventRecord(enc->ev_start, enc->lanes[0]), "event record");
        enc->started = true;
    }
    // Results the host has a view of are brought back as part of the command buffer (upstream's buffers are
    // unified memory: after commit_and_wait the CPU simply sees them); large ones are fetched on demand instead.
    for (mlxn_buffer *b : enc->retained) {
        Storage *st = b->st;
        std::lock_guard<std::mutex> lk(st->mu);
        if (st->host && st->dev_newer && st->bytes <= (size_t)(4u << 20)) {
            CUDA_TRY(cudaMemcpyAsync(st->host, st->dptr, st->bytes, cudaMemcpyDeviceToHost, enc->lanes[0]), "device-to-host copy");
            st->dev_newer = false;
            st->last_stream = enc->lanes[0];
            st->has_last = true;
        }
    }
    CUDA_TRY(cudaMemcpyAsync(enc->status_host, enc->status_dev, 4, cudaMemcpyDeviceToHost, enc->lanes[0]), "status copy");
    CUDA_TRY(cudaEventRecord(enc->ev_end, enc->lanes[0]), "event record");
    enc->committed = true;
    return MLXN_OK;
}

static const char *status_text(uint32_t s) {
    switch (s) {
    case ST_WAIT_FULL_TIMEOUT: return "a kernel gave up waiting for data to arrive in shared memory";
    case ST_WAIT_EMPTY_TIMEOUT: return "a kernel gave up waiting for a pipeline stage to be released";
    case ST_WAIT_MMA_TIMEOUT: return "a kernel gave up waiting for the tensor cores";
    case ST_WAIT_TMEM_TIMEOUT: return "a kernel gave up waiting for tensor memory";
    case ST_WAIT_PEER_TIMEOUT: return "a kernel gave up waiting for another rank at a barrier";
    case ST_WAIT_GRID_TIMEOUT: return "a kernel gave up waiting for its other blocks at a barrier";
    default: return "a kernel reported an error";
    }
}

extern "C" int mlxn_encoder_wait_until_completed(mlxn_encoder *enc) {
    if (!enc) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: encoder must not be null");
    cudaSetDevice(enc->ordinal);
    g_sync.fetch_add(1);
    cudaError_t e = cudaSuccess;
    if (enc->committed) {
        e = cudaEventSynchronize(enc->ev_end);
    } else {
        (void)encoder_flush_pending(enc);
        e = cudaStreamSynchronize(enc->aux);
        for (int l = 0; l < kLanes && e == cudaSuccess; l++) e = cudaStreamSynchronize(enc->lanes[l]);
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    encoder_release_retained(enc);
    enc->started = false;
    if (e != cudaSuccess) return cuda_fail(e, "GPU execution");
    if (enc->committed && *enc->status_host != 0) {
        const uint32_t s = *enc->status_host;
        *enc->status_host = 0;
        cudaMemsetAsync(enc->status_dev, 0, kStatusBlockBytes, enc->lanes[0]);
        return fail(MLXN_COMMAND_BUFFER_ERROR, "Command buffer error: %s (status %u)", status_text(s), s);
    }
    return MLXN_OK;
}

extern "C" int mlxn_encoder_commit_and_wait(mlxn_encoder *enc) {
    int rc = mlxn_encoder_commit(enc);
    if (rc) return rc;
    return mlxn_encoder_wait_until_completed(enc);
}

extern "C" int mlxn_encoder_commit_wait_with_gpu_time(mlxn_encoder *enc, double *gpu_seconds) {
    int rc = mlxn_encoder_commit(enc);
    if (rc) return rc;
    rc = mlxn_encoder_wait_until_completed(enc);
    if (rc) return rc;
    float ms = 0.0f;
    CUDA_TRY(cudaEventElapsedTime(&ms, enc->ev_start, enc->ev_end), "event elapsed time");
    if (gpu_seconds) *gpu_seconds = (double)ms * 1e-3;
    return MLXN_OK;
}

// Per-command-buffer profile (upstream kernel_profile, enabled by MLX_PROFILE_CB=1): device time per label.
static std::mutex g_prof_mu;
static std::map<std::string, std::pair<uint64_t, uint64_t>> g_prof;   // label -> (command buffers, nanoseconds)
static bool profile_cb_enabled() {
    static const bool on = [] { const char *e = getenv("MLX_PROFILE_CB"); return e && *e && strcmp(e, "0") != 0; }();
    return on;
}
extern "C" int mlxn_encoder_commit_and_wait_labeled(mlxn_encoder *enc, const char *label) {
    if (!enc) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: encoder must not be null");
    const char *name = label ? label : "";
    nvtxRangePushA(name);   // visible to a profiler that is attached; a no-op otherwise
    int rc;
    if (profile_cb_enabled()) {
        double s = 0.0;
        rc = mlxn_encoder_commit_wait_with_gpu_time(enc, &s);
        if (rc == MLXN_OK) {
            const uint64_t ns = (uint64_t)(s * 1e9);
            {
                std::lock_guard<std::mutex> lk(g_prof_mu);
                auto &e = g_prof[name];
                e.first++;
                e.second += ns;
            }
            fprintf(stderr, "[mlx-native] cb %s: %.3f us\n", name, s * 1e6);
        }
    } else {
        rc = mlxn_encoder_commit_and_wait(enc);
    }
    nvtxRangePop();
    return rc;
}
// Profile mode turns the asynchronous commit into a synchronous one to get the device time, as upstream does.
extern "C" int mlxn_encoder_commit_labeled(mlxn_encoder *enc, const char *label) {
    if (profile_cb_enabled()) return mlxn_encoder_commit_and_wait_labeled(enc, label);
    nvtxRangePushA(label ? label : "");
    const int rc = mlxn_encoder_commit(enc);
    nvtxRangePop();
    return rc;
}
extern "C" int mlxn_profile_cb_get(const char *label, uint64_t *count, uint64_t *nanoseconds) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    auto it = g_prof.find(label ? label : "");
    if (count) *count = it == g_prof.end() ? 0 : it->second.first;
    if (nanoseconds) *nanoseconds = it == g_prof.end() ? 0 : it->second.second;
    return MLXN_OK;
}
extern "C" void mlxn_profile_cb_reset(void) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    g_prof.clear();
}

extern "C" int mlxn_encoder_begin_capture(mlxn_encoder *enc) {
    if (!enc) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: encoder must not be null");
    if (enc->capturing) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: a capture is already open");
    cudaSetDevice(enc->ordinal);
    int jrc = encoder_join_lanes(enc);  // the capture starts from lane 0 alone; other lanes fork from inside it
    if (jrc) return jrc;
    CUDA_TRY(cudaStreamBeginCapture(enc->lanes[0], cudaStreamCaptureModeRelaxed), "begin capture");
    enc->capturing = true;
    // the recorded kernels must not address arenas that later eager work may outgrow and hand back: the capture
    // draws arenas of its own, which the graph keeps
    for (int l = 0; l < kLanes; l++) {
        enc->saved_scratch[l] = enc->scratch_lane[l];
        enc->saved_scratch_bytes[l] = enc->scratch_lane_bytes[l];
        enc->scratch_lane[l] = nullptr;
        enc->scratch_lane_bytes[l] = 0;
    }
    enc->cap_launch0 = g_launches.load();
    enc->cap_dispatch0 = g_dispatch.load();
    return MLXN_OK;
}
extern "C" int mlxn_encoder_end_capture(mlxn_encoder *enc, mlxn_graph **out) {
    if (!enc || !out) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: encoder and out must not be null");
    if (!enc->capturing) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: no capture is open");
    cudaSetDevice(enc->ordinal);
    int jrc = encoder_join_lanes(enc);  // every forked lane rejoins lane 0 before the capture ends
    enc->capturing = false;
    auto *g = new mlxn_graph();
    g->ordinal = enc->ordinal;
    for (int l = 0; l < kLanes; l++) {
        if (enc->scratch_lane[l]) g->scratch.push_back({enc->scratch_lane[l], enc->scratch_lane_bytes[l]});
        enc->scratch_lane[l] = enc->saved_scratch[l];
        enc->scratch_lane_bytes[l] = enc->saved_scratch_bytes[l];
        enc->saved_scratch[l] = nullptr;
        enc->saved_scratch_bytes[l] = 0;
    }
    for (auto &pr : enc->cap_retired) g->scratch.push_back(pr);
    enc->cap_retired.clear();
    g->sb = enc->sb;
    g->sb->refs.fetch_add(1);
    // Results the host already has a view of are fetched back by the graph itself (copy nodes behind all the work),
    // so that a replay costs no device-to-host call per result at commit time.
    if (!jrc) {
        for (mlxn_buffer *b : enc->cap_outputs) {
            Storage *st = b->st;
            std::lock_guard<std::mutex> lk(st->mu);
            bool fetch = st->host && st->bytes <= (size_t)(4u << 20);
            if (fetch) {
                for (size_t i = 0; i < g->fetched.size(); i++)
                    if (enc->cap_outputs[i]->st == st && g->fetched[i]) fetch = false;   // one copy per storage
            }
            if (fetch && cudaMemcpyAsync(st->host, st->dptr, st->bytes, cudaMemcpyDeviceToHost, enc->lanes[0]) != cudaSuccess) {
                (void)cudaGetLastError();
                fetch = false;
            }
            g->fetched.push_back(fetch);
        }
    }
    g->fetched.resize(enc->cap_outputs.size(), false);
    g->covered.assign(enc->cap_outputs.size(), false);
    for (size_t i = 0; i < enc->cap_outputs.size(); i++)
        for (size_t j = 0; j < enc->cap_outputs.size() && !g->covered[i]; j++)
            if (g->fetched[j] && enc->cap_outputs[j]->st == enc->cap_outputs[i]->st) g->covered[i] = true;
    cudaError_t e = cudaStreamEndCapture(enc->lanes[0], &g->graph);
    if (jrc && e == cudaSuccess) e = cudaErrorUnknown;
    if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
    if (e != cudaSuccess) {
        if (g->graph) cudaGraphDestroy(g->graph);
        for (auto &pr : g->scratch) scratch_give(g->ordinal, pr.first, pr.second);   // nothing was launched
        status_block_release(g->sb);
        delete g;
        for (mlxn_buffer *b : enc->cap_uploads) mlxn_buffer_release(b);
        for (mlxn_buffer *b : enc->cap_outputs) mlxn_buffer_release(b);
        enc->cap_uploads.clear();
        enc->cap_outputs.clear();
        return cuda_fail(e, "end capture");
    }
    g->uploads.swap(enc->cap_uploads);
    g->outputs.swap(enc->cap_outputs);
    g->launches = g_launches.load() - enc->cap_launch0;
    g->dispatches = g_dispatch.load() - enc->cap_dispatch0;
    // recording is not running: take the recorded work back out of the global counters
    g_launches.fetch_sub(g->launches);
    g_dispatch.fetch_sub(g->dispatches);
    *out = g;
    return MLXN_OK;
}
extern "C" int mlxn_graph_launch(mlxn_graph *graph, mlxn_encoder *enc) {
    if (!graph || !enc) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: graph and encoder must not be null");
    if (enc->capturing) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: graph launch while a capture is open");
    // the recorded kernels report through the status block of the encoder that recorded them
    if (graph->sb != enc->sb)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: a captured graph replays on the encoder that recorded it");
    int rc = encoder_begin_work(enc);
    if (rc) return rc;
    if ((rc = encoder_join_lanes(enc))) return rc;  // the graph's buffers are unknown here: it is its own group
    CUDA_TRY(cudaGraphLaunch(graph->exec, enc->lanes[0]), "graph launch");
    for (mlxn_buffer *b : graph->uploads) {
        {
            std::lock_guard<std::mutex> lk(b->st->mu);
            // the replay's copy node reads the pinned shadow when lane 0 gets there: a host write has to wait for it
            b->st->host_newer = false;
            b->st->last_stream = enc->lanes[0];
            b->st->has_last = true;
        }
        b->refs.fetch_add(1);
        enc->retained.push_back(b);
    }
    for (size_t oi = 0; oi < graph->outputs.size(); oi++) {
        mlxn_buffer *b = graph->outputs[oi];
        {
            std::lock_guard<std::mutex> lk(b->st->mu);
            // (a storage the graph fetches itself is current on the host once lane 0 has run the replay)
            const bool fetched_by_graph = graph->covered[oi];
            if (b->st->host) b->st->dev_newer = !fetched_by_graph;
            b->st->last_stream = enc->lanes[0];
            b->st->has_last = true;
        }
        b->refs.fetch_add(1);
        enc->retained.push_back(b);  // kept alive, and fetched back at commit like any other result
    }
    g_launches.fetch_add(graph->launches);
    g_dispatch.fetch_add(graph->dispatches);
    return MLXN_OK;
}
extern "C" void mlxn_graph_destroy(mlxn_graph *graph) {
    if (!graph) return;
    if (!graph->scratch.empty()) {
        // a replay may still be running on some stream: wait before the arenas go back
        int prev = 0;
        cudaGetDevice(&prev);
        cudaSetDevice(graph->ordinal);
        cudaDeviceSynchronize();
        for (auto &pr : graph->scratch) scratch_give(graph->ordinal, pr.first, pr.second);
        cudaSetDevice(prev);
    }
    status_block_release(graph->sb);
    for (mlxn_buffer *b : graph->uploads) mlxn_buffer_release(b);
    for (mlxn_buffer *b : graph->outputs) mlxn_buffer_release(b);
    if (graph->exec) cudaGraphExecDestroy(graph->exec);
    if (graph->graph) cudaGraphDestroy(graph->graph);
    delete graph;
}

// Grows the encoder's scratch arena (kept for its lifetime; an outgrown arena is freed at the next wait).
static int encoder_scratch(mlxn_encoder *e, size_t bytes, uint8_t **out) { return encoder_scratch_on(e, e->cur_lane, bytes, out); }
static int encoder_scratch_on(mlxn_encoder *e, int lane, size_t bytes, uint8_t **out) {
    uint8_t *&scratch = e->scratch_lane[lane];  // operations on different lanes may run at the same time
    size_t &scratch_bytes = e->scratch_lane_bytes[lane];
    if (bytes > scratch_bytes) {
        size_t want = bucket_size(bytes < (1u << 20) ? (1u << 20) : bytes);
        void *p = scratch_take(e->ordinal, want, &want);
        if (!p) {
            cudaError_t err = cudaMalloc(&p, want);
            if (err != cudaSuccess) {
                cudaGetLastError();
                return fail(MLXN_BUFFER_ALLOCATION_ERROR, "Failed to allocate device buffer of %zu bytes", want);
            }
        }
        if (scratch) (e->capturing ? e->cap_retired : e->retired).push_back({scratch, scratch_bytes});
        scratch = static_cast<uint8_t *>(p);
        scratch_bytes = want;
    }
    *out = scratch;
    return MLXN_OK;
}

// Binds a buffer to the encoder: uploads a newer host shadow on the encoder's stream, records the
// stream as the storage's last user, and keeps the buffer alive until the encoder's next wait.
static int bind(mlxn_encoder *e, mlxn_buffer *b, bool is_output) {
    Storage *s = b->st;
    std::lock_guard<std::mutex> lk(s->mu);
    if (s->ordinal != e->ordinal)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: buffer lives on device %d, encoder on device %d", s->ordinal, e->ordinal);
    bool own_lane = false;  // lanes of one encoder are ordered by its group logic, not by host-side waits
    for (int l = 0; l < kLanes; l++) own_lane = own_lane || s->last_stream == e->lanes[l];
    if (s->has_last && !own_lane) {
        CUDA_TRY(cudaStreamSynchronize(s->last_stream), "stream synchronize");
    }
    if (s->host_newer) {
        CUDA_TRY(cudaMemcpyAsync(s->dptr, s->host, s->bytes, cudaMemcpyHostToDevice, e->stream), "host-to-device copy");
        s->host_newer = false;
        if (e->capturing) {
            b->refs.fetch_add(1);
            e->cap_uploads.push_back(b);
        }
    }
    if (is_output && e->capturing) {
        b->refs.fetch_add(1);
        e->cap_outputs.push_back(b);
    }
    if (is_output && s->host) s->dev_newer = true;
    if (is_output) s->kernel_written = true;
    s->last_stream = e->stream;
    s->has_last = true;
    b->refs.fetch_add(1);
    e->retained.push_back(b);
    return MLXN_OK;
}

// Places an operation: decides whether it may join the current concurrent group (none of its buffers conflicts
// with what the group reads and writes; an input whose host shadow still has to be uploaded counts as written),
// picks its lane, and binds its buffers there.
struct OpBuf {
    mlxn_buffer *b;
    bool out;
};
// `lane`: the lane the operation would run on.
static bool op_conflicts(mlxn_encoder *e, std::initializer_list<OpBuf> bufs, int lane) {
    bool conflict = false;
    for (const OpBuf &ob : bufs) {
        if (!ob.b) continue;
        Storage *st = ob.b->st;
        bool uploads = false;
        {
            std::lock_guard<std::mutex> lk(st->mu);
            uploads = st->host_newer;
        }
        // (an upload copies the whole storage: it counts as a write of all of it)
        const size_t lo = uploads ? 0 : ob.b->offset, hi = uploads ? st->bytes : ob.b->offset + ob.b->len;
        auto has = [&](const std::vector<mlxn_encoder::Span> &v) {
            for (const auto &q : v)
                if (q.st == st && q.lo < hi && lo < q.hi) return true;
            return false;
        };
        const bool writes = ob.out || uploads;
        if (writes) conflict = conflict || has(e->grp_reads) || has(e->grp_writes);
        else conflict = conflict || has(e->grp_writes);
        for (const auto &u : e->grp_uploads)
            if (u.first == st && (writes || u.second != lane)) conflict = true;
    }
    return conflict;
}
// The lane an operation that does not conflict with the group gets: a mat-vec that leaves with the pending batch shares
// that batch's lane; everything else alternates.
static int op_lane(const mlxn_encoder *e, bool joins_batch) {
    const bool first = e->grp_reads.empty() && e->grp_writes.empty();
    return first ? 0 : (joins_batch && !e->pend.empty()) ? e->pend_lane : (e->cur_lane + 1) % kLanes;
}
// `ordered_in_batch`: the operation joins the pending batch as a dependent mat-vec (the batch's kernel orders it after
// the ones it conflicts with), so a conflict does not end the group.
static int op_begin(mlxn_encoder *e, std::initializer_list<OpBuf> bufs, bool joins_batch = false, bool ordered_in_batch = false) {
    int rc = encoder_begin_work(e);
    if (rc) return rc;
    const bool conflict = op_conflicts(e, bufs, op_lane(e, joins_batch));
    if (conflict && !ordered_in_batch && (rc = encoder_join_lanes(e))) return rc;
    const bool first = e->grp_reads.empty() && e->grp_writes.empty();
    e->grp_pend_only = joins_batch && (first || e->grp_pend_only);
    const int lane = op_lane(e, joins_batch);
    if (!e->grp_open) {
        CUDA_TRY(cudaEventRecord(e->ev_fork, e->lanes[0]), "event record");  // everything before this group
        e->grp_open = true;
    }
    if (lane != 0 && !e->lane_busy[lane]) {
        CUDA_TRY(cudaStreamWaitEvent(e->lanes[lane], e->ev_fork, 0), "stream wait");
        e->lane_busy[lane] = true;
    }
    e->cur_lane = lane;
    e->stream = e->lanes[lane];
    for (const OpBuf &ob : bufs) {
        if (!ob.b) continue;
        Storage *st = ob.b->st;
        bool uploads = false;
        {
            std::lock_guard<std::mutex> lk(st->mu);
            uploads = st->host_newer;
        }
        const mlxn_encoder::Span span{st, ob.b->offset, ob.b->offset + ob.b->len};
        if (ob.out) e->grp_writes.push_back(span);
        else e->grp_reads.push_back(span);
        if (uploads) e->grp_uploads.push_back({st, lane});   // its host shadow is copied in by bind() below, on this lane
        if ((rc = bind(e, ob.b, ob.out))) return rc;
    }
    return MLXN_OK;
}

// ------------------------------------------------------------------------------------------------
// the give-up path of the kernels' bounded waits, made reachable for a test
// ------------------------------------------------------------------------------------------------
// One CTA waits, with the given limit, on a shared-memory barrier that nothing ever arrives at.  The wait runs out,
// the kernel records ST_WAIT_FULL_TIMEOUT in the encoder's status word and returns normally: the context stays
// usable and the next commit reports CommandBufferError, exactly as a production kernel's expired wait would.
__global__ void wait_probe_kernel(uint32_t *status, uint64_t limit_ns) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ volatile uint32_t abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mlxn::mbar_init(&bar, 1);
        mlxn::mbar_init_fence();
    }
    __syncthreads();
    (void)mlxn::mbar_wait(&bar, 0u, &abort_flag, status, mlxn::ST_WAIT_FULL_TIMEOUT, 0u, limit_ns);
}

extern "C" int mlxn_debug_wait_probe(mlxn_encoder *enc, uint32_t limit_us) {
    if (!enc) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: encoder must not be null");
    if (limit_us == 0 || limit_us > 100000)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: wait probe limit (%u us) must be in 1..100000", limit_us);
    int rc = encoder_begin_work(enc);
    if (rc) return rc;
    if ((rc = encoder_join_lanes(enc))) return rc;
    wait_probe_kernel<<<1, 32, 0, enc->lanes[0]>>>(enc->status_dev, (uint64_t)limit_us * 1000ull);
    CUDA_TRY(cudaGetLastError(), "wait probe launch");
    g_launches.fetch_add(1);
    return MLXN_OK;
}

// ------------------------------------------------------------------------------------------------
// cross-rank barrier over peer memory (one process per GPU; no counterpart in the reference)
// ------------------------------------------------------------------------------------------------
// Every rank owns a flag array uint32[world] that the other ranks can store to (symmetric / IPC memory).  Thread r of
// the one-CTA kernel publishes this rank's epoch in rank r's array (slot = this rank) behind a system-wide fence, so
// that everything this GPU stored to its peers before the barrier is visible to whoever sees the flag, and then waits
// until rank r's epoch has arrived in its own array.  The wait is bounded: when it runs out the kernel records
// ST_WAIT_PEER_TIMEOUT and returns, and the next commit reports CommandBufferError (a rank that never arrives must not
// hang the others' GPUs).  Plain loads and stores only: no multicast, so a rank that dies leaves nothing bound.
struct PeerFlags {
    uint32_t *p[32];
};
__global__ void peer_barrier_kernel(uint32_t rank, uint32_t world, const PeerFlags flags, uint32_t epoch, uint64_t limit_ns,
                                    uint32_t *status) {
    const uint32_t r = threadIdx.x;
    if (r >= world) return;
    __threadfence_system();
    volatile uint32_t *theirs = flags.p[r] + rank;
    *theirs = epoch;
    __threadfence_system();
    volatile uint32_t *mine = flags.p[rank] + r;
    const uint64_t t0 = mlxn::global_timer_ns();
    for (uint32_t polls = 0;; polls++) {
        // epochs only grow; a difference in the upper half of the range means "not yet" (wrap-around safe)
        if ((int32_t)(*mine - epoch) >= 0) break;
        if ((polls & 63u) == 63u && mlxn::global_timer_ns() - t0 > limit_ns) {
            if (status) atomicCAS(status, 0u, (uint32_t)mlxn::ST_WAIT_PEER_TIMEOUT);
            break;
        }
        __nanosleep(100);
    }
    __threadfence_system();
}

// `flag_ptrs`: host array of `world` device addresses, entry r = rank r's flag array as mapped into this process.
extern "C" int mlxn_peer_barrier(mlxn_encoder *enc, uint32_t rank, uint32_t world, void *const *flag_ptrs, uint32_t epoch,
                                 uint32_t limit_us) {
    if (!enc || !flag_ptrs) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: encoder and flag pointers must not be null");
    if (world == 0 || world > 32 || rank >= world)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: peer barrier: rank %u of %u ranks (1..32)", rank, world);
    if (limit_us == 0 || limit_us > 10000000)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: peer barrier: wait limit (%u us) must be in 1..10000000", limit_us);
    for (uint32_t r = 0; r < world; r++)
        if (!flag_ptrs[r] || ((uintptr_t)flag_ptrs[r] & 3u))
            return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: peer barrier: flag array %u is null or misaligned", r);
    int rc = encoder_begin_work(enc);
    if (rc) return rc;
    if ((rc = encoder_join_lanes(enc))) return rc;   // everything encoded so far is ahead of the barrier
    PeerFlags table{};
    for (uint32_t r = 0; r < world; r++) table.p[r] = static_cast<uint32_t *>(flag_ptrs[r]);
    peer_barrier_kernel<<<1, 32, 0, enc->lanes[0]>>>(rank, world, table, epoch, (uint64_t)limit_us * 1000ull, enc->status_dev);
    CUDA_TRY(cudaGetLastError(), "peer barrier launch");
    g_launches.fetch_add(1);
    g_barrier.fetch_add(1);
    return MLXN_OK;
}

// ------------------------------------------------------------------------------------------------
// quantized_matmul_ggml
// ------------------------------------------------------------------------------------------------
static const char *mv_kernel_name(int t) {
    return t == GT_Q4_0 ? "kernel_mul_mv_q4_0_f32" : t == GT_Q8_0 ? "kernel_mul_mv_q8_0_f32" : t == GT_Q4_K ? "kernel_mul_mv_q4_K_f32" : "kernel_mul_mv_q6_K_f32";
}
static const char *mm_kernel_name(int t) {
    return t == GT_Q4_0 ? "kernel_mul_mm_q4_0_tensor_f32" : t == GT_Q8_0 ? "kernel_mul_mm_q8_0_tensor_f32" : "kernel_mul_mm_q6_K_tensor_f32";
}
static const char *mv_id_kernel_name(int t) {
    return t == GT_Q4_0 ? "kernel_mul_mv_id_q4_0_f32" : t == GT_Q8_0 ? "kernel_mul_mv_id_q8_0_f32" : t == GT_Q4_K ? "kernel_mul_mv_id_q4_K_f32"
         : t == GT_Q5_K ? "kernel_mul_mv_id_q5_K_f32" : "kernel_mul_mv_id_q6_K_f32";
}
static const char *mm_id_kernel_name(int t) {
    return t == GT_Q4_0 ? "kernel_mul_mm_id_q4_0_tensor_f32" : t == GT_Q8_0 ? "kernel_mul_mm_id_q8_0_tensor_f32" : t == GT_Q4_K ? "kernel_mul_mm_id_q4_K_tensor_f32" : "kernel_mul_mm_id_q6_K_tensor_f32";
}

static int check_handles(mlxn_encoder *enc, mlxn_device *dev, std::initializer_list<const void *> ptrs) {
    if (!enc || !dev) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: encoder and device must not be null");
    for (const void *p : ptrs)
        if (!p) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: buffers and params must not be null");
    return MLXN_OK;
}

struct ShardOut {            // row-sharded output: see QmvArgs
    uint32_t y_ld = 0, y_col0 = 0, n_peer = 0;
    float *peer[kMaxPeers] = {};
};
static int dispatch_mv(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input, mlxn_buffer *weight,
                       mlxn_buffer *output, const mlxn_qmm_params *p, const ShardOut *sh = nullptr) {
    int rc = touch_kernel(reg, dev, mv_kernel_name((int)p->ggml_type));
    if (rc) return rc;
    const int mode = opt_qmv();
    // "auto": the register-level kernel where it measured fastest (few activation rows: its cost grows with m, the
    // tensor-memory kernel's does not), the tensor-memory kernel for the rest
    auto wants_mma = [&](const QmvArgs &a) {
        if (mode == 4) return true;
        if (mode != 3) return false;
        // measured: batched, the register-level kernel is the faster one except for many activation rows on the
        // long-K and the widest Q6_K shapes
        if ((int)p->ggml_type == GT_Q4_K) return true;   // (its only other kernel is the plain one)
        if (a.m > 4) return false;
        if (a.m == 4 && a.k >= 8192) return false;
        return true;
    };
    auto make_args = [&](uint32_t m0) {
        QmvArgs a{};
        a.w = weight->dev();
        a.x = reinterpret_cast<const float *>(input->dev()) + (size_t)m0 * p->k;
        a.y = reinterpret_cast<float *>(output->dev()) + (size_t)m0 * (sh ? sh->y_ld : p->n);
        if (sh) {
            a.y_ld = sh->y_ld;
            a.y_col0 = sh->y_col0;
            a.n_peer = sh->n_peer;
            for (uint32_t i = 0; i < sh->n_peer; i++) a.y_peer[i] = sh->peer[i] + (size_t)m0 * sh->y_ld;
        }
        a.ids = nullptr;
        a.n = p->n;
        a.k = p->k;
        a.m = (p->m - m0) < 8 ? (p->m - m0) : 8;
        a.nprob = 1;
        a.top_k = 1;
        a.n_experts = 1;
        a.expert_stride = 0;
        a.status = enc->status_dev;
        a.early_weights = weight->st->kernel_written ? 0u : 1u;
        return a;
    };
    // A mat-vec for the register-level kernel is not launched at once: it waits for the operations that follow, and
    // conflict-free mat-vecs of the same block type leave as one kernel (upstream dispatches the operations between
    // two barriers concurrently, src/encoder.rs:837-853).  The group ends, and the kernel is launched, at the first
    // conflict, barrier, commit or capture boundary, or when the next mat-vec does not fit the batch.
    if (p->m <= 8) {
        const QmvArgs a0 = make_args(0);
        if (wants_mma(a0) && qmv_mma_supported((int)p->ggml_type, a0)) {
            const bool batch = g_opt_mv_batch.load() != 0;
            const bool pair = qmv_mma_pair_mode((int)p->ggml_type, a0);
            const bool fits = batch && !enc->pend.empty() && enc->pend_type == (int)p->ggml_type &&
                              enc->pend_mp == mv_row_class(a0.m) && enc->pend_pair == pair && enc->pend.size() < kMvBatchMax;
            if (!enc->pend.empty() && !fits && (rc = encoder_flush_pending(enc))) return rc;
            // A mat-vec that depends on the batch it would join (it reads a result of the batch, or writes over one)
            // still joins it when the group holds nothing but that batch: the kernel then starts it after the
            // mat-vecs ahead of it (a barrier across its grid) while the weights keep streaming.
            bool chained = false;
            if (fits && g_opt_mv_chain.load() && enc->grp_pend_only && a0.n_peer == 0 && enc->pend[0].n_peer == 0 &&
                op_conflicts(enc, {{input, false}, {weight, false}, {output, true}}, enc->pend_lane))
                chained = true;
            if ((rc = op_begin(enc, {{input, false}, {weight, false}, {output, true}}, true, chained))) return rc;
            // (a conflict found by op_begin has launched the batch and started a new group)
            if (enc->pend.empty()) {
                enc->pend_type = (int)p->ggml_type;
                enc->pend_mp = mv_row_class(a0.m);
                enc->pend_pair = pair;
                enc->pend_lane = enc->cur_lane;
            }
            enc->pend.push_back(a0);
            enc->pend.back().after_earlier = chained && enc->pend.size() > 1 ? 1u : 0u;
            for (mlxn_buffer *b : {input, weight, output}) {
                std::lock_guard<std::mutex> lk(b->st->mu);
                b->st->pend_enc = enc;
            }
            g_last_kernel = "qmv_mma";
            g_dispatch.fetch_add(1);
            if (!batch) return encoder_flush_pending(enc);
            return MLXN_OK;
        }
    }
    if ((rc = op_begin(enc, {{input, false}, {weight, false}, {output, true}}))) return rc;
    const bool stream = opt_qmv_stream();
    // rows are processed in groups of at most 8 (the reference launches one grid row per input row)
    for (uint32_t m0 = 0; m0 < p->m; m0 += 8) {
        const QmvArgs a = make_args(m0);
        // The tensor-memory kernel's time does not grow with the number of rows, the streaming SIMT kernel's does.
        static const int min_m = [] { const char *e = exp_env("MLXN_QMV_TC_MIN_M"); return e ? atoi(e) : 1; }();         // experiment switches
        static const int min_m_q6k = [] { const char *e = exp_env("MLXN_QMV_TC_MIN_M_Q6K"); return e ? atoi(e) : 1; }();
        const int need_m = (int)p->ggml_type == GT_Q6_K ? (a.k >= 8192 ? (min_m_q6k < 2 ? min_m_q6k : 2) : min_m_q6k) : min_m;
        const bool want_tc = mode == 2 || ((mode == 3 || mode == 4) && (int)a.m >= need_m);
        if ((mode == 4 || (mode == 3 && (int)p->ggml_type == GT_Q4_K)) && p->m > 8 && qmv_mma_supported((int)p->ggml_type, a)) {
            CUDA_TRY(launch_qmv_mma((int)p->ggml_type, &a, 1, dev->sm_count, g_opt_mma_ctas.load(), g_opt_mma_tpw.load(), enc->stream),
                     "mat-vec launch");
            g_launches.fetch_add(1);
            g_last_kernel = "qmv_mma";
            continue;
        }
        if (want_tc && mode != 4 && qmv_tc_supported((int)p->ggml_type, a)) {
            // tensor-memory path: packed activations, block sums and split-K partial sums live in the encoder's arena
            uint8_t *scratch = nullptr;
            if ((rc = encoder_scratch(enc, qmv_tc_scratch_bytes(a), &scratch))) return rc;
            int launches = 0;
            CUDA_TRY(launch_qmv_tc((int)p->ggml_type, a, scratch, enc->status_dev + 64, dev->sm_count, enc->stream, nullptr,
                                   nullptr, &launches),
                     "mat-vec launch");
            g_launches.fetch_add((uint64_t)launches);
            g_last_kernel = "qmv_tc";
            continue;
        }
        CUDA_TRY(launch_qmv((int)p->ggml_type, a, stream, dev->sm_count, enc->stream, &g_last_kernel), "mat-vec launch");
        g_launches.fetch_add(1);
    }
    g_dispatch.fetch_add(1);
    return MLXN_OK;
}

static int dispatch_mm(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input, mlxn_buffer *weight,
                       mlxn_buffer *output, const mlxn_qmm_params *p, const ShardOut *sh = nullptr) {
    int rc = touch_kernel(reg, dev, mm_kernel_name((int)p->ggml_type));
    if (rc) return rc;
    if ((rc = op_begin(enc, {{input, false}, {weight, false}, {output, true}}))) return rc;
    QmmArgs a{};
    a.w = weight->dev();
    a.x = reinterpret_cast<const float *>(input->dev());
    a.y = reinterpret_cast<float *>(output->dev());
    a.m = p->m;
    a.n = p->n;
    a.k = p->k;
    a.top_k = 1;
    a.n_experts = 1;
    a.total_rows = p->m;
    a.status = enc->status_dev;
    if (sh) {
        a.y_ld = sh->y_ld;
        a.y_col0 = sh->y_col0;
        a.n_peer = sh->n_peer;
        for (uint32_t i = 0; i < sh->n_peer; i++) a.y_peer[i] = sh->peer[i];
        if (!qmm_tc_supported(a))
            return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_ggml_sharded: the mat-mat form needs K to be a multiple of 32");
    }
    if ((sh || opt_qmm_tc()) && qmm_tc_supported(a)) {
        const uint32_t nt = qmm_tc_pick_nt((int)p->ggml_type, p->m, p->n, dev->sm_count, false);
        uint8_t *scratch = nullptr;
        if ((rc = encoder_scratch(enc, qmm_tc_scratch_bytes(a, nt, false), &scratch))) return rc;
        int launches = 0;
        CUDA_TRY(launch_qmm_tc((int)p->ggml_type, a, false, nt, scratch, enc->stream, &launches), "mat-mat launch");
        g_launches.fetch_add(launches);
        g_last_kernel = "qmm_tc";
    } else {
        CUDA_TRY(launch_qmm_simt((int)p->ggml_type, a, false, p->m, enc->stream), "mat-mat launch");
        g_launches.fetch_add(1);
        g_last_kernel = "qmm_simt";
    }
    g_dispatch.fetch_add(1);
    return MLXN_OK;
}

static int validate_dense(const char *who_types, mlxn_buffer *input, mlxn_buffer *weight, mlxn_buffer *output,
                          const mlxn_qmm_params *p, bool allow_q4k) {
    const int t = (int)p->ggml_type;
    const bool ok_type = t == GT_Q4_0 || t == GT_Q8_0 || t == GT_Q6_K || (allow_q4k && t == GT_Q4_K);
    if (!ok_type) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s does not support %s%s", who_types, ggml_name(t),
                              allow_q4k ? " — use a different dispatch path" : "");
    if (p->m == 0 || p->k == 0 || p->n == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: M, K, and N must all be > 0");
    const uint32_t qk = ggml_qk(t);
    if (p->k % qk != 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: K (%u) must be divisible by block QK (%u)", p->k, qk);
    if (!input || !weight || !output) return MLXN_OK;
    const size_t expected_w = (size_t)p->n * (p->k / qk) * ggml_block_bytes(t);
    if (weight->len < expected_w)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: Weight buffer too small: expected %zu bytes for %s [%ux%u], got %zu",
                    expected_w, ggml_name(t), p->n, p->k, weight->len);
    const size_t expected_in = (size_t)p->m * p->k * 4;
    if (input->len < expected_in)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: Input buffer too small: expected %zu bytes for [%ux%u] f32, got %zu",
                    expected_in, p->m, p->k, input->len);
    const size_t expected_out = (size_t)p->m * p->n * 4;
    if (output->len < expected_out)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: Output buffer too small: expected %zu bytes for [%ux%u] f32, got %zu",
                    expected_out, p->m, p->n, output->len);
    return MLXN_OK;
}

static int check_alignment(mlxn_buffer *input, mlxn_buffer *weight, mlxn_buffer *output) {
    if ((uintptr_t)weight->dev() & 1u)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: weight data must be 2-byte aligned (GGML blocks hold f16 scales)");
    if (((uintptr_t)input->dev() & 3u) || ((uintptr_t)output->dev() & 3u))
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: f32 buffers must be 4-byte aligned");
    return MLXN_OK;
}

extern "C" int mlxn_quantized_matmul_ggml(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input,
                                          mlxn_buffer *weight, mlxn_buffer *output, const mlxn_qmm_params *params) {
    int rc = check_handles(enc, dev, {input, weight, output, params});
    if (rc) return rc;
    if ((rc = validate_dense("quantized_matmul_ggml", input, weight, output, params, true))) return rc;
    if ((rc = check_alignment(input, weight, output))) return rc;
    // Q4_K has no dense mat-mat upstream either: it takes the mat-vec route at any m
    // (src/ops/quantized_matmul_ggml.rs:350-360)
    if (params->m > MLXN_MM_ROUTING_THRESHOLD && params->k >= 32 && (int)params->ggml_type != GT_Q4_K)
        return dispatch_mm(enc, reg, dev, input, weight, output, params);
    return dispatch_mv(enc, reg, dev, input, weight, output, params);
}

extern "C" int mlxn_quantized_matmul_ggml_sharded(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input,
                                                  mlxn_buffer *weight, mlxn_buffer *output, const mlxn_qmm_params *params,
                                                  uint32_t n_total, uint32_t col0, void *const *peer_outputs, uint32_t n_peers) {
    int rc = check_handles(enc, dev, {input, weight, output, params});
    if (rc) return rc;
    if (params->m == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_ggml_sharded: m must be > 0");
    if (params->m > MLXN_MM_ROUTING_THRESHOLD && (int)params->ggml_type == GT_Q4_K)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_ggml_sharded: Q4_K has no mat-mat form");
    if (n_peers > (uint32_t)kMaxPeers || (n_peers && !peer_outputs))
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_ggml_sharded: at most %d peer outputs", kMaxPeers);
    if ((uint64_t)col0 + params->n > n_total)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_ggml_sharded: columns [%u, %u) exceed n_total (%u)", col0,
                    col0 + params->n, n_total);
    // the local problem is validated as usual, against a [m, n] view; the output buffer must hold [m, n_total]
    if ((rc = validate_dense("quantized_matmul_ggml_sharded", input, weight, output, params, true))) return rc;
    if (output->len < (size_t)params->m * n_total * 4)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_ggml_sharded: output buffer too small: expected %zu bytes for [%u x %u] f32, got %zu",
                    (size_t)params->m * n_total * 4, params->m, n_total, output->len);
    if ((rc = check_alignment(input, weight, output))) return rc;
    ShardOut sh;
    sh.y_ld = n_total;
    sh.y_col0 = col0;
    sh.n_peer = n_peers;
    for (uint32_t i = 0; i < n_peers; i++) {
        if (!peer_outputs[i] || ((uintptr_t)peer_outputs[i] & 3u))
            return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_ggml_sharded: peer output %u is null or misaligned", i);
        sh.peer[i] = static_cast<float *>(peer_outputs[i]);
    }
    if (params->m > MLXN_MM_ROUTING_THRESHOLD) return dispatch_mm(enc, reg, dev, input, weight, output, params, &sh);
    return dispatch_mv(enc, reg, dev, input, weight, output, params, &sh);
}

// quantized_matmul_mm_tensor_perm021 (src/ops/quantized_matmul_ggml.rs:640-742): the O-projection reads the attention
// output where it lies — bf16 [n_heads, seq_len, head_dim] — instead of a permuted f32 copy.
extern "C" int mlxn_quantized_matmul_mm_tensor_perm021(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev,
                                                       mlxn_buffer *input_bf16, mlxn_buffer *weight, mlxn_buffer *output,
                                                       const mlxn_qmm_perm021_params *p) {
    int rc = check_handles(enc, dev, {input_bf16, weight, output, p});
    if (rc) return rc;
    const int t = (int)p->ggml_type;
    if (t != GT_Q4_0 && t != GT_Q6_K)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_mm_tensor_perm021: unsupported ggml_type %s (only Q4_0 and Q6_K are instantiated)",
                    ggml_name(t));
    if (p->head_dim == 0 || p->head_dim % 32 != 0)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_mm_tensor_perm021: head_dim %u must be a positive multiple of 32 (NK tile width)",
                    p->head_dim);
    if (p->m == 0 || p->n == 0 || p->k == 0)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_mm_tensor_perm021: M, K, and N must all be > 0");
    if (p->k % p->head_dim != 0)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_mm_tensor_perm021: k (%u) must be divisible by head_dim (%u)", p->k,
                    p->head_dim);
    const uint32_t qk = ggml_qk(t);
    if (p->k % qk != 0)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_mm_tensor_perm021: K (%u) must be divisible by block QK (%u)", p->k, qk);
    const size_t need_in = (size_t)p->k * p->m * 2;   // n_heads * seq_len * head_dim bf16
    if (input_bf16->len < need_in)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_mm_tensor_perm021: input_bf16 buffer too small (have %zu, need %zu)",
                    input_bf16->len, need_in);
    const size_t need_w = (size_t)p->n * (p->k / qk) * ggml_block_bytes(t), need_out = (size_t)p->m * p->n * 4;
    if (weight->len < need_w)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_mm_tensor_perm021: weight buffer too small (have %zu, need %zu)", weight->len, need_w);
    if (output->len < need_out)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_mm_tensor_perm021: output buffer too small (have %zu, need %zu)", output->len, need_out);
    if (((uintptr_t)weight->dev() & 1u) || ((uintptr_t)output->dev() & 3u) || ((uintptr_t)input_bf16->dev() & 15u))
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_mm_tensor_perm021: weight data must be 2-byte, output 4-byte, input_bf16 16-byte aligned");
    if ((rc = touch_kernel(reg, dev, t == GT_Q4_0 ? "kernel_mul_mm_q4_0_tensor_bf16_perm021" : "kernel_mul_mm_q6_K_tensor_bf16_perm021"))) return rc;
    if ((rc = op_begin(enc, {{input_bf16, false}, {weight, false}, {output, true}}))) return rc;
    QmmArgs a{};
    a.w = weight->dev();
    a.x = nullptr;
    a.x_bf16 = reinterpret_cast<const uint16_t *>(input_bf16->dev());
    a.head_dim = p->head_dim;
    a.y = reinterpret_cast<float *>(output->dev());
    a.m = p->m;
    a.n = p->n;
    a.k = p->k;
    a.top_k = 1;
    a.n_experts = 1;
    a.total_rows = p->m;
    a.status = enc->status_dev;
    const uint32_t nt = qmm_tc_pick_nt(t, p->m, p->n, dev->sm_count, false);
    uint8_t *scratch = nullptr;
    if ((rc = encoder_scratch(enc, qmm_tc_scratch_bytes(a, nt, false), &scratch))) return rc;
    int launches = 0;
    CUDA_TRY(launch_qmm_tc(t, a, false, nt, scratch, enc->stream, &launches), "mat-mat launch");
    g_launches.fetch_add(launches);
    g_last_kernel = "qmm_tc";
    g_dispatch.fetch_add(1);
    return MLXN_OK;
}

extern "C" int mlxn_dispatch_mm_for_test(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input,
                                         mlxn_buffer *weight, mlxn_buffer *output, const mlxn_qmm_params *params) {
    int rc = check_handles(enc, dev, {input, weight, output, params});
    if (rc) return rc;
    if ((rc = validate_dense("dispatch_mm_for_test", input, weight, output, params, false))) return rc;
    if ((rc = check_alignment(input, weight, output))) return rc;
    return dispatch_mm(enc, reg, dev, input, weight, output, params);
}

// ------------------------------------------------------------------------------------------------
// quantized_matmul_id_ggml
// ------------------------------------------------------------------------------------------------
static int validate_id(const char *who, mlxn_buffer *input, mlxn_buffer *weight, mlxn_buffer *ids, mlxn_buffer *output,
                       const mlxn_qmm_id_params *p) {
    const int t = (int)p->ggml_type;
    if (p->n_tokens == 0 || p->k == 0 || p->n == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: n_tokens, K, and N must all be > 0", who);
    if (p->top_k == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: top_k must be > 0", who);
    if (p->n_experts == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: n_experts must be > 0", who);
    if (p->n_experts > 65535u)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: n_experts (%u) must be <= 65535", who, p->n_experts);
    if (t < 0 || t > MLXN_GGML_I16) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: unknown ggml_type %d", who, t);
    const uint32_t qk = ggml_qk(t);
    if (p->k % qk != 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: K (%u) must be divisible by block QK (%u)", who, p->k, qk);
    const size_t expected_in = (size_t)p->n_tokens * p->k * 4;
    if (input->len < expected_in)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: input buffer too small: expected %zu bytes for [%u x %u] f32, got %zu",
                    who, expected_in, p->n_tokens, p->k, input->len);
    const size_t per_expert = (size_t)p->n * (p->k / qk) * ggml_block_bytes(t);
    if (p->expert_stride < per_expert)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: expert_stride (%llu) < per_expert_bytes (%zu)", who,
                    (unsigned long long)p->expert_stride, per_expert);
    const size_t total_w = per_expert * p->n_experts;
    if (weight->len < total_w)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: weight buffer too small: expected %zu bytes for %u experts, got %zu",
                    who, total_w, p->n_experts, weight->len);
    // this build also reads expert e at e*expert_stride, so the strided extent must be inside the buffer
    if (weight->len < (size_t)(p->n_experts - 1) * p->expert_stride + per_expert)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: weight buffer too small for %u experts at expert_stride %llu: got %zu bytes",
                    who, p->n_experts, (unsigned long long)p->expert_stride, weight->len);
    const size_t total_rows = (size_t)p->n_tokens * p->top_k;
    if (ids->len < total_rows * 4)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: ids buffer too small: expected %zu bytes for [%u * %u] u32, got %zu",
                    who, total_rows * 4, p->n_tokens, p->top_k, ids->len);
    const size_t expected_out = total_rows * p->n * 4;
    if (output->len < expected_out)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: output buffer too small: expected %zu bytes for [%zu x %u] f32, got %zu",
                    who, expected_out, total_rows, p->n, output->len);
    if (t != GT_Q4_0 && t != GT_Q8_0 && t != GT_Q6_K && t != GT_Q4_K && t != GT_Q5_K)
        return fail(MLXN_KERNEL_NOT_FOUND, "Kernel not found: expert-routed kernels for %s are not built into this library yet", ggml_name(t));
    if (total_rows > 0x7FFFFFFFull / 1) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: %s: n_tokens * top_k is too large", who);
    return MLXN_OK;
}

// `up` != nullptr: the fused SwiGLU form (src/ops/quantized_matmul_id_ggml.rs:551-670): `input` is the gate, both are
// [n_tokens * top_k, k] with one row per OUTPUT row, and the activations are silu(gate) * up.
static int dispatch_id_mv(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input, mlxn_buffer *weight,
                          mlxn_buffer *ids, mlxn_buffer *output, const mlxn_qmm_id_params *p, mlxn_buffer *up = nullptr) {
    const int t = (int)p->ggml_type;
    int rc = touch_kernel(reg, dev, up ? "kernel_mul_mv_id_q4_0_f32_swiglu" : mv_id_kernel_name(t));
    if (rc) return rc;
    const uint32_t rows = p->n_tokens * p->top_k;
    QmvArgs a{};
    a.w = weight->dev();
    a.x = reinterpret_cast<const float *>(input->dev());
    a.x2 = up ? reinterpret_cast<const float *>(up->dev()) : nullptr;
    a.y = reinterpret_cast<float *>(output->dev());
    a.ids = reinterpret_cast<const uint32_t *>(ids->dev());
    a.n = p->n;
    a.k = p->k;
    a.m = 1;
    a.nprob = rows;
    a.top_k = up ? 1 : p->top_k;   // (fused: every output row has its own input row)
    a.n_experts = p->n_experts;
    a.expert_stride = p->expert_stride;
    a.status = enc->status_dev;
    // Few rows (decode): every (token, slot) row is one mat-vec of the register-level kernel, and the rows of this call,
    // and of the calls around it that do not depend on it (gate and up of one layer), leave as one launch.
    const int mode = opt_qmv();
    if ((mode == 3 || mode == 4) && rows <= kMvBatchMax && qmv_mma_supported_routed(t, a)) {
        const bool batch = g_opt_mv_batch.load() != 0;
        const bool fits = batch && !enc->pend.empty() && enc->pend_type == t && enc->pend_mp == 1 && !enc->pend_pair &&
                          enc->pend.size() + rows <= kMvBatchMax;
        if (!enc->pend.empty() && !fits && (rc = encoder_flush_pending(enc))) return rc;
        if ((rc = op_begin(enc, {{input, false}, {up, false}, {weight, false}, {ids, false}, {output, true}}, true))) return rc;
        if (enc->pend.empty()) {
            enc->pend_type = t;
            enc->pend_mp = 1;
            enc->pend_pair = false;
            enc->pend_lane = enc->cur_lane;
        }
        for (uint32_t r = 0; r < rows; r++) {
            QmvArgs ar = a;
            ar.nprob = 1;
            ar.id_index = r;
            ar.x = a.x + (size_t)(r / a.top_k) * p->k;
            ar.x2 = a.x2 ? a.x2 + (size_t)r * p->k : nullptr;
            ar.y = a.y + (size_t)r * p->n;
            ar.early_weights = 0;
            enc->pend.push_back(ar);
        }
        for (mlxn_buffer *b : {input, up, weight, ids, output}) {
            if (!b) continue;
            std::lock_guard<std::mutex> lk(b->st->mu);
            b->st->pend_enc = enc;
        }
        g_last_kernel = "qmv_mma";
        g_dispatch.fetch_add(1);
        if (!batch) return encoder_flush_pending(enc);
        return MLXN_OK;
    }
    if ((rc = op_begin(enc, {{input, false}, {up, false}, {weight, false}, {ids, false}, {output, true}}))) return rc;
    int launches = 1;
    if (up && !(opt_qmv_stream() && qmv_stream_available(t, a, dev->sm_count))) {
        // no fused form for this shape: SwiGLU into the encoder's scratch, then the plain routed mat-vec
        uint8_t *scratch = nullptr;
        if ((rc = encoder_scratch(enc, (size_t)rows * p->k * 4, &scratch))) return rc;
        CUDA_TRY(launch_silu_mul(a.x, a.x2, reinterpret_cast<float *>(scratch), rows * p->k, enc->stream), "silu_mul launch");
        a.x = reinterpret_cast<const float *>(scratch);
        a.x2 = nullptr;
        launches = 2;
    }
    CUDA_TRY(launch_qmv(t, a, opt_qmv_stream(), dev->sm_count, enc->stream, &g_last_kernel), "mat-vec launch");
    g_launches.fetch_add((uint64_t)launches);
    g_dispatch.fetch_add(1);
    return MLXN_OK;
}

// two-stage route: bucket (token, slot) pairs by expert, then the grouped mat-mat
static int dispatch_id_mm_stages(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input,
                                 mlxn_buffer *weight, mlxn_buffer *ids, mlxn_buffer *output, uint32_t *htpe, int32_t *hids,
                                 uint32_t hids_stride, size_t scratch_used, const mlxn_qmm_id_params *p) {
    char map0_name[48];
    snprintf(map0_name, sizeof(map0_name), "kernel_mul_mm_id_map0_ne20_%u", p->top_k);
    int rc = touch_kernel(reg, dev, known_kernel(map0_name) ? map0_name : "kernel_mul_mm_id_map0_ne20_n");
    if (rc) return rc;
    if ((rc = touch_kernel(reg, dev, mm_id_kernel_name((int)p->ggml_type)))) return rc;
    CUDA_TRY(launch_moe_map0(reinterpret_cast<const uint32_t *>(ids->dev()), p->n_tokens, p->top_k, p->n_experts,
                             hids_stride, htpe, hids, reinterpret_cast<float *>(output->dev()), p->n, enc->stream),
             "map0 launch");
    g_launches.fetch_add(1);
    g_dispatch.fetch_add(1);
    g_barrier.fetch_add(1);  // upstream's RAW fence between map0 and mm_id (stream order provides it here)
    QmmArgs a{};
    a.w = weight->dev();
    a.x = reinterpret_cast<const float *>(input->dev());
    a.y = reinterpret_cast<float *>(output->dev());
    a.m = p->n_tokens;
    a.n = p->n;
    a.k = p->k;
    a.htpe = htpe;
    a.hids = hids;
    a.hids_stride = hids_stride;
    a.top_k = p->top_k;
    a.n_experts = p->n_experts;
    a.total_rows = p->n_tokens * p->top_k;
    a.expert_stride = p->expert_stride;
    a.status = enc->status_dev;
    if (opt_qmm_tc() && qmm_tc_supported(a)) {
        const uint32_t nt = qmm_tc_pick_nt((int)p->ggml_type, p->n_tokens, p->n, dev->sm_count, true);
        uint8_t *scratch = nullptr;
        const size_t need = qmm_tc_scratch_bytes(a, nt, true);
        if ((rc = encoder_scratch(enc, scratch_used + need, &scratch))) return rc;
        int launches = 0;
        CUDA_TRY(launch_qmm_tc((int)p->ggml_type, a, true, nt, scratch + scratch_used, enc->stream, &launches), "mat-mat launch");
        g_launches.fetch_add(launches);
        g_last_kernel = "qmm_tc_id";
    } else {
        CUDA_TRY(launch_qmm_simt((int)p->ggml_type, a, true, p->n_tokens, enc->stream), "mat-mat launch");
        g_launches.fetch_add(1);
        g_last_kernel = "qmm_simt_id";
    }
    g_dispatch.fetch_add(1);
    return MLXN_OK;
}

// Upstream routes to the grouped mat-mat only for top_k in {1, 8} (the two instantiations of its bucketing kernel,
// src/ops/quantized_matmul_id_ggml.rs:265-273) and names the other values as a gap
// (docs/moe-q-perf-audit-2026-04-27.md:79-84); the bucketing kernel here takes any top_k, so every top_k takes the route.
static bool id_routes_to_mm(const mlxn_qmm_id_params *p) {
    return p->n_tokens > mlxn_mm_id_routing_threshold() && p->k >= 32 && (int)p->ggml_type != GT_Q5_K;
}

extern "C" size_t mlxn_id_mm_htpe_bytes(const mlxn_qmm_id_params *p) { return p ? (size_t)p->n_experts * 4 : 0; }
extern "C" size_t mlxn_id_mm_hids_bytes(const mlxn_qmm_id_params *p) { return p ? (size_t)p->n_experts * p->n_tokens * 4 : 0; }

extern "C" int mlxn_quantized_matmul_id_ggml(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input,
                                             mlxn_buffer *weight, mlxn_buffer *ids, mlxn_buffer *output,
                                             const mlxn_qmm_id_params *params) {
    int rc = check_handles(enc, dev, {input, weight, ids, output, params});
    if (rc) return rc;
    if ((rc = validate_id("quantized_matmul_id_ggml", input, weight, ids, output, params))) return rc;
    if ((rc = check_alignment(input, weight, output))) return rc;
    if (!id_routes_to_mm(params)) return dispatch_id_mv(enc, reg, dev, input, weight, ids, output, params);
    if ((rc = op_begin(enc, {{input, false}, {weight, false}, {ids, false}, {output, true}}))) return rc;
    // routing scratch comes out of the encoder's arena instead of two fresh allocations per call
    const size_t htpe_b = (mlxn_id_mm_htpe_bytes(params) + 1023) / 1024 * 1024;
    const size_t hids_b = (mlxn_id_mm_hids_bytes(params) + 1023) / 1024 * 1024;
    QmmArgs probe{};
    probe.k = params->k;
    probe.n_experts = params->n_experts;
    probe.total_rows = params->n_tokens * params->top_k;
    const size_t tc_b = qmm_tc_scratch_bytes(probe, qmm_tc_pick_nt((int)params->ggml_type, params->n_tokens, params->n, dev->sm_count, true), true);
    uint8_t *scratch = nullptr;
    if ((rc = encoder_scratch(enc, htpe_b + hids_b + tc_b, &scratch))) return rc;
    return dispatch_id_mm_stages(enc, reg, dev, input, weight, ids, output, reinterpret_cast<uint32_t *>(scratch),
                                 reinterpret_cast<int32_t *>(scratch + htpe_b), params->n_tokens, htpe_b + hids_b, params);
}

// quantized_matmul_id_swiglu_q4_0 (src/ops/quantized_matmul_id_ggml.rs:551-670), for Q4_0, Q8_0 and Q6_K:
// output[r, :] = W[ids[r]] . (silu(gate[r, :]) * up[r, :]) for the n_tokens * top_k rows r.
extern "C" int mlxn_quantized_matmul_id_swiglu(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *gate,
                                               mlxn_buffer *up, mlxn_buffer *weight, mlxn_buffer *ids, mlxn_buffer *output,
                                               const mlxn_qmm_id_params *params) {
    int rc = check_handles(enc, dev, {gate, up, weight, ids, output, params});
    if (rc) return rc;
    const int t = (int)params->ggml_type;
    if (t != GT_Q4_0 && t != GT_Q8_0 && t != GT_Q6_K)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_id_swiglu: expected Q4_0, Q8_0 or Q6_K, got %s", ggml_name(t));
    if (params->n_tokens == 0 || params->k == 0 || params->n == 0)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_id_swiglu: n_tokens, K, and N must all be > 0");
    if (params->top_k == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_id_swiglu: top_k must be > 0");
    // gate and up hold one row per (token, slot) pair: validate the rest as the routed mat-vec over n_tokens * top_k "tokens"
    mlxn_qmm_id_params q = *params;
    const uint64_t rows = (uint64_t)params->n_tokens * params->top_k;
    if (rows > 0x7FFFFFFFull) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_id_swiglu: n_tokens * top_k is too large");
    q.n_tokens = (uint32_t)rows;
    q.top_k = 1;
    if ((rc = validate_id("quantized_matmul_id_swiglu", gate, weight, ids, output, &q))) return rc;
    if (up->len < (size_t)rows * params->k * 4)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: quantized_matmul_id_swiglu: up buffer too small: expected %zu bytes, got %zu",
                    (size_t)rows * params->k * 4, up->len);
    if ((rc = check_alignment(gate, weight, output))) return rc;
    if ((uintptr_t)up->dev() & 3u) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: f32 buffers must be 4-byte aligned");
    return dispatch_id_mv(enc, reg, dev, gate, weight, ids, output, &q, up);
}

// ------------------------------------------------------------------------------------------------
// The expert half of a MoE FFN layer as one call (no upstream counterpart: upstream encodes the three routed products and
// the SwiGLU one by one, e.g. benches/bench_mul_mm_id_qwen36_ffn.rs).  Same results as that chain, bit for bit; what the
// one call saves on the grouped route is preparation the three products share: the pairs are bucketed by expert once
// (the down projection's rows are the same (token, slot) pairs in the same order), the tile list is built once, the
// activations are packed once for gate and up, and the SwiGLU is formed while the down projection's operand is packed
// (no stand-alone SwiGLU launch, no [pairs, ffn] intermediate).  Seven launches instead of thirteen.
//   gate_out, up_out: f32 [n_tokens * top_k, ffn]; down_out: f32 [n_tokens * top_k, hidden], one row per pair.
// Rows of pairs whose id names no expert: zeros in down_out, unspecified in gate_out / up_out on the grouped route.
// Few tokens (n_tokens <= the routing threshold), Q5_K or shapes outside the tensor-core kernel take the chain itself.
// ------------------------------------------------------------------------------------------------
extern "C" int mlxn_moe_ffn_layer(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *x, mlxn_buffer *ids,
                                  mlxn_buffer *gate_w, mlxn_buffer *up_w, mlxn_buffer *down_w, mlxn_buffer *gate_out,
                                  mlxn_buffer *up_out, mlxn_buffer *down_out, const mlxn_moe_ffn_params *p) {
    int rc = check_handles(enc, dev, {x, ids, gate_w, up_w, down_w, gate_out, up_out, down_out, p});
    if (rc) return rc;
    const uint64_t pairs = (uint64_t)p->n_tokens * p->top_k;
    if (pairs == 0 || pairs > 0x7FFFFFFFull)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: moe_ffn_layer: n_tokens * top_k must be in 1..2^31-1");
    mlxn_qmm_id_params pg{p->n_tokens, p->top_k, p->ffn, p->hidden, p->n_experts, p->gate_type, p->gate_stride};
    mlxn_qmm_id_params pu{p->n_tokens, p->top_k, p->ffn, p->hidden, p->n_experts, p->up_type, p->up_stride};
    mlxn_qmm_id_params pd{(uint32_t)pairs, 1, p->hidden, p->ffn, p->n_experts, p->down_type, p->down_stride};
    if ((rc = validate_id("moe_ffn_layer (gate)", x, gate_w, ids, gate_out, &pg))) return rc;
    if ((rc = validate_id("moe_ffn_layer (up)", x, up_w, ids, up_out, &pu))) return rc;
    if ((rc = validate_id("moe_ffn_layer (down)", gate_out, down_w, ids, down_out, &pd))) return rc;
    if ((rc = check_alignment(x, gate_w, gate_out)) || (rc = check_alignment(x, up_w, up_out)) ||
        (rc = check_alignment(gate_out, down_w, down_out)))
        return rc;
    auto probe = [&](const mlxn_qmm_id_params &q, mlxn_buffer *w) {
        QmmArgs a{};
        a.w = w->dev();
        a.k = q.k;
        a.expert_stride = q.expert_stride;
        return qmm_tc_supported(a);
    };
    const bool grouped = id_routes_to_mm(&pg) && id_routes_to_mm(&pu) && id_routes_to_mm(&pd) && opt_qmm_tc() &&
                         probe(pg, gate_w) && probe(pu, up_w) && probe(pd, down_w);
    if (!grouped) {
        // the chain itself: few tokens take the routed mat-vecs and the fused SwiGLU mat-vec; whatever else is left
        // takes the calls one by one, with the SwiGLU written over up_out
        if ((rc = mlxn_quantized_matmul_id_ggml(enc, reg, dev, x, gate_w, ids, gate_out, &pg))) return rc;
        if ((rc = mlxn_quantized_matmul_id_ggml(enc, reg, dev, x, up_w, ids, up_out, &pu))) return rc;
        const int td = (int)p->down_type;
        if (!id_routes_to_mm(&pd) && (td == GT_Q4_0 || td == GT_Q8_0 || td == GT_Q6_K)) {
            mlxn_qmm_id_params ps = pd;
            return mlxn_quantized_matmul_id_swiglu(enc, reg, dev, gate_out, up_out, down_w, ids, down_out, &ps);
        }
        if (pairs * p->ffn > 0xFFFFFFFFull) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: moe_ffn_layer: n_tokens * top_k * ffn is too large");
        if ((rc = mlxn_silu_mul(enc, reg, dev, gate_out, up_out, up_out, (uint32_t)(pairs * p->ffn)))) return rc;
        return mlxn_quantized_matmul_id_ggml(enc, reg, dev, up_out, down_w, ids, down_out, &pd);
    }
    if ((rc = op_begin(enc, {{x, false}, {ids, false}, {gate_w, false}, {up_w, false}, {down_w, false}, {gate_out, true},
                             {up_out, true}, {down_out, true}})))
        return rc;
    char map0_name[48];
    snprintf(map0_name, sizeof(map0_name), "kernel_mul_mm_id_map0_ne20_%u", p->top_k);
    if ((rc = touch_kernel(reg, dev, known_kernel(map0_name) ? map0_name : "kernel_mul_mm_id_map0_ne20_n"))) return rc;
    if ((rc = touch_kernel(reg, dev, mm_id_kernel_name((int)p->gate_type))) || (rc = touch_kernel(reg, dev, mm_id_kernel_name((int)p->up_type))) ||
        (rc = touch_kernel(reg, dev, mm_id_kernel_name((int)p->down_type))))
        return rc;
    // scratch: bucket sizes, buckets ([experts, n_tokens]: a token holds an expert at most once, and the down projection's
    // rows are the same pairs), then the tile list and the packed activations (sized for the longer of the two K)
    const uint32_t nt = qmm_tc_pick_nt((int)p->gate_type, p->n_tokens, p->ffn, dev->sm_count, true);
    const size_t htpe_b = ((size_t)p->n_experts * 4 + 1023) / 1024 * 1024;
    const size_t hids_b = ((size_t)p->n_experts * p->n_tokens * 4 + 1023) / 1024 * 1024;
    QmmArgs sz{};
    sz.k = p->hidden > p->ffn ? p->hidden : p->ffn;
    sz.n_experts = p->n_experts;
    sz.total_rows = (uint32_t)pairs;
    uint8_t *scratch = nullptr;
    if ((rc = encoder_scratch(enc, htpe_b + hids_b + qmm_tc_scratch_bytes(sz, nt, true), &scratch))) return rc;
    uint32_t *htpe = reinterpret_cast<uint32_t *>(scratch);
    int32_t *hids = reinterpret_cast<int32_t *>(scratch + htpe_b);
    uint8_t *tc = scratch + htpe_b + hids_b;
    CUDA_TRY(launch_moe_map0(reinterpret_cast<const uint32_t *>(ids->dev()), p->n_tokens, p->top_k, p->n_experts, p->n_tokens,
                             htpe, hids, reinterpret_cast<float *>(down_out->dev()), p->hidden, enc->stream),
             "map0 launch");
    g_launches.fetch_add(1);
    g_barrier.fetch_add(1);
    auto product = [&](const mlxn_qmm_id_params &q, mlxn_buffer *in, mlxn_buffer *in2, mlxn_buffer *w, mlxn_buffer *out,
                       uint32_t reuse) -> int {
        QmmArgs a{};
        a.w = w->dev();
        a.x = reinterpret_cast<const float *>(in->dev());
        a.x2 = in2 ? reinterpret_cast<const float *>(in2->dev()) : nullptr;
        a.y = reinterpret_cast<float *>(out->dev());
        a.m = q.n_tokens;
        a.n = q.n;
        a.k = q.k;
        a.htpe = htpe;
        a.hids = hids;
        a.hids_stride = p->n_tokens;
        a.top_k = q.top_k;
        a.n_experts = q.n_experts;
        a.total_rows = (uint32_t)pairs;
        a.expert_stride = q.expert_stride;
        a.status = enc->status_dev;
        a.reuse = reuse;
        int launches = 0;
        CUDA_TRY(launch_qmm_tc((int)q.ggml_type, a, true, nt, tc, enc->stream, &launches), "mat-mat launch");
        g_launches.fetch_add(launches);
        g_dispatch.fetch_add(1);
        return MLXN_OK;
    };
    if ((rc = product(pg, x, nullptr, gate_w, gate_out, 0u))) return rc;          // builds the tile list, packs x
    if ((rc = product(pu, x, nullptr, up_w, up_out, 3u))) return rc;              // takes both over
    if ((rc = product(pd, gate_out, up_out, down_w, down_out, 1u))) return rc;    // same tiles; packs silu(gate) * up
    g_last_kernel = "qmm_tc_id";
    g_dispatch.fetch_add(1);
    return MLXN_OK;
}

static int check_scratch_buffers(mlxn_buffer *htpe, mlxn_buffer *hids, const mlxn_qmm_id_params *p) {
    if (htpe->len < mlxn_id_mm_htpe_bytes(p))
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: htpe buffer too small: expected %zu bytes, got %zu", mlxn_id_mm_htpe_bytes(p), htpe->len);
    if (hids->len < mlxn_id_mm_hids_bytes(p))
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: hids buffer too small: expected %zu bytes, got %zu", mlxn_id_mm_hids_bytes(p), hids->len);
    if (((uintptr_t)htpe->dev() & 3u) || ((uintptr_t)hids->dev() & 3u))
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: scratch buffers must be 4-byte aligned");
    return MLXN_OK;
}

extern "C" int mlxn_quantized_matmul_id_ggml_pooled(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev,
                                                    mlxn_buffer *input, mlxn_buffer *weight, mlxn_buffer *ids,
                                                    mlxn_buffer *output, mlxn_buffer *htpe, mlxn_buffer *hids,
                                                    uint32_t n_experts_cap, uint32_t n_tokens_cap,
                                                    const mlxn_qmm_id_params *params) {
    int rc = check_handles(enc, dev, {input, weight, ids, output, htpe, hids, params});
    if (rc) return rc;
    if ((rc = validate_id("quantized_matmul_id_ggml_pooled", input, weight, ids, output, params))) return rc;
    if ((rc = check_alignment(input, weight, output))) return rc;
    if (!id_routes_to_mm(params)) return dispatch_id_mv(enc, reg, dev, input, weight, ids, output, params);
    if (params->n_experts > n_experts_cap)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: IdMmScratch: n_experts (%u) > cap (%u)", params->n_experts, n_experts_cap);
    if (params->n_tokens > n_tokens_cap)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: IdMmScratch: n_tokens (%u) > cap (%u)", params->n_tokens, n_tokens_cap);
    if ((rc = check_scratch_buffers(htpe, hids, params))) return rc;
    if ((rc = op_begin(enc, {{input, false}, {weight, false}, {ids, false}, {output, true}, {htpe, true}, {hids, true}})))
        return rc;
    return dispatch_id_mm_stages(enc, reg, dev, input, weight, ids, output, reinterpret_cast<uint32_t *>(htpe->dev()),
                                 reinterpret_cast<int32_t *>(hids->dev()), params->n_tokens, 0, params);
}

extern "C" int mlxn_dispatch_id_mm_for_test(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *input,
                                            mlxn_buffer *weight, mlxn_buffer *ids, mlxn_buffer *htpe, mlxn_buffer *hids,
                                            mlxn_buffer *output, const mlxn_qmm_id_params *params) {
    int rc = check_handles(enc, dev, {input, weight, ids, output, htpe, hids, params});
    if (rc) return rc;
    if ((rc = validate_id("dispatch_id_mm_for_test", input, weight, ids, output, params))) return rc;
    if ((rc = check_alignment(input, weight, output))) return rc;
    if ((rc = check_scratch_buffers(htpe, hids, params))) return rc;
    if ((rc = op_begin(enc, {{input, false}, {weight, false}, {ids, false}, {output, true}, {htpe, true}, {hids, true}})))
        return rc;
    return dispatch_id_mm_stages(enc, reg, dev, input, weight, ids, output, reinterpret_cast<uint32_t *>(htpe->dev()),
                                 reinterpret_cast<int32_t *>(hids->dev()), params->n_tokens, 0, params);
}

// ------------------------------------------------------------------------------------------------
// MoE glue
// ------------------------------------------------------------------------------------------------
extern "C" int mlxn_moe_softmax_topk(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *logits,
                                     mlxn_buffer *out_ids, mlxn_buffer *out_weights, uint32_t n_tokens,
                                     uint32_t n_experts, uint32_t top_k) {
    int rc = check_handles(enc, dev, {logits, out_ids, out_weights});
    if (rc) return rc;
    if (n_tokens == 0 || n_experts == 0 || top_k == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: moe_softmax_topk: n_tokens, n_experts and top_k must all be > 0");
    if (top_k > n_experts) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: moe_softmax_topk: top_k (%u) > n_experts (%u)", top_k, n_experts);
    if (top_k > 64) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: moe_softmax_topk: top_k (%u) > 64", top_k);
    if (n_experts > 8192) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: moe_softmax_topk: n_experts (%u) > 8192", n_experts);
    if (logits->len < (size_t)n_tokens * n_experts * 4 || out_ids->len < (size_t)n_tokens * top_k * 4 ||
        out_weights->len < (size_t)n_tokens * top_k * 4)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: moe_softmax_topk: a buffer is too small");
    if ((rc = touch_kernel(reg, dev, "moe_softmax_topk_f32"))) return rc;
    if ((rc = op_begin(enc, {{logits, false}, {out_ids, true}, {out_weights, true}}))) return rc;
    CUDA_TRY(launch_moe_softmax_topk(reinterpret_cast<const float *>(logits->dev()), n_tokens, n_experts, top_k,
                                     reinterpret_cast<uint32_t *>(out_ids->dev()), reinterpret_cast<float *>(out_weights->dev()),
                                     enc->stream),
             "moe_softmax_topk launch");
    g_launches.fetch_add(1);
    g_dispatch.fetch_add(1);
    g_last_kernel = "moe_softmax_topk";
    return MLXN_OK;
}

extern "C" int mlxn_silu_mul(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *gate, mlxn_buffer *up,
                             mlxn_buffer *out, uint32_t n) {
    int rc = check_handles(enc, dev, {gate, up, out});
    if (rc) return rc;
    if (n == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: silu_mul: n must be > 0");
    if (gate->len < (size_t)n * 4 || up->len < (size_t)n * 4 || out->len < (size_t)n * 4)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: silu_mul: a buffer is too small for %u f32 elements", n);
    if ((rc = touch_kernel(reg, dev, "silu_mul_f32"))) return rc;
    if ((rc = op_begin(enc, {{gate, false}, {up, false}, {out, true}}))) return rc;
    CUDA_TRY(launch_silu_mul(reinterpret_cast<const float *>(gate->dev()), reinterpret_cast<const float *>(up->dev()),
                             reinterpret_cast<float *>(out->dev()), n, enc->stream),
             "silu_mul launch");
    g_launches.fetch_add(1);
    g_dispatch.fetch_add(1);
    g_last_kernel = "silu_mul";
    return MLXN_OK;
}

static int moe_weighted_reduce_impl(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *expert_w,
                                   mlxn_buffer *y_expert, mlxn_buffer *sh_logit, mlxn_buffer *y_shared,
                                   mlxn_buffer *residual, mlxn_buffer *local_ids, mlxn_buffer *out, uint32_t n_tokens,
                                   uint32_t top_k, uint32_t h) {
    int rc = check_handles(enc, dev, {expert_w, y_expert, out});
    if (rc) return rc;
    if (n_tokens == 0 || top_k == 0 || h == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: moe_weighted_reduce: n_tokens, top_k and h must all be > 0");
    if (expert_w->len < (size_t)n_tokens * top_k * 4 || y_expert->len < (size_t)n_tokens * top_k * h * 4 ||
        out->len < (size_t)n_tokens * h * 4 || (y_shared && y_shared->len < (size_t)n_tokens * h * 4) ||
        (sh_logit && sh_logit->len < (size_t)n_tokens * 4) || (residual && residual->len < (size_t)n_tokens * h * 4) ||
        (local_ids && local_ids->len < (size_t)n_tokens * top_k * 4))
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: moe_weighted_reduce: a buffer is too small");
    if ((rc = touch_kernel(reg, dev, "moe_weighted_reduce_f32"))) return rc;
    if ((rc = op_begin(enc, {{expert_w, false}, {y_expert, false}, {out, true}, {sh_logit, false}, {y_shared, false},
                             {residual, false}, {local_ids, false}})))
        return rc;
    CUDA_TRY(launch_moe_weighted_reduce(reinterpret_cast<const float *>(expert_w->dev()),
                                        reinterpret_cast<const float *>(y_expert->dev()),
                                        sh_logit ? reinterpret_cast<const float *>(sh_logit->dev()) : nullptr,
                                        y_shared ? reinterpret_cast<const float *>(y_shared->dev()) : nullptr,
                                        residual ? reinterpret_cast<const float *>(residual->dev()) : nullptr,
                                        local_ids ? reinterpret_cast<const uint32_t *>(local_ids->dev()) : nullptr,
                                        reinterpret_cast<float *>(out->dev()), n_tokens, top_k, h, enc->stream),
             "moe_weighted_reduce launch");
    g_launches.fetch_add(1);
    g_dispatch.fetch_add(1);
    g_last_kernel = "moe_weighted_reduce";
    return MLXN_OK;
}

extern "C" int mlxn_moe_weighted_reduce(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *expert_w,
                                        mlxn_buffer *y_expert, mlxn_buffer *sh_logit, mlxn_buffer *y_shared,
                                        mlxn_buffer *residual, mlxn_buffer *out, uint32_t n_tokens, uint32_t top_k,
                                        uint32_t h) {
    return moe_weighted_reduce_impl(enc, reg, dev, expert_w, y_expert, sh_logit, y_shared, residual, nullptr, out, n_tokens,
                                    top_k, h);
}

// Expert-sharded form (no upstream counterpart): the partial sum over this rank's experts only.
extern "C" int mlxn_moe_weighted_reduce_local(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *expert_w,
                                              mlxn_buffer *y_expert, mlxn_buffer *local_ids, mlxn_buffer *out,
                                              uint32_t n_tokens, uint32_t top_k, uint32_t h) {
    if (!local_ids) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: moe_weighted_reduce_local: local_ids is null");
    return moe_weighted_reduce_impl(enc, reg, dev, expert_w, y_expert, nullptr, nullptr, nullptr, local_ids, out, n_tokens,
                                    top_k, h);
}

extern "C" int mlxn_moe_expert_shard_route(mlxn_encoder *enc, mlxn_registry *reg, mlxn_device *dev, mlxn_buffer *ids,
                                           mlxn_buffer *local_ids, uint32_t n_pairs, uint32_t expert_lo,
                                           uint32_t expert_count) {
    (void)reg;
    int rc = check_handles(enc, dev, {ids, local_ids});
    if (rc) return rc;
    if (n_pairs == 0 || expert_count == 0) return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: moe_expert_shard_route: n_pairs and expert_count must be > 0");
    if (ids->len < (size_t)n_pairs * 4 || local_ids->len < (size_t)n_pairs * 4)
        return fail(MLXN_INVALID_ARGUMENT, "Invalid argument: moe_expert_shard_route: a buffer is too small");
    if ((rc = op_begin(enc, {{ids, false}, {local_ids, true}}))) return rc;
    CUDA_TRY(launch_moe_expert_shard_route(reinterpret_cast<const uint32_t *>(ids->dev()),
                                           reinterpret_cast<uint32_t *>(local_ids->dev()), n_pairs, expert_lo, expert_count,
                                           enc->stream),
             "moe_expert_shard_route launch");
    g_launches.fetch_add(1);
    g_dispatch.fetch_add(1);
    g_last_kernel = "moe_expert_shard_route";
    return MLXN_OK;
}
