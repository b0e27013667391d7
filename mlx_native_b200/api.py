"""Host-side mirror of the mlx-native operator API for the GGML quantized matmul path.

Class, method and function names follow the upstream Rust crate (src/lib.rs:68-123) so that code
and tests written against it read the same here; every call goes through the C ABI in
include/mlxn_b200.h.  Errors are raised as MlxError subclasses named after the upstream enum
variants (src/error.rs:21-84).
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

import numpy as np

from . import _native
from ._native import QmmIdParams, QmmParams, QmmPerm021Params


# ---------------------------------------------------------------- errors (src/error.rs:21-89)
class MlxError(Exception):
    status = -1

    def is_transient(self) -> bool:
        return bool(_native.lib().mlxn_status_is_transient(self.status))


class DeviceNotFound(MlxError):
    status = 1


class CommandBufferError(MlxError):
    status = 2


class KernelNotFound(MlxError):
    status = 3


class BufferAllocationError(MlxError):
    status = 4


class InvalidArgument(MlxError):
    status = 5


class UnsupportedDtype(MlxError):
    status = 6


_ERRORS = {c.status: c for c in (DeviceNotFound, CommandBufferError, KernelNotFound, BufferAllocationError,
                                 InvalidArgument, UnsupportedDtype)}


def _check(rc: int) -> None:
    if rc != 0:
        msg = _native.lib().mlxn_last_error_message().decode("utf-8", "replace")
        raise _ERRORS.get(rc, MlxError)(msg)


# ---------------------------------------------------------------- DType (src/dtypes.rs:7-51)
class DType(enum.IntEnum):
    F32 = 0
    F16 = 1
    BF16 = 2
    U8 = 3
    U16 = 4
    U32 = 5
    I32 = 6

    def size_of(self) -> int:
        return int(_native.lib().mlxn_dtype_size(int(self)))

    def name_str(self) -> str:
        return _native.lib().mlxn_dtype_name(int(self)).decode()


_NP_DTYPES = {DType.F32: np.float32, DType.F16: np.float16, DType.U8: np.uint8, DType.U16: np.uint16,
              DType.U32: np.uint32, DType.I32: np.int32, DType.BF16: np.uint16}


# ---------------------------------------------------------------- GgmlType (src/ops/quantized_matmul_ggml.rs:48-100)
class GgmlType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q8_0 = 3
    Q4_K = 4
    Q5_K = 5
    Q6_K = 6
    I16 = 7

    def block_values(self) -> int:
        return int(_native.lib().mlxn_ggml_block_values(int(self)))

    def block_bytes(self) -> int:
        return int(_native.lib().mlxn_ggml_block_bytes(int(self)))


MM_ROUTING_THRESHOLD = 8      # src/ops/quantized_matmul_ggml.rs:180
MM_ID_ROUTING_THRESHOLD = 32  # src/ops/quantized_matmul_id_ggml.rs:397


def mm_id_routing_threshold() -> int:
    return int(_native.lib().mlxn_mm_id_routing_threshold())


@dataclass(frozen=True)
class GgmlQuantizedMatmulParams:      # src/ops/quantized_matmul_ggml.rs:183-194
    m: int
    n: int
    k: int
    ggml_type: GgmlType

    def _c(self) -> QmmParams:
        return QmmParams(self.m, self.n, self.k, int(self.ggml_type))


@dataclass(frozen=True)
class GgmlQuantizedMatmulPerm021Params:   # src/ops/quantized_matmul_ggml.rs:612-625
    m: int
    n: int
    k: int
    head_dim: int
    ggml_type: GgmlType

    def _c(self):
        return _native.QmmPerm021Params(self.m, self.n, self.k, self.head_dim, int(self.ggml_type))


@dataclass(frozen=True)
class GgmlQuantizedMatmulIdParams:    # src/ops/quantized_matmul_id_ggml.rs:44-61
    n_tokens: int
    top_k: int
    n: int
    k: int
    n_experts: int
    expert_stride: int
    ggml_type: GgmlType

    def _c(self) -> QmmIdParams:
        return QmmIdParams(self.n_tokens, self.top_k, self.n, self.k, self.n_experts, int(self.ggml_type),
                           self.expert_stride)


@dataclass(frozen=True)
class GgmlIdMmDispatchParams(GgmlQuantizedMatmulIdParams):   # src/ops/quantized_matmul_id_ggml.rs:850-879
    def htpe_bytes(self) -> int:
        return int(_native.lib().mlxn_id_mm_htpe_bytes(C.byref(self._c())))

    def hids_bytes(self) -> int:
        return int(_native.lib().mlxn_id_mm_hids_bytes(C.byref(self._c())))


# ---------------------------------------------------------------- device / buffer / pool
def _shape_arg(shape):
    shape = list(shape or [])
    arr = (C.c_size_t * max(len(shape), 1))(*shape) if shape else None
    return arr, len(shape)


class MlxBuffer:
    """Reference-counted handle onto device memory (src/buffer.rs:63-66)."""

    def __init__(self, handle: int):
        self._h = C.c_void_p(handle)

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _native.lib().mlxn_buffer_release(h)
            except Exception:
                pass
            self._h = None

    def clone(self) -> "MlxBuffer":
        _native.lib().mlxn_buffer_retain(self._h)
        return MlxBuffer(self._h.value)

    def dtype(self) -> DType:
        return DType(_native.lib().mlxn_buffer_dtype(self._h))

    def shape(self) -> list[int]:
        L = _native.lib()
        return [int(L.mlxn_buffer_shape(self._h, i)) for i in range(L.mlxn_buffer_rank(self._h))]

    def byte_len(self) -> int:
        return int(_native.lib().mlxn_buffer_byte_len(self._h))

    def element_count(self) -> int:
        return int(_native.lib().mlxn_buffer_element_count(self._h))

    def byte_offset(self) -> int:
        return int(_native.lib().mlxn_buffer_byte_offset(self._h))

    def contents_ptr(self) -> int:
        """Device address of the first byte (upstream returns a unified-memory pointer)."""
        return int(_native.lib().mlxn_buffer_device_ptr(self._h) or 0)

    def slice_view(self, byte_offset: int, n_elements: int) -> "MlxBuffer":
        out = C.c_void_p()
        _check(_native.lib().mlxn_buffer_slice_view(self._h, byte_offset, n_elements, C.byref(out)))
        return MlxBuffer(out.value)

    def _map(self, np_dtype, write: bool) -> np.ndarray:
        p = C.c_void_p()
        _check(_native.lib().mlxn_buffer_host_map(self._h, int(write), C.byref(p)))
        n = self.byte_len()
        raw = (C.c_uint8 * n).from_address(p.value)
        raw._owner = self  # the view keeps the buffer (and its pinned shadow) alive
        arr = np.frombuffer(raw, dtype=np.uint8).view(np_dtype)
        arr.flags.writeable = write
        return arr

    def as_slice(self, np_dtype=None) -> np.ndarray:
        """Read-only host view of the contents (src/buffer.rs:294-317): waits for device work on the
        buffer and downloads it if the device copy is newer."""
        return self._map(np_dtype or _NP_DTYPES[self.dtype()], False)

    def as_mut_slice(self, np_dtype=None) -> np.ndarray:
        """Writable host view (src/buffer.rs:324-348): what is written is uploaded by the next
        operation that binds the buffer."""
        return self._map(np_dtype or _NP_DTYPES[self.dtype()], True)

    def upload(self, data: np.ndarray, dst_offset: int = 0) -> None:
        a = np.ascontiguousarray(data)
        _check(_native.lib().mlxn_buffer_upload(self._h, a.ctypes.data_as(C.c_void_p), a.nbytes, dst_offset))

    def download(self, np_dtype=np.uint8, byte_len: int | None = None, src_offset: int = 0) -> np.ndarray:
        n = self.byte_len() - src_offset if byte_len is None else byte_len
        out = np.empty(n, dtype=np.uint8)
        _check(_native.lib().mlxn_buffer_download(self._h, out.ctypes.data_as(C.c_void_p), n, src_offset))
        return out.view(np_dtype)


class MlxDevice:
    """src/device.rs:22-26."""

    def __init__(self, ordinal: int = -1):
        out = C.c_void_p()
        _check(_native.lib().mlxn_device_create(ordinal, C.byref(out)))
        self._h = out

    @classmethod
    def new(cls, ordinal: int = -1) -> "MlxDevice":
        return cls(ordinal)

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _native.lib().mlxn_device_destroy(h)
            except Exception:
                pass
            self._h = None

    def name(self) -> str:
        return _native.lib().mlxn_device_name(self._h).decode()

    def ordinal(self) -> int:
        return int(_native.lib().mlxn_device_ordinal(self._h))

    def sm_count(self) -> int:
        return int(_native.lib().mlxn_device_sm_count(self._h))

    def alloc_buffer(self, byte_len: int, dtype: DType, shape=None) -> MlxBuffer:
        arr, rank = _shape_arg(shape)
        out = C.c_void_p()
        _check(_native.lib().mlxn_buffer_alloc(self._h, byte_len, int(dtype), arr, rank, C.byref(out)))
        return MlxBuffer(out.value)

    def wrap_device_memory(self, device_ptr: int, byte_len: int, dtype: DType, shape=None) -> MlxBuffer:
        """MlxBuffer::from_raw (src/buffer.rs:122) over memory owned by the caller (e.g. a torch tensor)."""
        arr, rank = _shape_arg(shape)
        out = C.c_void_p()
        _check(_native.lib().mlxn_buffer_wrap(self._h, C.c_void_p(device_ptr), byte_len, int(dtype), arr, rank,
                                              C.byref(out)))
        return MlxBuffer(out.value)

    def command_encoder(self) -> "CommandEncoder":
        return CommandEncoder(self)


class MlxBufferPool:
    """src/buffer_pool.rs:53-378."""

    def __init__(self):
        out = C.c_void_p()
        _check(_native.lib().mlxn_pool_create(C.byref(out)))
        self._h = out

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _native.lib().mlxn_pool_destroy(h)
            except Exception:
                pass
            self._h = None

    def alloc(self, device: MlxDevice, byte_len: int, dtype: DType, shape=None) -> MlxBuffer:
        arr, rank = _shape_arg(shape)
        out = C.c_void_p()
        _check(_native.lib().mlxn_pool_alloc(self._h, device._h, byte_len, int(dtype), arr, rank, C.byref(out)))
        return MlxBuffer(out.value)

    def alloc_batch(self, device: MlxDevice, requests) -> list[MlxBuffer]:
        """src/buffer_pool.rs:114-135: requests are (byte_len, dtype, shape) triples; all or nothing."""
        reqs = list(requests)
        n = len(reqs)
        lens = (C.c_size_t * max(n, 1))(*[int(r[0]) for r in reqs])
        dts = (C.c_int * max(n, 1))(*[int(r[1]) for r in reqs])
        shapes = [list(r[2]) if len(r) > 2 and r[2] is not None else [] for r in reqs]
        flat = [int(d) for sh in shapes for d in sh]
        flat_arr = (C.c_size_t * max(len(flat), 1))(*flat)
        ranks = (C.c_size_t * max(n, 1))(*[len(sh) for sh in shapes])
        outs = (C.c_void_p * max(n, 1))()
        _check(_native.lib().mlxn_pool_alloc_batch(self._h, device._h, n, lens, dts, flat_arr, ranks, outs))
        return [MlxBuffer(outs[i]) for i in range(n)]

    def release(self, buffer: MlxBuffer) -> None:
        h, buffer._h = buffer._h, None
        _check(_native.lib().mlxn_pool_release(self._h, h))

    def reset(self) -> None:
        _native.lib().mlxn_pool_reset(self._h)

    def register_existing(self, device: MlxDevice, buffer: MlxBuffer) -> None:
        _check(_native.lib().mlxn_pool_register_existing(self._h, device._h, buffer._h))

    def free_count(self) -> int:
        return int(_native.lib().mlxn_pool_free_count(self._h))

    def free_bytes(self) -> int:
        return int(_native.lib().mlxn_pool_free_bytes(self._h))

    def in_use_count(self) -> int:
        return int(_native.lib().mlxn_pool_in_use_count(self._h))

    def clear(self) -> None:
        _native.lib().mlxn_pool_clear(self._h)


class KernelRegistry:
    """src/kernel_registry.rs:37-44: a name table here, since kernels are compiled ahead of time."""

    def __init__(self):
        out = C.c_void_p()
        _check(_native.lib().mlxn_registry_create(C.byref(out)))
        self._h = out

    @classmethod
    def new(cls) -> "KernelRegistry":
        return cls()

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _native.lib().mlxn_registry_destroy(h)
            except Exception:
                pass
            self._h = None

    def get_pipeline(self, name: str, device: MlxDevice | None = None) -> str:
        _check(_native.lib().mlxn_registry_get_pipeline(self._h, device._h if device else None, name.encode()))
        return name

    def is_cached(self, name: str) -> bool:
        return bool(_native.lib().mlxn_registry_is_cached(self._h, name.encode()))

    def cached_count(self) -> int:
        return int(_native.lib().mlxn_registry_cached_count(self._h))

    def source_count(self) -> int:
        return int(_native.lib().mlxn_registry_source_count(self._h))


class CapturedGraph:
    def __init__(self, handle: int):
        self._h = C.c_void_p(handle)

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _native.lib().mlxn_graph_destroy(h)
            except Exception:
                pass
            self._h = None

    def launch(self, encoder: "CommandEncoder") -> None:
        _check(_native.lib().mlxn_graph_launch(self._h, encoder._h))


class CommandEncoder:
    """src/encoder.rs:507-591: one CUDA stream; operations run in encode order."""

    def __init__(self, device: MlxDevice):
        out = C.c_void_p()
        _check(_native.lib().mlxn_encoder_create(device._h, C.byref(out)))
        self._h = out
        self._device = device

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _native.lib().mlxn_encoder_destroy(h)
            except Exception:
                pass
            self._h = None

    def memory_barrier(self) -> None:
        _check(_native.lib().mlxn_encoder_memory_barrier(self._h))

    def commit(self) -> None:
        _check(_native.lib().mlxn_encoder_commit(self._h))

    def wait_until_completed(self) -> None:
        _check(_native.lib().mlxn_encoder_wait_until_completed(self._h))

    def commit_and_wait(self) -> None:
        _check(_native.lib().mlxn_encoder_commit_and_wait(self._h))

    def commit_and_wait_labeled(self, label: str) -> None:
        """src/encoder.rs:1893-1929: the label names an NVTX range; with MLX_PROFILE_CB=1 the command buffer's device
        time is recorded under it (profile_cb_get)."""
        _check(_native.lib().mlxn_encoder_commit_and_wait_labeled(self._h, label.encode()))

    def commit_labeled(self, label: str) -> None:
        _check(_native.lib().mlxn_encoder_commit_labeled(self._h, label.encode()))

    def debug_wait_probe(self, limit_us: int = 1000) -> None:
        """Enqueues the kernel whose bounded wait runs out (see mlxn_debug_wait_probe)."""
        _check(_native.lib().mlxn_debug_wait_probe(self._h, int(limit_us)))

    def commit_wait_with_gpu_time(self) -> float:
        t = C.c_double()
        _check(_native.lib().mlxn_encoder_commit_wait_with_gpu_time(self._h, C.byref(t)))
        return t.value

    def stream(self) -> int:
        return int(_native.lib().mlxn_encoder_stream(self._h) or 0)

    def begin_capture(self) -> None:
        _check(_native.lib().mlxn_encoder_begin_capture(self._h))

    def end_capture(self) -> CapturedGraph:
        out = C.c_void_p()
        _check(_native.lib().mlxn_encoder_end_capture(self._h, C.byref(out)))
        return CapturedGraph(out.value)


# ---------------------------------------------------------------- counters (src/encoder.rs:271-330)
def dispatch_count() -> int:
    return int(_native.lib().mlxn_dispatch_count())


def sync_count() -> int:
    return int(_native.lib().mlxn_sync_count())


def cmd_buf_count() -> int:
    return int(_native.lib().mlxn_cmd_buf_count())


def barrier_count() -> int:
    return int(_native.lib().mlxn_barrier_count())


def kernel_launch_count() -> int:
    return int(_native.lib().mlxn_kernel_launch_count())


def reset_counters() -> None:
    _native.lib().mlxn_reset_counters()


def set_option(key: str, value: str) -> None:
    _check(_native.lib().mlxn_set_option(key.encode(), value.encode()))


def last_kernel_name() -> str:
    return _native.lib().mlxn_last_kernel_name().decode()


def peer_barrier(encoder: "CommandEncoder", rank: int, world: int, flag_ptrs, epoch: int, limit_us: int = 2000000) -> None:
    """Cross-rank barrier over peer memory (see mlxn_peer_barrier): flag_ptrs[r] = device address of rank r's flag array
    (uint32[world], zero-initialised) as mapped into this process; `epoch` grows by one per barrier."""
    arr = (C.c_void_p * world)(*[C.c_void_p(int(p)) for p in flag_ptrs])
    _check(_native.lib().mlxn_peer_barrier(encoder._h, rank, world, arr, epoch & 0xFFFFFFFF, limit_us))


def profile_cb_get(label: str) -> tuple[int, int]:
    """(command buffers, device nanoseconds) recorded under `label` while MLX_PROFILE_CB=1 (src/kernel_profile.rs)."""
    n, ns = C.c_uint64(), C.c_uint64()
    _check(_native.lib().mlxn_profile_cb_get(label.encode(), C.byref(n), C.byref(ns)))
    return int(n.value), int(ns.value)


def profile_cb_reset() -> None:
    _native.lib().mlxn_profile_cb_reset()


# ---------------------------------------------------------------- the hot path
def _h(x):
    return x._h if x is not None else None


def quantized_matmul_ggml(encoder: CommandEncoder, registry: KernelRegistry | None, device: MlxDevice,
                          input: MlxBuffer, weight: MlxBuffer, output: MlxBuffer,
                          params: GgmlQuantizedMatmulParams) -> None:
    """src/ops/quantized_matmul_ggml.rs:267-361."""
    _check(_native.lib().mlxn_quantized_matmul_ggml(encoder._h, _h(registry), device._h, _h(input), _h(weight),
                                                    _h(output), C.byref(params._c())))


def quantized_matmul_ggml_sharded(encoder: CommandEncoder, registry: KernelRegistry | None, device: MlxDevice,
                                  input: MlxBuffer, weight: MlxBuffer, output: MlxBuffer,
                                  params: GgmlQuantizedMatmulParams, n_total: int, col0: int,
                                  peer_outputs: list[int] | tuple[int, ...] = ()) -> None:
    """Row-sharded mat-vec (m <= 8) for tensor parallelism; no counterpart upstream (single GPU).  `weight` holds
    params.n of the n_total rows (rows col0 .. col0 + n of the full matrix); `output` is this rank's full
    [m, n_total] result buffer.  The kernel stores its columns there and at the same place in every buffer of
    `peer_outputs` (device addresses of the other ranks' result buffers mapped into this process), so all ranks
    hold the whole result once every rank's kernel has finished; ordering between ranks is the caller's."""
    arr = (C.c_void_p * max(1, len(peer_outputs)))(*[C.c_void_p(p) for p in peer_outputs])
    _check(_native.lib().mlxn_quantized_matmul_ggml_sharded(encoder._h, _h(registry), device._h, _h(input), _h(weight),
                                                            _h(output), C.byref(params._c()), n_total, col0, arr,
                                                            len(peer_outputs)))


def dispatch_mm_for_test(encoder, registry, device, input, weight, output, params) -> None:
    """src/ops/quantized_matmul_ggml.rs:371-402."""
    _check(_native.lib().mlxn_dispatch_mm_for_test(encoder._h, _h(registry), device._h, _h(input), _h(weight),
                                                   _h(output), C.byref(params._c())))


def quantized_matmul_mm_tensor_perm021(encoder, registry, device, input_bf16, weight, output,
                                       params: GgmlQuantizedMatmulPerm021Params) -> None:
    """src/ops/quantized_matmul_ggml.rs:640-742: the mat-mat on bf16 activations laid out [n_heads, seq_len, head_dim]."""
    _check(_native.lib().mlxn_quantized_matmul_mm_tensor_perm021(encoder._h, _h(registry), device._h, _h(input_bf16),
                                                                 _h(weight), _h(output), C.byref(params._c())))


def noalloc_scratch_limit() -> int:
    return int(_native.lib().mlxn_noalloc_scratch_limit())


def quantized_matmul_ggml_mm_noalloc(cuda_stream: int, input_ptr: int, weight_ptr: int, output_ptr: int,
                                     params: GgmlQuantizedMatmulParams) -> None:
    """Tensor-core mat-mat on raw device pointers that allocates nothing (no counterpart upstream): for callers
    that may not allocate device memory — an allocator that owns all of HBM, a loop that must avoid the driver's
    allocation path, a plug-in that only gets pointers.  The packed activations live in a fixed 16 MiB array inside
    the library, so m*k is limited (see noalloc_scratch_limit) and overlapping calls on one GPU race."""
    _check(_native.lib().mlxn_quantized_matmul_ggml_mm_noalloc(C.c_void_p(cuda_stream), C.c_void_p(input_ptr),
                                                               C.c_void_p(weight_ptr), C.c_void_p(output_ptr),
                                                               C.byref(params._c())))


def quantized_matmul_id_ggml(encoder, registry, device, input, weight, ids, output,
                             params: GgmlQuantizedMatmulIdParams) -> None:
    """src/ops/quantized_matmul_id_ggml.rs:163-276."""
    _check(_native.lib().mlxn_quantized_matmul_id_ggml(encoder._h, _h(registry), device._h, _h(input), _h(weight),
                                                       _h(ids), _h(output), C.byref(params._c())))


def quantized_matmul_id_swiglu(encoder, registry, device, gate, up, weight, ids, output,
                               params: GgmlQuantizedMatmulIdParams) -> None:
    """Fused SwiGLU + expert-routed mat-vec for Q4_0, Q8_0 and Q6_K: output[r] = W[ids[r]] . (silu(gate[r]) * up[r]),
    gate / up f32 [n_tokens * top_k, k] (src/shaders/quantized_matmul_id_ggml.metal:231-319)."""
    _check(_native.lib().mlxn_quantized_matmul_id_swiglu(encoder._h, _h(registry), device._h, _h(gate), _h(up), _h(weight),
                                                         _h(ids), _h(output), C.byref(params._c())))


def quantized_matmul_id_swiglu_q4_0(encoder, registry, device, gate, up, weight, ids, output,
                                    params: GgmlQuantizedMatmulIdParams) -> None:
    """src/ops/quantized_matmul_id_ggml.rs:551-670 (Q4_0 only, as upstream)."""
    if params.ggml_type != GgmlType.Q4_0:
        raise InvalidArgument(f"Invalid argument: quantized_matmul_id_swiglu_q4_0: expected Q4_0, got {GgmlType(params.ggml_type).name}")
    quantized_matmul_id_swiglu(encoder, registry, device, gate, up, weight, ids, output, params)


@dataclass(frozen=True)
class MoeFfnLayerParams:
    """Shapes of one MoE FFN layer's expert half: gate / up are [n_experts][ffn][hidden], down is [n_experts][hidden][ffn];
    the strides are the bytes from one expert's matrix to the next."""
    n_tokens: int
    top_k: int
    hidden: int
    ffn: int
    n_experts: int
    gate_type: GgmlType
    up_type: GgmlType
    down_type: GgmlType
    gate_stride: int
    up_stride: int
    down_stride: int

    def _c(self) -> "_native.MoeFfnParams":
        return _native.MoeFfnParams(self.n_tokens, self.top_k, self.hidden, self.ffn, self.n_experts, int(self.gate_type),
                                    int(self.up_type), int(self.down_type), self.gate_stride, self.up_stride, self.down_stride)


def moe_ffn_layer(encoder, registry, device, x, ids, gate_w, up_w, down_w, gate_out, up_out, down_out,
                  params: MoeFfnLayerParams) -> None:
    """Gate and up projections, SwiGLU and down projection of the routed experts as one call, with the results of the chain
    quantized_matmul_id_ggml (gate), (up), silu_mul, quantized_matmul_id_ggml (down; n_tokens * top_k rows, top_k = 1) bit
    for bit (upstream encodes that chain call by call: benches/bench_mul_mm_id_qwen36_ffn.rs).  down_out holds one row per
    (token, slot) pair; gate_out and up_out are intermediates of [n_tokens * top_k, ffn] f32 each."""
    _check(_native.lib().mlxn_moe_ffn_layer(encoder._h, _h(registry), device._h, _h(x), _h(ids), _h(gate_w), _h(up_w), _h(down_w),
                                            _h(gate_out), _h(up_out), _h(down_out), C.byref(params._c())))


class IdMmScratch:
    """src/ops/quantized_matmul_id_ggml.rs:672-719."""

    def __init__(self, htpe: MlxBuffer, hids: MlxBuffer, n_experts_cap: int, n_tokens_cap: int):
        self.htpe, self.hids = htpe, hids
        self._n_experts_cap, self._n_tokens_cap = n_experts_cap, n_tokens_cap

    @classmethod
    def alloc(cls, device: MlxDevice, n_experts: int, max_n_tokens: int) -> "IdMmScratch":
        htpe = device.alloc_buffer(n_experts * 4, DType.U32, [n_experts])
        hids = device.alloc_buffer(n_experts * max_n_tokens * 4, DType.U32, [n_experts, max_n_tokens])
        return cls(htpe, hids, n_experts, max_n_tokens)


def quantized_matmul_id_ggml_pooled(encoder, registry, device, input, weight, ids, output, scratch: IdMmScratch,
                                    params: GgmlQuantizedMatmulIdParams) -> None:
    """src/ops/quantized_matmul_id_ggml.rs:288-389."""
    _check(_native.lib().mlxn_quantized_matmul_id_ggml_pooled(
        encoder._h, _h(registry), device._h, _h(input), _h(weight), _h(ids), _h(output), _h(scratch.htpe),
        _h(scratch.hids), scratch._n_experts_cap, scratch._n_tokens_cap, C.byref(params._c())))


def dispatch_id_mm_for_test(encoder, registry, device, input, weight, ids, htpe, hids, output, params) -> None:
    """src/ops/quantized_matmul_id_ggml.rs:902-1129."""
    _check(_native.lib().mlxn_dispatch_id_mm_for_test(encoder._h, _h(registry), device._h, _h(input), _h(weight),
                                                      _h(ids), _h(htpe), _h(hids), _h(output),
                                                      C.byref(params._c())))


def moe_softmax_topk(encoder, registry, device, logits, out_ids, out_weights, n_tokens, n_experts, top_k) -> None:
    """src/ops/moe_softmax_topk.rs:112-128."""
    _check(_native.lib().mlxn_moe_softmax_topk(encoder._h, _h(registry), device._h, _h(logits), _h(out_ids),
                                               _h(out_weights), n_tokens, n_experts, top_k))


def silu_mul(encoder, registry, device, gate, up, out, n) -> None:
    """src/ops/silu_mul.rs."""
    _check(_native.lib().mlxn_silu_mul(encoder._h, _h(registry), device._h, _h(gate), _h(up), _h(out), n))


def moe_weighted_reduce(encoder, registry, device, expert_w, y_expert, out, n_tokens, top_k, h, sh_logit=None,
                        y_shared=None, residual=None) -> None:
    """src/ops/moe_weighted_reduce.rs."""
    _check(_native.lib().mlxn_moe_weighted_reduce(encoder._h, _h(registry), device._h, _h(expert_w), _h(y_expert),
                                                  _h(sh_logit), _h(y_shared), _h(residual), _h(out), n_tokens, top_k,
                                                  h))


def moe_expert_shard_route(encoder, registry, device, ids, local_ids, n_pairs, expert_lo, expert_count) -> None:
    """Expert-sharded MoE (no upstream counterpart): global expert ids -> this rank's local ids, 0xFFFFFFFF for
    pairs whose expert lives on another rank."""
    _check(_native.lib().mlxn_moe_expert_shard_route(encoder._h, _h(registry), device._h, _h(ids), _h(local_ids),
                                                     n_pairs, expert_lo, expert_count))


def moe_weighted_reduce_local(encoder, registry, device, expert_w, y_expert, local_ids, out, n_tokens, top_k, h) -> None:
    """Partial `moe_weighted_reduce` over the pairs routed to this rank's experts; an all-reduce over the ranks'
    results completes the sum."""
    _check(_native.lib().mlxn_moe_weighted_reduce_local(encoder._h, _h(registry), device._h, _h(expert_w), _h(y_expert),
                                                        _h(local_ids), _h(out), n_tokens, top_k, h))


# ---------------------------------------------------------------- graph executor / session (src/graph.rs:862-941, 1029-1732)
class GraphSession:
    """A single-encoder session whose op methods delegate to the free functions (src/graph.rs:1135-1208)."""

    def __init__(self, device: MlxDevice):
        self._device = device
        self.encoder = device.command_encoder()
        self._barriers = 0

    def device(self) -> MlxDevice:
        return self._device

    def encoder_mut(self) -> CommandEncoder:
        return self.encoder

    def barrier(self) -> None:
        self.encoder.memory_barrier()
        self._barriers += 1

    def barrier_between(self, reads, writes) -> None:
        """src/graph.rs:1494-1530.  The buffer lists are not needed: the encoder itself tracks which storages the
        running group reads and writes and joins its lanes on a conflict; an explicit barrier is always safe."""
        self.barrier()

    def track_dispatch(self, reads, writes) -> None:
        """src/graph.rs:1532-1560.  A no-op for the same reason: every operation registers its buffers with the
        encoder's conflict tracking when it is encoded."""

    def barrier_count(self) -> int:
        return self._barriers

    def quantized_matmul_ggml(self, registry, device, input, weight, output, params) -> None:
        quantized_matmul_ggml(self.encoder, registry, device, input, weight, output, params)

    def quantized_matmul_id_ggml(self, registry, device, input, weight, ids, output, params) -> None:
        quantized_matmul_id_ggml(self.encoder, registry, device, input, weight, ids, output, params)

    def quantized_matmul_id_ggml_pooled(self, registry, device, input, weight, ids, output, scratch, params) -> None:
        quantized_matmul_id_ggml_pooled(self.encoder, registry, device, input, weight, ids, output, scratch, params)

    def commit(self) -> CommandEncoder:
        self.encoder.commit()
        return self.encoder

    def finish(self) -> None:
        self.encoder.commit_and_wait()

    def finish_with_gpu_time(self) -> float:
        return self.encoder.commit_wait_with_gpu_time()

    def finish_with_timing(self):
        import time

        t0 = time.perf_counter()
        self.encoder.commit()
        t1 = time.perf_counter()
        self.encoder.wait_until_completed()
        t2 = time.perf_counter()
        return (t1 - t0, t2 - t1)


class GraphExecutor:
    """src/graph.rs:862-941."""

    def __init__(self, device: MlxDevice):
        self._device = device

    @classmethod
    def new(cls, device: MlxDevice) -> "GraphExecutor":
        return cls(device)

    def device(self) -> MlxDevice:
        return self._device

    def begin(self) -> GraphSession:
        return GraphSession(self._device)
