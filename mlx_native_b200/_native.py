"""ctypes binding of libmlxn_b200.so (the C ABI declared in include/mlxn_b200.h).

The library is never replaced by a CPU path: if it is missing it is built with nvcc, and if
that fails the import raises.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

_lib = None

vp, sz, i32, u32, u64 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_uint64
pvp = C.POINTER(C.c_void_p)


class QmmParams(C.Structure):
    _fields_ = [("m", u32), ("n", u32), ("k", u32), ("ggml_type", u32)]


class QmmPerm021Params(C.Structure):
    _fields_ = [("m", u32), ("n", u32), ("k", u32), ("head_dim", u32), ("ggml_type", u32)]


class QmmIdParams(C.Structure):
    _fields_ = [("n_tokens", u32), ("top_k", u32), ("n", u32), ("k", u32), ("n_experts", u32),
                ("ggml_type", u32), ("expert_stride", u64)]


class MoeFfnParams(C.Structure):
    _fields_ = [("n_tokens", u32), ("top_k", u32), ("hidden", u32), ("ffn", u32), ("n_experts", u32),
                ("gate_type", u32), ("up_type", u32), ("down_type", u32),
                ("gate_stride", u64), ("up_stride", u64), ("down_stride", u64)]


# name -> (restype, argtypes); this table is also what tests check against the header
SIGNATURES = {
    "mlxn_last_error_message": (C.c_char_p, []),
    "mlxn_status_is_transient": (i32, [i32]),
    "mlxn_dtype_size": (sz, [i32]),
    "mlxn_dtype_name": (C.c_char_p, [i32]),
    "mlxn_ggml_block_values": (u32, [i32]),
    "mlxn_ggml_block_bytes": (u32, [i32]),
    "mlxn_mm_id_routing_threshold": (u32, []),
    "mlxn_device_create": (i32, [i32, pvp]),
    "mlxn_device_destroy": (None, [vp]),
    "mlxn_device_name": (C.c_char_p, [vp]),
    "mlxn_device_ordinal": (i32, [vp]),
    "mlxn_device_sm_count": (i32, [vp]),
    "mlxn_buffer_alloc": (i32, [vp, sz, i32, C.POINTER(sz), sz, pvp]),
    "mlxn_buffer_wrap": (i32, [vp, vp, sz, i32, C.POINTER(sz), sz, pvp]),
    "mlxn_buffer_slice_view": (i32, [vp, u64, sz, pvp]),
    "mlxn_buffer_retain": (None, [vp]),
    "mlxn_buffer_release": (None, [vp]),
    "mlxn_buffer_dtype": (i32, [vp]),
    "mlxn_buffer_rank": (sz, [vp]),
    "mlxn_buffer_shape": (sz, [vp, sz]),
    "mlxn_buffer_byte_len": (sz, [vp]),
    "mlxn_buffer_element_count": (sz, [vp]),
    "mlxn_buffer_byte_offset": (u64, [vp]),
    "mlxn_buffer_device_ptr": (vp, [vp]),
    "mlxn_buffer_host_map": (i32, [vp, i32, pvp]),
    "mlxn_buffer_upload": (i32, [vp, vp, sz, sz]),
    "mlxn_buffer_download": (i32, [vp, vp, sz, sz]),
    "mlxn_pool_create": (i32, [pvp]),
    "mlxn_pool_destroy": (None, [vp]),
    "mlxn_pool_alloc": (i32, [vp, vp, sz, i32, C.POINTER(sz), sz, pvp]),
    "mlxn_pool_alloc_batch": (i32, [vp, vp, sz, C.POINTER(sz), C.POINTER(i32), C.POINTER(sz), C.POINTER(sz), pvp]),
    "mlxn_pool_release": (i32, [vp, vp]),
    "mlxn_pool_reset": (None, [vp]),
    "mlxn_pool_register_existing": (i32, [vp, vp, vp]),
    "mlxn_pool_free_count": (sz, [vp]),
    "mlxn_pool_free_bytes": (sz, [vp]),
    "mlxn_pool_in_use_count": (sz, [vp]),
    "mlxn_pool_clear": (None, [vp]),
    "mlxn_registry_create": (i32, [pvp]),
    "mlxn_registry_destroy": (None, [vp]),
    "mlxn_registry_get_pipeline": (i32, [vp, vp, C.c_char_p]),
    "mlxn_registry_is_cached": (i32, [vp, C.c_char_p]),
    "mlxn_registry_cached_count": (sz, [vp]),
    "mlxn_registry_source_count": (sz, [vp]),
    "mlxn_encoder_create": (i32, [vp, pvp]),
    "mlxn_encoder_destroy": (None, [vp]),
    "mlxn_encoder_memory_barrier": (i32, [vp]),
    "mlxn_encoder_commit": (i32, [vp]),
    "mlxn_encoder_wait_until_completed": (i32, [vp]),
    "mlxn_encoder_commit_and_wait": (i32, [vp]),
    "mlxn_encoder_commit_wait_with_gpu_time": (i32, [vp, C.POINTER(C.c_double)]),
    "mlxn_encoder_stream": (vp, [vp]),
    "mlxn_encoder_commit_labeled": (i32, [vp, C.c_char_p]),
    "mlxn_encoder_commit_and_wait_labeled": (i32, [vp, C.c_char_p]),
    "mlxn_profile_cb_get": (i32, [C.c_char_p, C.POINTER(u64), C.POINTER(u64)]),
    "mlxn_profile_cb_reset": (None, []),
    "mlxn_encoder_begin_capture": (i32, [vp]),
    "mlxn_encoder_end_capture": (i32, [vp, pvp]),
    "mlxn_graph_launch": (i32, [vp, vp]),
    "mlxn_graph_destroy": (None, [vp]),
    "mlxn_dispatch_count": (u64, []),
    "mlxn_sync_count": (u64, []),
    "mlxn_cmd_buf_count": (u64, []),
    "mlxn_barrier_count": (u64, []),
    "mlxn_reset_counters": (None, []),
    "mlxn_kernel_launch_count": (u64, []),
    "mlxn_quantized_matmul_ggml": (i32, [vp, vp, vp, vp, vp, vp, C.POINTER(QmmParams)]),
    "mlxn_quantized_matmul_ggml_sharded": (i32, [vp, vp, vp, vp, vp, vp, C.POINTER(QmmParams), C.c_uint32, C.c_uint32,
                                                 C.POINTER(C.c_void_p), C.c_uint32]),
    "mlxn_quantized_matmul_mm_tensor_perm021": (i32, [vp, vp, vp, vp, vp, vp, C.POINTER(QmmPerm021Params)]),
    "mlxn_dispatch_mm_for_test": (i32, [vp, vp, vp, vp, vp, vp, C.POINTER(QmmParams)]),
    "mlxn_quantized_matmul_id_ggml": (i32, [vp, vp, vp, vp, vp, vp, vp, C.POINTER(QmmIdParams)]),
    "mlxn_quantized_matmul_id_swiglu": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, C.POINTER(QmmIdParams)]),
    "mlxn_moe_ffn_layer": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, C.POINTER(MoeFfnParams)]),
    "mlxn_quantized_matmul_id_ggml_pooled": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32,
                                                   C.POINTER(QmmIdParams)]),
    "mlxn_dispatch_id_mm_for_test": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, C.POINTER(QmmIdParams)]),
    "mlxn_id_mm_htpe_bytes": (sz, [C.POINTER(QmmIdParams)]),
    "mlxn_id_mm_hids_bytes": (sz, [C.POINTER(QmmIdParams)]),
    "mlxn_moe_softmax_topk": (i32, [vp, vp, vp, vp, vp, vp, u32, u32, u32]),
    "mlxn_silu_mul": (i32, [vp, vp, vp, vp, vp, vp, u32]),
    "mlxn_moe_weighted_reduce": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32]),
    "mlxn_moe_weighted_reduce_local": (i32, [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32]),
    "mlxn_moe_expert_shard_route": (i32, [vp, vp, vp, vp, vp, u32, u32, u32]),
    "mlxn_noalloc_scratch_limit": (sz, []),
    "mlxn_quantized_matmul_ggml_mm_noalloc": (i32, [vp, vp, vp, vp, C.POINTER(QmmParams)]),
    "mlxn_peer_barrier": (i32, [vp, u32, u32, C.POINTER(C.c_void_p), u32, u32]),
    "mlxn_set_option": (i32, [C.c_char_p, C.c_char_p]),
    "mlxn_debug_wait_probe": (i32, [vp, u32]),
    "mlxn_last_kernel_name": (C.c_char_p, []),
}


def lib_path() -> str:
    return _build.LIB


def lib():
    """Loads (building first if needed) the CUDA library.  Raises if it cannot be built or loaded."""
    global _lib
    if _lib is None:
        if not os.path.exists(_build.LIB):
            _build.build()
        L = C.CDLL(_build.LIB)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib
