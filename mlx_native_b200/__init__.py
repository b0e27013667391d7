"""B200 (sm_100a) implementation of mlx-native's GGML block-quantized matmul path.

The public names mirror the upstream crate's re-exports for this path (src/lib.rs:102-113).
"""
from .api import (  # noqa: F401
    MM_ID_ROUTING_THRESHOLD, MM_ROUTING_THRESHOLD, BufferAllocationError, CapturedGraph, CommandBufferError,
    CommandEncoder, DeviceNotFound, DType, GgmlIdMmDispatchParams, GgmlQuantizedMatmulIdParams,
    GgmlQuantizedMatmulParams, GgmlQuantizedMatmulPerm021Params, GgmlType, GraphExecutor, GraphSession, IdMmScratch, InvalidArgument, KernelNotFound,
    KernelRegistry, MlxBuffer, MlxBufferPool, MlxDevice, MlxError, UnsupportedDtype, barrier_count, cmd_buf_count,
    dispatch_count, dispatch_id_mm_for_test, dispatch_mm_for_test, kernel_launch_count, last_kernel_name,
    mm_id_routing_threshold, moe_softmax_topk, moe_expert_shard_route, moe_weighted_reduce_local, noalloc_scratch_limit, quantized_matmul_ggml_mm_noalloc, moe_weighted_reduce, quantized_matmul_ggml, quantized_matmul_mm_tensor_perm021, quantized_matmul_ggml_sharded, quantized_matmul_id_ggml,
    quantized_matmul_id_ggml_pooled, quantized_matmul_id_swiglu, quantized_matmul_id_swiglu_q4_0, moe_ffn_layer, MoeFfnLayerParams, peer_barrier, profile_cb_get, profile_cb_reset, reset_counters, set_option, silu_mul, sync_count,
)
