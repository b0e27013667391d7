"""Row (N) sharding of GGML weight matrices across GPUs and assembly of the gathered outputs.

Weights are row-major blocks, so the rows [r*n/g, (r+1)*n/g) of rank r are one contiguous byte range.
Each rank computes y_r = x * W_r^T of shape [m, n/g]; an all-gather yields [g, m, n/g], which
`assemble_gathered` turns back into [m, n].
"""
from __future__ import annotations

import numpy as np

BLOCK = {2: (32, 18), 3: (32, 34), 6: (256, 210)}  # ggml type code -> (values per block, bytes per block)


def row_bytes(ggml_type: int, k: int) -> int:
    qk, bb = BLOCK[int(ggml_type)]
    if k % qk:
        raise ValueError(f"K ({k}) must be divisible by block QK ({qk})")
    return k // qk * bb


def shard_rows(n: int, rank: int, world: int) -> tuple[int, int]:
    """Row range [lo, hi) of `rank`; n must divide evenly (all benchmark shapes do)."""
    if n % world:
        raise ValueError(f"N ({n}) is not divisible by the number of ranks ({world})")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_weight_bytes(wq: np.ndarray, ggml_type: int, n: int, k: int, rank: int, world: int) -> np.ndarray:
    lo, hi = shard_rows(n, rank, world)
    rb = row_bytes(ggml_type, k)
    flat = np.ascontiguousarray(wq, dtype=np.uint8).reshape(-1)
    if flat.size < n * rb:
        raise ValueError("weight buffer too small for [n, k]")
    return flat[lo * rb:hi * rb]


def assemble_gathered(gathered: np.ndarray) -> np.ndarray:
    """[g, m, n/g] -> [m, n]"""
    g, m, per = gathered.shape
    return np.ascontiguousarray(np.transpose(gathered, (1, 0, 2))).reshape(m, g * per)


# ---------------------------------------------------------------------------------------------- expert sharding
NOT_LOCAL = 0xFFFFFFFF  # id of a (token, slot) pair whose expert lives on another rank


def shard_experts(n_experts: int, rank: int, world: int) -> tuple[int, int]:
    """(first expert, count) of `rank`: contiguous blocks of n_experts / world experts."""
    if n_experts % world:
        raise ValueError(f"n_experts ({n_experts}) is not divisible by the number of ranks ({world})")
    per = n_experts // world
    return rank * per, per


def shard_expert_bytes(wq: np.ndarray, expert_stride: int, n_experts: int, rank: int, world: int) -> np.ndarray:
    """The stacked expert weights [n_experts][expert_stride bytes] of `rank`'s experts (one contiguous byte range)."""
    lo, cnt = shard_experts(n_experts, rank, world)
    flat = np.ascontiguousarray(wq, dtype=np.uint8).reshape(-1)
    if flat.size < n_experts * expert_stride:
        raise ValueError("weight buffer too small for [n_experts, expert_stride]")
    return flat[lo * expert_stride:(lo + cnt) * expert_stride]


def local_expert_ids(ids: np.ndarray, lo: int, count: int) -> np.ndarray:
    """Host mirror of `moe_expert_shard_route`: global ids -> local ids, NOT_LOCAL for other ranks' experts."""
    ids = np.asarray(ids, dtype=np.uint32)
    mine = (ids >= lo) & (ids < lo + count)
    return np.where(mine, ids - np.uint32(lo), np.uint32(NOT_LOCAL)).astype(np.uint32)
