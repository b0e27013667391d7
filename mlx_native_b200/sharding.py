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


# ---------------------------------------------------------------------------------------------- all-to-all dispatch
class MoeAllToAll:
    """Token dispatch and combine of an expert-sharded MoE layer as two all-to-all exchanges (no counterpart in the
    reference, which runs on one GPU).

    Rank r owns the experts [r E/g, (r+1) E/g) and a slice of the tokens.  `plan` sorts this rank's (token, slot) pairs
    by the rank that owns their expert and exchanges the per-rank counts (one small all-to-all; the counts come to
    the host, because the data exchanges need their split sizes there).  `dispatch` sends every pair's activation row
    and local expert id to the owner; the owner runs gate / up / SwiGLU / down on what it received, one row per pair;
    `combine` sends the result rows back and puts them into the original pair order.  Nothing is reduced on the way:
    every pair's row is computed by exactly one rank with the same kernels as on one GPU, so after the weighted
    reduce over a token's slots the layer's output is bit-identical to the one-GPU layer.

    Works on any torch.distributed backend (NCCL on device tensors; gloo on CPU tensors in the tests)."""

    def __init__(self, n_experts: int, top_k: int, group=None):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if n_experts % self.world:
            raise ValueError(f"n_experts ({n_experts}) is not divisible by the number of ranks ({self.world})")
        self.per = n_experts // self.world
        self.top_k = top_k

    def plan(self, ids):
        """ids: integer tensor [n_local_tokens * top_k] of global expert ids.  Returns a dict with the send order, the
        split sizes of both directions and the local expert id of every pair in send order."""
        import torch

        ids = ids.reshape(-1).to(torch.int64)
        owner = torch.div(ids, self.per, rounding_mode="floor")
        order = torch.argsort(owner, stable=True)
        send_counts = torch.bincount(owner, minlength=self.world).to(torch.int64)
        recv_counts = torch.empty_like(send_counts)
        self.dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        return {"order": order, "send": [int(v) for v in send_counts.tolist()], "recv": [int(v) for v in recv_counts.tolist()],
                "local_ids": (ids[order] - owner[order] * self.per).to(torch.int32)}

    def dispatch(self, plan, x, out_rows=None, out_ids=None):
        """x: [n_local_tokens, hidden].  Returns (rows [P, hidden], local expert ids [P] int32) received by this rank,
        P = sum(plan["recv"]); `out_rows` / `out_ids` (capacity >= P) are used as the receive buffers if given."""
        import torch

        send_rows = x[torch.div(plan["order"], self.top_k, rounding_mode="floor")].contiguous()
        total = sum(plan["recv"])
        rows = out_rows[:total] if out_rows is not None else torch.empty((total, x.shape[1]), dtype=x.dtype, device=x.device)
        lids = out_ids[:total] if out_ids is not None else torch.empty((total,), dtype=torch.int32, device=x.device)
        self.dist.all_to_all_single(rows, send_rows, plan["recv"], plan["send"], group=self.group)
        self.dist.all_to_all_single(lids, plan["local_ids"].contiguous(), plan["recv"], plan["send"], group=self.group)
        return rows, lids

    def combine(self, plan, y, out=None):
        """y: [P, hidden] rows computed here, in receive order.  Returns [n_local_tokens * top_k, hidden] rows of this
        rank's pairs in their original (token, slot) order."""
        import torch

        n_pairs = plan["order"].numel()
        back = torch.empty((n_pairs, y.shape[1]), dtype=y.dtype, device=y.device)
        self.dist.all_to_all_single(back, y.contiguous(), plan["send"], plan["recv"], group=self.group)
        res = out if out is not None else torch.empty_like(back)
        res[plan["order"]] = back
        return res


class PeerBarrier:
    """The library's cross-rank barrier (mlxn_peer_barrier) over a flag array in torch symmetric memory: one object per
    process group, `wait(encoder)` enqueues one barrier behind everything the encoder holds.  Rendezvous (mapping the
    ranks' flag arrays into one another's address space) is torch's; the barrier itself is this library's kernel, with a
    bounded wait and plain peer loads / stores (multicast is switched off for the mapping)."""

    def __init__(self, device_index: int, group=None, limit_us: int = 2000000):
        import os

        import torch
        import torch.distributed as dist

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.flags = symm_mem.empty(max(self.world, 8), dtype=torch.int32, device=f"cuda:{device_index}")
        self.handle = symm_mem.rendezvous(self.flags, group if group is not None else dist.group.WORLD)
        self.flags.zero_()
        torch.cuda.synchronize()
        dist.barrier(group)                                     # every rank's flags are zero before anyone signals
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.epoch = 0
        self.limit_us = limit_us

    def wait(self, encoder) -> None:
        from . import api

        self.epoch += 1
        api.peer_barrier(encoder, self.rank, self.world, self.ptrs, self.epoch, self.limit_us)
