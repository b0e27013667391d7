"""One gloo rank of tests/test_sharding_gloo.py:
  python shard_worker.py rank world port ggml_type n k m out_dir        row-sharded mat-vec + all-gather
  python shard_worker.py rank world port moe T E top_k out_dir          expert-sharded MoE FFN layer + all-reduce
  python shard_worker.py rank world port moe_a2a T E top_k out_dir      the same with all-to-all dispatch / combine"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def main(rank, world, port, ggml_type, n, k, m, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from mlx_native_b200 import sharding
    from oracle import oracle as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)                       # same data on every rank
    wq = orc.quantize(ggml_type, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    x = rng.standard_normal((m, k)).astype(np.float32)
    w_loc = sharding.shard_weight_bytes(wq, ggml_type, n, k, rank, world)
    lo, hi = sharding.shard_rows(n, rank, world)
    y_loc, _ = orc.qmatmul(ggml_type, w_loc, x, hi - lo, k)
    y_all = torch.empty((world * m, hi - lo), dtype=torch.float32)   # concatenation along dim 0
    dist.all_gather_into_tensor(y_all, torch.from_numpy(y_loc))
    y = sharding.assemble_gathered(y_all.numpy().reshape(world, m, hi - lo))
    if rank == 0:
        y_ref, _ = orc.qmatmul(ggml_type, wq, x, n, k)
        np.save(os.path.join(out_dir, "ok.npy"), np.array([np.array_equal(y, y_ref)]))
    dist.barrier()
    dist.destroy_process_group()



def main_moe(rank, world, port, T, E, top_k, out_dir):
    """Every rank runs the oracle on the (token, slot) pairs routed to its experts only, with its slice of the
    stacked expert weights and local ids; the all-reduce of the partial combines must give the one-rank layer."""
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from mlx_native_b200 import sharding
    from oracle import oracle as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    hidden, ffn = 256, 256
    rng = np.random.default_rng(1)                       # same data on every rank
    wg = orc.quantize(orc.Q4_0, (rng.standard_normal((E * ffn, hidden)) * 0.02).astype(np.float32), rule="ggml")
    wu = orc.quantize(orc.Q4_0, (rng.standard_normal((E * ffn, hidden)) * 0.02).astype(np.float32), rule="ggml")
    wd = orc.quantize(orc.Q6_K, (rng.standard_normal((E * hidden, ffn)) * 0.02).astype(np.float32))
    x = rng.standard_normal((T, hidden)).astype(np.float32)
    ids, rw = orc.moe_softmax_topk(rng.standard_normal((T, E)).astype(np.float32), top_k)
    flat = ids.reshape(-1)

    lo, cnt = sharding.shard_experts(E, rank, world)
    lids = sharding.local_expert_ids(flat, lo, cnt)
    mine = np.nonzero(lids != sharding.NOT_LOCAL)[0]
    sg, su, sd = wg.size // E, wu.size // E, wd.size // E
    wg_l = sharding.shard_expert_bytes(wg, sg, E, rank, world)
    wu_l = sharding.shard_expert_bytes(wu, su, E, rank, world)
    wd_l = sharding.shard_expert_bytes(wd, sd, E, rank, world)
    yd = np.zeros((T * top_k, hidden), dtype=np.float32)
    if mine.size:
        xs = x[mine // top_k]
        g, _ = orc.qmatmul_id(orc.Q4_0, wg_l, sg, xs, lids[mine], 1, ffn, hidden, cnt)
        u, _ = orc.qmatmul_id(orc.Q4_0, wu_l, su, xs, lids[mine], 1, ffn, hidden, cnt)
        dn, _ = orc.qmatmul_id(orc.Q6_K, wd_l, sd, orc.silu_mul(g, u), lids[mine], 1, hidden, ffn, cnt)
        yd[mine] = dn
    w_loc = np.where((lids != sharding.NOT_LOCAL).reshape(T, top_k), rw, np.float32(0.0)).astype(np.float32)
    part = torch.from_numpy(orc.moe_weighted_reduce(yd, w_loc, T, top_k, hidden).copy())
    dist.all_reduce(part)                                # the combine step
    # every pair belongs to exactly one rank
    owned = torch.from_numpy((lids != sharding.NOT_LOCAL).astype(np.int32))
    dist.all_reduce(owned)
    if rank == 0:
        g, _ = orc.qmatmul_id(orc.Q4_0, wg, sg, x, flat, top_k, ffn, hidden, E)
        u, _ = orc.qmatmul_id(orc.Q4_0, wu, su, x, flat, top_k, ffn, hidden, E)
        dn, _ = orc.qmatmul_id(orc.Q6_K, wd, sd, orc.silu_mul(g, u), flat, 1, hidden, ffn, E)
        want = orc.moe_weighted_reduce(dn, rw, T, top_k, hidden)
        ok = bool((owned.numpy() == 1).all()) and float(np.max(np.abs(part.numpy() - want))) <= 1e-5 * float(np.abs(want).max())
        np.save(os.path.join(out_dir, "ok.npy"), np.array([ok]))
    dist.barrier()
    dist.destroy_process_group()


def main_moe_a2a(rank, world, port, T, E, top_k, out_dir):
    """Token-sharded input, expert-sharded weights, all-to-all dispatch and combine (sharding.MoeAllToAll) with the
    oracle as the expert compute: the gathered layer output must equal the one-rank layer bit for bit."""
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from mlx_native_b200 import sharding
    from oracle import oracle as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    hidden, ffn = 256, 256
    rng = np.random.default_rng(2)                       # same data on every rank
    wg = orc.quantize(orc.Q4_0, (rng.standard_normal((E * ffn, hidden)) * 0.02).astype(np.float32), rule="ggml")
    wu = orc.quantize(orc.Q4_0, (rng.standard_normal((E * ffn, hidden)) * 0.02).astype(np.float32), rule="ggml")
    wd = orc.quantize(orc.Q6_K, (rng.standard_normal((E * hidden, ffn)) * 0.02).astype(np.float32))
    x = rng.standard_normal((T, hidden)).astype(np.float32)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    sg, su, sd = wg.size // E, wu.size // E, wd.size // E
    lo, cnt = sharding.shard_experts(E, rank, world)
    wg_l = sharding.shard_expert_bytes(wg, sg, E, rank, world)
    wu_l = sharding.shard_expert_bytes(wu, su, E, rank, world)
    wd_l = sharding.shard_expert_bytes(wd, sd, E, rank, world)
    # this rank's tokens: a contiguous slice (uneven on purpose when T % world != 0)
    t_lo, t_hi = T * rank // world, T * (rank + 1) // world
    ids_l, rw_l = orc.moe_softmax_topk(logits[t_lo:t_hi], top_k) if t_hi > t_lo else (np.zeros((0, top_k), np.uint32), np.zeros((0, top_k), np.float32))
    a2a = sharding.MoeAllToAll(E, top_k)
    plan = a2a.plan(torch.from_numpy(ids_l.astype(np.int64).reshape(-1)))
    rows, lids = a2a.dispatch(plan, torch.from_numpy(x[t_lo:t_hi].copy()))
    P = rows.shape[0]
    if P:
        li = lids.numpy().astype(np.uint32)
        g, _ = orc.qmatmul_id(orc.Q4_0, wg_l, sg, rows.numpy(), li, 1, ffn, hidden, cnt)
        u, _ = orc.qmatmul_id(orc.Q4_0, wu_l, su, rows.numpy(), li, 1, ffn, hidden, cnt)
        dn, _ = orc.qmatmul_id(orc.Q6_K, wd_l, sd, orc.silu_mul(g, u), li, 1, hidden, ffn, cnt)
    else:
        dn = np.zeros((0, hidden), np.float32)
    y_pairs = a2a.combine(plan, torch.from_numpy(np.ascontiguousarray(dn))).numpy()
    out_l = orc.moe_weighted_reduce(y_pairs, rw_l, t_hi - t_lo, top_k, hidden) if t_hi > t_lo else np.zeros((0, hidden), np.float32)
    gathered = [None] * world
    dist.all_gather_object(gathered, out_l)
    if rank == 0:
        ids, rw = orc.moe_softmax_topk(logits, top_k)
        flat = ids.reshape(-1)
        g, _ = orc.qmatmul_id(orc.Q4_0, wg, sg, x, flat, top_k, ffn, hidden, E)
        u, _ = orc.qmatmul_id(orc.Q4_0, wu, su, x, flat, top_k, ffn, hidden, E)
        dn, _ = orc.qmatmul_id(orc.Q6_K, wd, sd, orc.silu_mul(g, u), flat, 1, hidden, ffn, E)
        want = orc.moe_weighted_reduce(dn, rw, T, top_k, hidden)
        got = np.concatenate(gathered, axis=0)
        np.save(os.path.join(out_dir, "ok.npy"), np.array([got.shape == want.shape and np.array_equal(got, want)]))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    a = sys.argv[1:]
    if a[3] == "moe_a2a":
        main_moe_a2a(int(a[0]), int(a[1]), int(a[2]), int(a[4]), int(a[5]), int(a[6]), a[7])
        sys.exit(0)
    if a[3] == "moe":
        main_moe(int(a[0]), int(a[1]), int(a[2]), int(a[4]), int(a[5]), int(a[6]), a[7])
        sys.exit(0)
    main(int(a[0]), int(a[1]), int(a[2]), int(a[3]), int(a[4]), int(a[5]), int(a[6]), a[7])
