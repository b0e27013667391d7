"""One gloo rank of tests/test_sharding_gloo.py: python shard_worker.py rank world port ggml_type n k m out_dir"""
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



if __name__ == "__main__":
    a = sys.argv[1:]
    main(int(a[0]), int(a[1]), int(a[2]), int(a[3]), int(a[4]), int(a[5]), int(a[6]), a[7])
