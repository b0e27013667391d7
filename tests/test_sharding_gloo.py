"""The N-sharded multi-GPU path on CPU: two gloo ranks each run the oracle on their row shard, all-gather the
slices and must reproduce the single-rank result bit for bit (each output row is computed by exactly one rank)."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("ggml_type,n,k,m", [(3, 64, 256, 2), (6, 48, 768, 1), (2, 128, 128, 8)])
def test_two_rank_row_sharding_matches_single_rank(tmp_path, ggml_type, n, k, m):
    port = _free_port()
    worker = os.path.join(ROOT, "tests", "shard_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", str(port), str(ggml_type), str(n), str(k), str(m),
                               str(tmp_path)]) for r in range(2)]
    for p in procs:
        assert p.wait(timeout=300) == 0
    assert bool(np.load(tmp_path / "ok.npy")[0])


@pytest.mark.parametrize("T,E,top_k", [(5, 8, 2), (12, 16, 8)])
def test_two_rank_expert_sharding_matches_single_rank(tmp_path, T, E, top_k):
    port = _free_port()
    worker = os.path.join(ROOT, "tests", "shard_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", str(port), "moe", str(T), str(E), str(top_k),
                               str(tmp_path)]) for r in range(2)]
    for p in procs:
        assert p.wait(timeout=300) == 0
    assert bool(np.load(tmp_path / "ok.npy")[0])


@pytest.mark.parametrize("T,E,top_k,world", [(5, 8, 2, 2), (12, 16, 8, 2), (1, 8, 4, 2), (9, 12, 3, 3)])
def test_all_to_all_dispatch_combine_is_bit_identical_to_one_rank(tmp_path, T, E, top_k, world):
    port = _free_port()
    worker = os.path.join(ROOT, "tests", "shard_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), str(world), str(port), "moe_a2a", str(T), str(E), str(top_k),
                               str(tmp_path)]) for r in range(world)]
    for p in procs:
        assert p.wait(timeout=300) == 0
    assert bool(np.load(tmp_path / "ok.npy")[0])


def test_sharding_helpers_errors():
    sys.path.insert(0, ROOT)
    from mlx_native_b200 import sharding

    assert sharding.shard_rows(12288, 3, 8) == (4608, 6144)
    assert sharding.row_bytes(6, 5120) == 4200
    with pytest.raises(ValueError):
        sharding.shard_rows(10, 0, 3)
    with pytest.raises(ValueError):
        sharding.row_bytes(2, 48)
    assert sharding.shard_experts(128, 5, 8) == (80, 16)
    with pytest.raises(ValueError):
        sharding.shard_experts(10, 0, 4)
    assert sharding.local_expert_ids(np.array([0, 15, 16, 31, 32], np.uint32), 16, 16).tolist() == [
        sharding.NOT_LOCAL, sharding.NOT_LOCAL, 0, 15, sharding.NOT_LOCAL]
    g = np.arange(2 * 3 * 4, dtype=np.float32).reshape(2, 3, 4)
    a = sharding.assemble_gathered(g)
    assert a.shape == (3, 8) and a[1].tolist() == [4, 5, 6, 7, 16, 17, 18, 19]
