"""The package's numpy block packers against the oracle's C packers (bit-exact) and its dequantizers."""
import numpy as np
import pytest

from mlx_native_b200 import ggml_pack as gp
from oracle import oracle as orc

PAIRS = [(orc.Q4_0, gp.Q4_0), (orc.Q8_0, gp.Q8_0), (orc.Q6_K, gp.Q6_K)]


@pytest.mark.parametrize("ot,gt", PAIRS)
def test_pack_matches_oracle_packer(ot, gt):
    rng = np.random.default_rng(5)
    v = (rng.standard_normal((48, 1024), dtype=np.float32) * np.float32(0.02))
    v[3, :256] = 0.0            # an all-zero block: d = 0, codes at the zero point
    v[7, 5] = 3.0               # an outlier
    v[9, :32] = -v[9, :32].__abs__()   # all-negative block
    assert np.array_equal(gp.pack(gt, v), orc.quantize(ot, v, rule="ggml"))


@pytest.mark.parametrize("ot,gt,tol", [(orc.Q4_0, gp.Q4_0, 1 / 7.5), (orc.Q8_0, gp.Q8_0, 1 / 200.0), (orc.Q6_K, gp.Q6_K, 1 / 20.0)])
def test_round_trip_error(ot, gt, tol):
    rng = np.random.default_rng(6)
    v = rng.standard_normal((8, 512), dtype=np.float32)
    back = orc.dequantize(ot, gp.pack(gt, v)).reshape(v.shape)
    amax = np.abs(v).reshape(-1, gp.BLOCK_VALUES[gt]).max(axis=1).repeat(gp.BLOCK_VALUES[gt]).reshape(v.shape)
    assert np.all(np.abs(back - v) <= tol * amax + 1e-6)


def test_rejects_ragged_and_unknown():
    with pytest.raises(ValueError):
        gp.pack(gp.Q6_K, np.zeros(100, dtype=np.float32))
    with pytest.raises(ValueError):
        gp.pack(4, np.zeros(256, dtype=np.float32))
