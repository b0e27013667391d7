"""The committed vectors of tests/golden/ (frozen oracle answers, see make_golden.py): the oracle must still give them
(CPU), and the CUDA path must give them within the parity bounds (GPU, through the C ABI)."""
import os

import numpy as np
import pytest

from oracle import oracle as orc

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "matmul_vectors.npz"))
CASES = [(t, c) for t in ("Q4_0", "Q8_0", "Q6_K") for c in ("lcg", "normal")]
OT = {"Q4_0": orc.Q4_0, "Q8_0": orc.Q8_0, "Q6_K": orc.Q6_K}


def shape_of(t, c):
    w, x = GOLD[f"{t}_{c}_w"], GOLD[f"{t}_{c}_x"]
    k = x.shape[1]
    return w, x, w.size // orc.row_bytes(OT[t], k), k


@pytest.mark.parametrize("t,c", CASES)
def test_oracle_reproduces_the_frozen_vectors(t, c):
    w, x, n, k = shape_of(t, c)
    y, ad = orc.qmatmul(OT[t], w, x, n, k)
    assert np.array_equal(y, GOLD[f"{t}_{c}_y"]) and np.array_equal(ad, GOLD[f"{t}_{c}_absdot"])


@pytest.mark.gpu
@pytest.mark.parametrize("qmv", ["auto", "mma", "tc", "stream", "simple"])
@pytest.mark.parametrize("t,c", CASES)
def test_cuda_matches_the_frozen_vectors(t, c, qmv):
    import mlx_native_b200 as mx
    from tests.gpu_util import MM_TOL, MV_TOL, TYPES, Ctx, norm_err

    w, x, n, k = shape_of(t, c)
    ctx = Ctx()
    mx.set_option("qmv", qmv)
    try:
        y = ctx.matmul(TYPES[t][0], w, x, n, k)
        assert norm_err(y, GOLD[f"{t}_{c}_y"], GOLD[f"{t}_{c}_absdot"]) <= MV_TOL
        if qmv == "auto":
            ymm = ctx.matmul(TYPES[t][0], w, x, n, k, force_mm=True)
            assert norm_err(ymm, GOLD[f"{t}_{c}_y"], GOLD[f"{t}_{c}_absdot"]) <= MM_TOL
    finally:
        mx.set_option("qmv", "auto")
