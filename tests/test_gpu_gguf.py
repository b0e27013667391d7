"""Weights loaded from a GGUF file straight into device buffers and consumed by the matmul kernels: whole tensors,
the row shard of a matrix and the expert shard of a stacked tensor, and the host-dequantized F32 load."""
import numpy as np
import pytest

import mlx_native_b200 as mx
from mlx_native_b200 import gguf, sharding
from oracle import oracle as orc
from tests.gguf_writer import write_gguf
from tests.gpu_util import MV_TOL, Ctx, norm_err, normal_acts, normal_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    n, k, E, ne, ke = 256, 512, 4, 64, 256
    t = dict(w8=normal_weights(1, n, k, orc.Q8_0), w6=normal_weights(2, n, k, orc.Q6_K),
             ex=normal_weights(3, E * ne, ke, orc.Q4_0), nf=normal_acts(4, 3, 8))
    path = tmp_path_factory.mktemp("gguf") / "tiny.gguf"
    write_gguf(path, [("general.architecture", "str", "test")],
               [("blk.0.ffn_up.weight", (n, k), 8, t["w8"]), ("output.weight", (n, k), 14, t["w6"]),
                ("blk.0.ffn_gate_exps.weight", (E, ne, ke), 2, t["ex"]), ("norm.weight", (3, 8), 0, t["nf"])])
    return path, t, (n, k, E, ne, ke)


def test_load_tensor_and_matvec(ctx, model):
    path, t, (n, k, *_rest) = model
    x = normal_acts(9, 2, k)
    with gguf.GgufFile.open(path) as g:
        for name, key, gt, ot in (("blk.0.ffn_up.weight", "w8", mx.GgmlType.Q8_0, orc.Q8_0),
                                  ("output.weight", "w6", mx.GgmlType.Q6_K, orc.Q6_K)):
            wb = g.load_tensor(name, ctx.device)
            assert wb.dtype() == mx.DType.U8 and list(wb.shape()) == [n, k] and wb.byte_len() == t[key].size
            assert np.array_equal(wb.as_slice(np.uint8), t[key])
            y = ctx.matmul(gt, None, x, n, k, weight_buf=wb)
            y_ref, ad = orc.qmatmul(ot, t[key], x, n, k)
            assert norm_err(y, y_ref, ad) <= MV_TOL
        nb = g.load_tensor("norm.weight", ctx.device)
        assert nb.dtype() == mx.DType.F32 and np.array_equal(nb.as_slice(np.float32).reshape(3, 8), t["nf"])
        fb = g.load_tensor_f32("output.weight", ctx.device)
        assert fb.dtype() == mx.DType.F32 and list(fb.shape()) == [n, k]
        assert np.array_equal(fb.as_slice(np.float32), orc.dequantize(orc.Q6_K, t["w6"]))
        with pytest.raises(gguf.GgufParseError, match="not found"):
            g.load_tensor("missing", ctx.device)
        # src/gguf/mod.rs:1127-1137: the loaded buffer is also registered with the pool
        pool = mx.MlxBufferPool()
        pb = g.load_tensor_into_pool("output.weight", ctx.device, pool)
        assert np.array_equal(pb.as_slice(np.uint8), t["w6"])
        with pytest.raises(gguf.GgufParseError, match="not found"):
            g.load_tensor_into_pool("missing", ctx.device, pool)


def test_sharded_loads(ctx, model):
    path, t, (n, k, E, ne, ke) = model
    with gguf.GgufFile.open(path) as g:
        for r in range(4):
            wb = g.load_tensor_rows("output.weight", ctx.device, r, 4)
            assert list(wb.shape()) == [n // 4, k]
            assert np.array_equal(wb.as_slice(np.uint8), sharding.shard_weight_bytes(t["w6"], 6, n, k, r, 4))
        for r in range(2):
            eb = g.load_tensor_experts("blk.0.ffn_gate_exps.weight", ctx.device, r, 2)
            assert list(eb.shape()) == [E // 2, ne, ke]
            assert np.array_equal(eb.as_slice(np.uint8), sharding.shard_expert_bytes(t["ex"], t["ex"].size // E, E, r, 2))
        with pytest.raises(gguf.GgufParseError, match="cannot be split"):
            g.load_tensor_rows("output.weight", ctx.device, 0, 3)
        with pytest.raises(gguf.GgufParseError, match="not a matrix"):
            g.load_tensor_rows("blk.0.ffn_gate_exps.weight", ctx.device, 0, 2)
