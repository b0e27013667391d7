"""bf16 "perm021" mat-mat (upstream quantized_matmul_mm_tensor_perm021, src/ops/quantized_matmul_ggml.rs:640-742): the
O-projection on the attention output where it lies, bf16 [n_heads, seq_len, head_dim], against the oracle on the permuted
f32 copy (the pair of operations the upstream kernel replaced: permute_021_bf16_to_f32 + the f32-input mat-mat)."""
import numpy as np
import pytest

import mlx_native_b200 as mx
from oracle import oracle as orc
from tests.gpu_util import MM_TOL, TYPES, Ctx, norm_err, normal_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns, round to nearest even (finite inputs)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize("tname,m,n,n_heads,head_dim", [("Q4_0", 64, 256, 4, 64), ("Q6_K", 40, 192, 2, 128), ("Q4_0", 1, 64, 8, 32),
                                                        ("Q6_K", 300, 512, 8, 256), ("Q4_0", 2455 % 700 + 9, 320, 16, 128)])
def test_perm021_matches_permute_then_matmul(ctx, tname, m, n, n_heads, head_dim):
    gtype, otype = TYPES[tname]
    k = n_heads * head_dim
    w = normal_weights(900 + m, n, k, otype)
    rng = np.random.default_rng(m * 7 + n)
    att = to_bf16_bits(rng.standard_normal((n_heads, m, head_dim)).astype(np.float32))      # [heads, seq, head_dim]
    x = from_bf16_bits(att).transpose(1, 0, 2).reshape(m, k).copy()                          # the permuted f32 copy
    d = ctx.device
    inp = d.alloc_buffer(att.nbytes, mx.DType.BF16, [n_heads, m, head_dim])
    inp.upload(att)
    out = d.alloc_buffer(m * n * 4, mx.DType.F32, [m, n])
    enc = d.command_encoder()
    mx.quantized_matmul_mm_tensor_perm021(enc, ctx.registry, d, inp, ctx.buf(w, mx.DType.U8), out,
                                          mx.GgmlQuantizedMatmulPerm021Params(m, n, k, head_dim, gtype))
    enc.commit_and_wait()
    assert mx.last_kernel_name() == "qmm_tc"
    y = out.as_slice(np.float32).reshape(m, n)
    y_ref, ad = orc.qmatmul(otype, w, x, n, k, nthreads=8)
    assert norm_err(y, y_ref, ad) <= MM_TOL
    # the same f16 operands as the f32-input mat-mat on the permuted copy (the cast chain bf16 -> f32 -> f16 is the same):
    # equal up to the order in which K halves of a split tile are added
    y2 = ctx.matmul(gtype, w, x, n, k, force_mm=True)
    assert norm_err(y, y2, ad) <= 1e-6


def test_perm021_argument_errors(ctx):
    d = ctx.device
    w = ctx.buf(normal_weights(1, 64, 256, TYPES["Q4_0"][1]), mx.DType.U8)
    inp = d.alloc_buffer(8 * 256 * 2, mx.DType.BF16)
    out = d.alloc_buffer(8 * 64 * 4, mx.DType.F32)

    def call(p, i=inp, o=out):
        mx.quantized_matmul_mm_tensor_perm021(d.command_encoder(), ctx.registry, d, i, w, o, p)

    P = mx.GgmlQuantizedMatmulPerm021Params
    with pytest.raises(mx.InvalidArgument, match="only Q4_0 and Q6_K are instantiated"):
        call(P(8, 64, 256, 64, mx.GgmlType.Q8_0))
    with pytest.raises(mx.InvalidArgument, match="head_dim 48 must be a positive multiple of 32"):
        call(P(8, 64, 256, 48, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match=r"k \(256\) must be divisible by head_dim \(96\)"):
        call(P(8, 64, 256, 96, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match="input_bf16 buffer too small"):
        call(P(9, 64, 256, 64, mx.GgmlType.Q4_0))
    with pytest.raises(mx.InvalidArgument, match="output buffer too small"):
        call(P(8, 64, 256, 64, mx.GgmlType.Q4_0), o=d.alloc_buffer(16, mx.DType.F32))
