"""GGUF reader on the CPU: header / metadata / tensor table parsing, error cases (src/gguf/mod.rs:784-905), and the
host dequantizers against the oracle."""
import struct

import numpy as np
import pytest

from mlx_native_b200 import gguf
from mlx_native_b200.api import GgmlType
from oracle import oracle as orc
from tests.gguf_writer import write_gguf


def sample(tmp_path, alignment=None):
    rng = np.random.default_rng(0)
    w8 = orc.quantize(orc.Q8_0, (rng.standard_normal((16, 64)) * 0.02).astype(np.float32))
    w6 = orc.quantize(orc.Q6_K, (rng.standard_normal((4, 512)) * 0.02).astype(np.float32))
    wk = orc.quantize(orc.Q4_K, (rng.standard_normal((2, 4, 256)) * 0.02).astype(np.float32))
    f = rng.standard_normal((3, 5)).astype(np.float32)
    h = rng.standard_normal(7).astype(np.float16)
    path = tmp_path / "m.gguf"
    write_gguf(path, [("general.name", "str", "tiny"), ("llama.block_count", "u32", 2), ("x.small", "u8", 9),
                      ("x.neg", "i32", -4), ("x.eps", "f32", 1e-5), ("x.big", "f64", 2.5), ("x.flag", "bool", True),
                      ("x.list", "arr", ("str", ["a", "bc"])), ("x.n64", "u64", 1 << 40)],
               [("blk.0.w8", (16, 64), 8, w8), ("blk.0.w6", (4, 512), 14, w6), ("experts.wk", (2, 4, 256), 12, wk),
                ("norm.f32", (3, 5), 0, f), ("bias.f16", (7,), 1, h)], alignment=alignment)
    return path, dict(w8=w8, w6=w6, wk=wk, f=f, h=h)


@pytest.mark.parametrize("alignment", [None, 64, 8])
def test_parse_and_read(tmp_path, alignment):
    path, t = sample(tmp_path, alignment)
    with gguf.GgufFile.open(path) as g:
        assert g.tensor_count() == 5 and g.metadata_count() == (9 if alignment is None else 10)
        assert g.metadata_string("general.name") == "tiny" and g.metadata_string("llama.block_count") is None
        assert g.metadata_u32("llama.block_count") == 2 and g.metadata_u32("x.small") == 9
        assert g.metadata_u32("x.neg") is None and g.metadata_u32("x.n64") is None and g.metadata_u32("missing") is None
        assert g.metadata_f32("x.eps") == pytest.approx(1e-5) and g.metadata_f32("x.big") == 2.5
        assert g.metadata("x.flag") is True and g.metadata("x.list") == ["a", "bc"] and g.metadata("x.n64") == 1 << 40
        assert sorted(g.tensor_names()) == ["bias.f16", "blk.0.w6", "blk.0.w8", "experts.wk", "norm.f32"]
        i = g.tensor_info("blk.0.w6")
        assert i.shape == (4, 512) and i.ggml_type == GgmlType.Q6_K and i.byte_len == 4 * 2 * 210
        assert g.tensor_info("experts.wk").shape == (2, 4, 256) and g.tensor_info("nope") is None
        assert g.tensor_data_offset % (alignment or 32) == 0
        assert np.array_equal(g.read_tensor_bytes("blk.0.w8"), t["w8"])
        assert np.array_equal(g.read_tensor_bytes("experts.wk"), t["wk"])
        assert np.array_equal(g.read_tensor_bytes("norm.f32").view(np.float32), t["f"].reshape(-1))
        with pytest.raises(gguf.GgufParseError, match="not found"):
            g.read_tensor_bytes("nope")


@pytest.mark.parametrize("name,ot,gt", [("w8", orc.Q8_0, GgmlType.Q8_0), ("w6", orc.Q6_K, GgmlType.Q6_K), ("wk", orc.Q4_K, GgmlType.Q4_K)])
def test_host_dequantizers_match_oracle(tmp_path, name, ot, gt):
    _, t = sample(tmp_path)
    assert np.array_equal(gguf.dequantize_to_f32(t[name], gt), orc.dequantize(ot, t[name]))


def test_q4_0_and_float_dequantizers():
    rng = np.random.default_rng(1)
    w = orc.quantize(orc.Q4_0, (rng.standard_normal((8, 64)) * 0.02).astype(np.float32), rule="ggml")
    assert np.array_equal(gguf.dequantize_to_f32(w, GgmlType.Q4_0), orc.dequantize(orc.Q4_0, w))
    h = rng.standard_normal(9).astype(np.float16)
    assert np.array_equal(gguf.dequantize_to_f32(h.view(np.uint8), GgmlType.F16), h.astype(np.float32))


def test_q5_k_host_dequantizer_matches_the_oracle():
    rng = np.random.default_rng(5)
    blk = rng.integers(0, 256, (24, 176), dtype=np.uint8)
    blk[:, 0:2] = (rng.standard_normal(24) * 0.01).astype(np.float16).view(np.uint8).reshape(24, 2)
    blk[:, 2:4] = (rng.standard_normal(24) * 0.01).astype(np.float16).view(np.uint8).reshape(24, 2)
    got = gguf.dequantize_to_f32(blk.reshape(-1), GgmlType.Q5_K)
    assert np.array_equal(got, orc.dequantize(orc.Q5_K, blk.reshape(-1)))


def test_rejects_bad_files(tmp_path):
    with pytest.raises(gguf.IoError, match="cannot open"):
        gguf.GgufFile.open(tmp_path / "absent.gguf")
    p = tmp_path / "bad.gguf"
    write_gguf(p, [], [], magic=0x12345678)
    with pytest.raises(gguf.GgufParseError, match="bad magic"):
        gguf.GgufFile.open(p)
    write_gguf(p, [], [], version=2)
    with pytest.raises(gguf.GgufParseError, match="only v3"):
        gguf.GgufFile.open(p)
    write_gguf(p, [], [], alignment=24)
    with pytest.raises(gguf.GgufParseError, match="power of two"):
        gguf.GgufFile.open(p)
    write_gguf(p, [], [("t", (3, 40), 8, b"\0" * 8)])                 # 120 elements: not whole Q8_0 blocks
    with pytest.raises(gguf.GgufParseError, match="tensor 't'.*not divisible"):
        gguf.GgufFile.open(p)
    write_gguf(p, [], [("t", (32,), 99, b"\0" * 8)])
    with pytest.raises(gguf.GgufParseError, match="unsupported GGML type ID 99"):
        gguf.GgufFile.open(p)
    p.write_bytes(struct.pack("<IIQQ", 0x46554747, 3, 200_000, 0))
    with pytest.raises(gguf.GgufParseError, match="100k"):
        gguf.GgufFile.open(p)
    p.write_bytes(struct.pack("<IIQ", 0x46554747, 3, 1))             # truncated header
    with pytest.raises(gguf.GgufParseError, match="unexpected end of file"):
        gguf.GgufFile.open(p)
    write_gguf(p, [], [("t", (32,), 8, b"\0" * 10)])                  # data shorter than the table says
    with gguf.GgufFile.open(p) as g, pytest.raises(gguf.IoError, match="unexpected end of file"):
        g.read_tensor_bytes("t")
