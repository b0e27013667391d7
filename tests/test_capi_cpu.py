"""CPU-only checks of the boundary: the shared library loads, exports every symbol the header declares,
and the host-side logic that needs no GPU behaves like upstream (src/lib.rs:283-308, src/dtypes.rs:56-77)."""
import ctypes
import os
import re
import subprocess

import pytest

import mlx_native_b200 as mx
from mlx_native_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "mlxn_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mlxn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_native.lib_path()) if os.path.exists(_native.lib_path()) else _native.lib()
    names = declared_symbols()
    assert len(names) > 60
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/mlxn_b200.h but not exported"
    # and the ctypes table binds exactly the declared set
    assert sorted(_native.SIGNATURES) == names


def test_header_compiles_as_c_and_cpp(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "mlxn_b200.h"\nint main(void){ mlxn_qmm_params p = {1,2,3,MLXN_GGML_Q4_0}; return (int)p.m - 1; }\n')
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", str(src), "-o",
                           str(tmp_path / "t.o")])
    subprocess.check_call(["g++", "-std=c++17", "-Wall", "-Werror", "-x", "c++", "-I", os.path.join(ROOT, "include"), "-c",
                           str(src), "-o", str(tmp_path / "t2.o")])
    assert ctypes.sizeof(_native.QmmParams) == 16 and ctypes.sizeof(_native.QmmIdParams) == 32
    # the ctypes mirrors have the C structs' sizes and field offsets (printed by a program compiled against the header)
    probe = tmp_path / "sizes.c"
    probe.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "mlxn_b200.h"\nint main(void){ printf("%zu %zu %zu %zu %zu %zu\\n", '
                     'sizeof(mlxn_qmm_params), sizeof(mlxn_qmm_id_params), offsetof(mlxn_qmm_id_params, expert_stride), '
                     'sizeof(mlxn_moe_ffn_params), offsetof(mlxn_moe_ffn_params, gate_stride), sizeof(mlxn_qmm_perm021_params)); return 0; }\n')
    exe = tmp_path / "sizes"
    subprocess.check_call(["gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), str(probe), "-o", str(exe)])
    got = [int(v) for v in subprocess.check_output([str(exe)]).split()]
    assert got == [ctypes.sizeof(_native.QmmParams), ctypes.sizeof(_native.QmmIdParams), _native.QmmIdParams.expert_stride.offset,
                   ctypes.sizeof(_native.MoeFfnParams), _native.MoeFfnParams.gate_stride.offset, ctypes.sizeof(_native.QmmPerm021Params)]


def test_block_geometry_and_dtypes():
    G = mx.GgmlType
    assert [(t.block_values(), t.block_bytes()) for t in (G.F32, G.F16, G.Q4_0, G.Q8_0, G.Q4_K, G.Q5_K, G.Q6_K, G.I16)] == \
        [(1, 4), (1, 2), (32, 18), (32, 34), (256, 144), (256, 176), (256, 210), (1, 2)]
    D = mx.DType
    assert [d.size_of() for d in (D.F32, D.F16, D.BF16, D.U8, D.U16, D.U32, D.I32)] == [4, 2, 2, 1, 2, 4, 4]
    assert D.BF16.name_str() == "bf16"
    assert mx.MM_ROUTING_THRESHOLD == 8 and mx.MM_ID_ROUTING_THRESHOLD == 32


def test_registry_names():
    r = mx.KernelRegistry.new()
    assert r.cached_count() == 0 and r.source_count() >= 20
    with pytest.raises(mx.KernelNotFound, match="Kernel not found: nonexistent_kernel"):
        r.get_pipeline("nonexistent_kernel")
    for name in ("kernel_mul_mv_q4_0_f32", "kernel_mul_mm_q6_K_tensor_f32", "kernel_mul_mv_id_q8_0_f32",
                 "kernel_mul_mm_id_map0_ne20_8", "kernel_mul_mm_id_q4_0_tensor_f32"):
        assert not r.is_cached(name)
        r.get_pipeline(name)
        assert r.is_cached(name)
    assert r.cached_count() == 5


def test_no_cpu_fallback_without_a_gpu():
    try:
        import torch

        if torch.cuda.is_available():
            pytest.skip("a GPU is present")
    except ImportError:
        pass
    with pytest.raises(mx.DeviceNotFound):
        mx.MlxDevice.new()
    assert not mx.DeviceNotFound("x").is_transient() and mx.CommandBufferError("x").is_transient()


def test_options_and_threshold_env():
    mx.set_option("qmv", "simple")
    mx.set_option("qmv", "stream")
    mx.set_option("qmv", "tc")
    mx.set_option("qmv", "auto")
    with pytest.raises(mx.InvalidArgument):
        mx.set_option("qmv", "cpu")
    with pytest.raises(mx.InvalidArgument):
        mx.set_option("nope", "1")
    code = "import mlx_native_b200 as mx; print(mx.mm_id_routing_threshold())"
    env = dict(os.environ, HF2Q_MM_ID_ROUTING_THRESHOLD="99999", PYTHONPATH=ROOT)
    assert subprocess.check_output(["python", "-c", code], env=env).strip() == b"99999"
    env["HF2Q_MM_ID_ROUTING_THRESHOLD"] = "junk"
    assert subprocess.check_output(["python", "-c", code], env=env).strip() == b"32"


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "mlx_native_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"
