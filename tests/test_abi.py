"""The C-ABI library loads, exports exactly what include/mor_b200.h declares, and
validates arguments on the host (no kernel is launched in this file)."""
import ctypes
import os
import re
import subprocess

import pytest

from mor_b200 import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "mor_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"MOR_B200_API\s+[\w\s\*]+?\b(mor_b200_\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    assert len(names) == 34
    for n in ("mor_b200_fake_quantize", "mor_b200_block_scaling", "mor_b200_channel_scaling", "mor_b200_e8mx",
              "mor_b200_quant_dequant", "mor_b200_e4m3_with_e8_scale", "mor_b200_fake_quantize_group",
              "mor_b200_workspace_bytes"):
        assert n in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(cabi.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/mor_b200.h but not exported"
    out = subprocess.run(["nm", "-D", "--defined-only", cabi.LIB_PATH], capture_output=True, text=True).stdout
    exported = sorted(l.split()[-1] for l in out.splitlines() if " T " in l)
    assert exported == declared_functions(), "the library exports symbols the header does not declare"


def test_python_binding_covers_the_header():
    assert sorted(cabi.SIGNATURES) == declared_functions()


def test_header_compiles_as_c_and_cpp(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "mor_b200.h"\nint main(void){return mor_b200_version()==0;}\n')
    for cc, std in (("gcc", "-std=c99"), ("g++", "-std=c++17")):
        exe = tmp_path / ("t_" + cc)
        r = subprocess.run([f"/usr/bin/{cc}", std, "-Wall", "-Werror", "-x", "c" if cc == "gcc" else "c++", str(src),
                            f"-I{ROOT}/include", f"-L{os.path.dirname(cabi.LIB_PATH)}", "-lmor_b200",
                            f"-Wl,-rpath,{os.path.dirname(cabi.LIB_PATH)}", "-o", str(exe)],
                           capture_output=True, text=True)
        assert r.returncode == 0, r.stderr


def test_version_and_status_strings():
    L = cabi.lib()
    assert L.mor_b200_version() >= 100
    assert L.mor_b200_status_string(0) == b"ok"
    for code in (-1, -2, -3, -4, -5):
        assert L.mor_b200_status_string(code) not in (b"ok", b"unknown status")


def test_workspace_sizes():
    wb = cabi.workspace_bytes
    head = 256 + 4096  # scalars, then 1024 partial sums of a long error array
    assert wb(cabi.OP_E8MX, 4096, 4096, 128, 128) == head
    # head + block amax + block errors, each rounded to 256 bytes
    assert wb(cabi.OP_BLOCK_SCALING, 256, 256, 128, 128) == head + 256 + 256
    assert wb(cabi.OP_BLOCK_SCALING, 4096, 4096, 128, 128) == head + 2 * 4096
    assert wb(cabi.OP_BLOCK_SCALING, 256, 256, 16, 16) == 0          # not a multiple of 32 x 64
    assert wb(cabi.OP_BLOCK_SCALING, 250, 256, 128, 128) == 0        # does not divide
    assert wb(cabi.OP_CHANNEL_SCALING, 8192, 8192, 1, 8192) == head + 2 * 4 * 8192
    assert wb(cabi.OP_CHANNEL_SCALING, 16384, 8192, 1, 32) == head + 4 * 16384 * 64   # one error per 128 columns
    assert wb(cabi.OP_CHANNEL_SCALING, 256, 256, 256, 1) == head + 4 * 256 + 256
    assert wb(cabi.OP_CHANNEL_SCALING, 256, 256, 2, 2) == 0
    assert cabi.lib().mor_b200_scaling_error_stride(cabi.OP_CHANNEL_SCALING, 1, 32) == 4
    assert cabi.lib().mor_b200_scaling_error_stride(cabi.OP_CHANNEL_SCALING, 256, 1) == 64
    assert cabi.lib().mor_b200_scaling_num_errors(cabi.OP_BLOCK_SCALING, 131072, 16384, 128, 128) == 1024 * 128


def test_argument_errors_come_back_as_status_codes():
    """Validation happens before any CUDA call, so this runs without a device."""
    L = cabi.lib()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf) & ~15
    assert L.mor_b200_fake_quantize(None, p, p, 0, 16, 16, 4, 4, 1.0, 1, 1, None) == -1
    assert L.mor_b200_fake_quantize(p, p, p, 7, 16, 16, 4, 4, 1.0, 1, 1, None) == -1      # dtype
    assert L.mor_b200_fake_quantize(p, p, p, 0, 16, 15, 4, 4, 1.0, 1, 1, None) == -1      # odd columns
    assert L.mor_b200_fake_quantize(p, p, p, 0, 16, 16, 4, 4, 1.0, 1, 9, None) == -1      # sf_type
    assert L.mor_b200_fake_quantize(p, p, p, 0, 64, 64, 2, 1024, 1.0, 1, 1, None) == -2   # MoR block < 32 rows
    assert L.mor_b200_block_scaling(p, p, 0, 256, 256, 128, 128, 0.045, 0, p, p, p, 0, p, p, 4096, None) == -1
    assert L.mor_b200_block_scaling(p, p, 0, 256, 256, 128, 128, 0.045, 1, p, p, p, 0, p, None, 0, None) == -3
    assert L.mor_b200_block_scaling(p, p, 0, 256, 256, 128, 128, 0.045, 1, p, p, p, 0, p, p, 16, None) == -3
    assert L.mor_b200_channel_scaling(p, p, 0, 256, 256, 2, 2, 0.045, 1, p, p, p, 0, p, p, 4096, None) == -1
    assert L.mor_b200_e8mx(p, p, 64, 64, 0, 1, p, 4096, None) == -1
    assert L.mor_b200_quant_dequant(None, p, 4, 4, 0, None) == -1
    assert L.mor_b200_fake_quantize_group(p, p, None, 0, 64, 64, 48, 0, 2, None) == -1    # 48 does not divide 64
    assert L.mor_b200_scaling_finalize(p, 4, 3, p, 0.045, p, p, p, 4096, None) == -1      # stride not a power of 2


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    import importlib
    import mor_b200.cabi as c2
    monkeypatch.setattr(c2, "LIB_PATH", str(tmp_path / "nope.so"))
    monkeypatch.setattr(c2, "_lib", None)
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        c2.lib()
    importlib.reload(c2)


def test_ops_surface_matches_reference_signatures():
    """mor/ops.py of the reference: same names, same positional parameters."""
    import inspect
    import mor
    expect = {
        "fake_quantize": ["a", "dim_x", "dim_y", "block_x", "block_y", "clamp_threshold", "mode", "sf_type"],
        "fake_quantize_no_alloc": ["a", "dim_x", "dim_y", "block_x", "block_y", "clamp_threshold", "mode", "sf_type", "output"],
        "fake_quantize_block_scaling": ["a", "dim_x", "dim_y", "block_x", "block_y", "e4m3_threshold", "ss_mode"],
        "fake_quantize_block_scaling_inplace": ["a", "dim_x", "dim_y", "block_x", "block_y", "e4m3_threshold", "ss_mode"],
        "fake_quantize_channel_scaling": ["a", "dim_x", "dim_y", "block_x", "block_y", "e4m3_threshold", "ss_mode"],
        "fake_quantize_channel_scaling_inplace": ["a", "dim_x", "dim_y", "block_x", "block_y", "e4m3_threshold", "ss_mode"],
        "fake_quantize_e8mx": ["a", "dim_x", "dim_y", "block_x", "block_y", "quantize_type", "scaling_strategy"],
        "fake_quantize_e8mx_inplace": ["a", "dim_x", "dim_y", "block_x", "block_y", "quantize_type", "scaling_strategy", "output"],
        "quant_dequant_e4m3": ["a", "dim_x", "dim_y", "block_x", "block_y"],
        "quant_dequant_e5m2": ["a", "dim_x", "dim_y", "block_x", "block_y"],
        "quant_dequant_e2m3": ["a", "dim_x", "dim_y", "block_x", "block_y"],
        "quant_dequant_e3m2": ["a", "dim_x", "dim_y", "block_x", "block_y"],
        "e4m3_with_e8_scale_rne": ["a", "dim_x", "dim_y", "block_x", "block_y"],
        "e4m3_with_e8_scale_rz": ["a", "dim_x", "dim_y", "block_x", "block_y"],
    }
    for name, params in expect.items():
        assert list(inspect.signature(getattr(mor.ops, name)).parameters) == params, name


# the operator schemas of the reference extension (mor/csrc/fake_quantize.cpp:12-25), which a drop-in must register unchanged
REFERENCE_SCHEMAS = [
    "fake_quantize(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float clamp_threshold, int mode, int sf_type) -> Tensor[]",
    "fake_quantize_no_alloc(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float clamp_threshold, int mode, int sf_type, Tensor result) -> Tensor",
    "quant_dequant_e4m3(Tensor input, int dim_x, int dim_y, int block_x, int block_y) -> Tensor",
    "quant_dequant_e5m2(Tensor input, int dim_x, int dim_y, int block_x, int block_y) -> Tensor",
    "quant_dequant_e3m2(Tensor input, int dim_x, int dim_y, int block_x, int block_y) -> Tensor",
    "quant_dequant_e2m3(Tensor input, int dim_x, int dim_y, int block_x, int block_y) -> Tensor",
    "e4m3_with_e8_scale_rne(Tensor input, int dim_x, int dim_y, int block_x, int block_y) -> Tensor",
    "e4m3_with_e8_scale_rz(Tensor input, int dim_x, int dim_y, int block_x, int block_y) -> Tensor",
    "fake_quantize_block_scaling(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float e4m3_threshold, int ss_mode) -> Tensor[]",
    "fake_quantize_block_scaling_inplace(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float e4m3_threshold, int ss_mode) -> Tensor[]",
    "fake_quantize_e8mx(Tensor input, int dim_x, int dim_y, int block_x, int block_y, int quantize_type, int scaling_strategy) -> Tensor",
    "fake_quantize_e8mx_inplace(Tensor input, int dim_x, int dim_y, int block_x, int block_y, int quantize_type, int scaling_strategy, Tensor result) -> ()",
    "fake_quantize_channel_scaling(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float e4m3_threshold, int ss_mode) -> Tensor[]",
    "fake_quantize_channel_scaling_inplace(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float e4m3_threshold, int ss_mode) -> Tensor[]",
]


def test_registered_schemas_are_the_reference_ones():
    import torch
    import mor  # noqa: F401
    for schema in REFERENCE_SCHEMAS:
        name = schema.split("(", 1)[0]
        assert str(getattr(torch.ops.mor, name).default._schema) == "mor::" + schema, name
    with pytest.raises(NotImplementedError):   # CUDA only: no CPU kernel, no fallback
        torch.ops.mor.fake_quantize.default(torch.zeros(4, 4, dtype=torch.bfloat16), 4, 4, 2, 2, 1.0, 1, 1)
