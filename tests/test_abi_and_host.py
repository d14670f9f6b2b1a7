"""CPU-side checks: the C-ABI library loads and exports every symbol the header
declares, status codes map to the reference's exception types, host-side helpers
(sharding, scale handling, rounding policy switch) behave, and nothing in the
product path imports the oracle."""
import ctypes
import os
import re

import pytest
import torch

from triton_int_b200 import _build, _lib, config
from triton_int_b200.nn import decoder

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "triton_int_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ti_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = header_functions()
    assert {"ti_gemm_i8", "ti_layernorm", "ti_gelu_q", "ti_softmax_q", "ti_device_status"} <= set(names)
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert lib.ti_version() >= 100
    assert os.path.dirname(_lib.lib_path()).endswith("triton_int_b200")


def test_struct_layouts_match_header_field_order():
    text = open(os.path.join(ROOT, "include", "triton_int_b200.h")).read()

    def fields(struct):
        body = text[text.index("typedef struct {", text.index(struct) - 2500 if struct == "ti_gemm_params;" else 0):]
        return body

    for cname, cls in (("ti_gemm_params", _lib.GemmParams), ("ti_layernorm_params", _lib.LayerNormParams)):
        end = text.index("} " + cname + ";")
        start = text.rfind("typedef struct {", 0, end)
        body = re.sub(r"/\*.*?\*/", "", text[start:end], flags=re.S)
        decl = []
        for stmt in body.split(";"):
            stmt = stmt.replace("typedef struct {", "").strip()
            if not stmt:
                continue
            names = stmt.split(",")
            first = names[0].split()[-1]
            decl.append(first.lstrip("*"))
            decl += [n.strip().lstrip("*") for n in names[1:]]
        assert decl == [f[0] for f in cls._fields_], (cname, decl)


def test_no_cpu_path_and_error_mapping():
    from triton_int_b200.kernels import bmm, fused, linear
    x = torch.zeros((4, 32), dtype=torch.int8)
    w = torch.zeros((8, 32), dtype=torch.int8)
    with pytest.raises(RuntimeError, match="no CPU path"):
        linear.linear_a8_w8_b32_o32(x, w, None)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fused.layer_norm_fwd_fused_single_pass_q(torch.zeros(2, 8), torch.ones(8), None, 1e-5)
    with pytest.raises(AssertionError):
        linear.linear_a8_w8_b32_o32(x, torch.zeros((8, 31), dtype=torch.int8), None)
    with pytest.raises(AssertionError):
        bmm.bmm_s8t_s8n_s32t(x, w)
    with pytest.raises(AssertionError):
        _lib.check(_lib.TI_ERR_SHAPE, "x")
    with pytest.raises(RuntimeError):
        _lib.check(_lib.TI_ERR_ALIGN, "x")


def test_c_abi_rejects_host_pointers_without_a_gpu():
    lib = _lib.load()
    p = _lib.GemmParams()
    buf = (ctypes.c_int8 * 64)()
    p.a = p.b = p.c = ctypes.addressof(buf)
    p.m = p.n = p.k = 4
    p.batch = 1
    p.out_dtype, p.epilogue = _lib.TI_I32, _lib.EPI_I32
    rc = lib.ti_gemm_i8(ctypes.byref(p))
    assert rc in (_lib.TI_ERR_DEVICE, _lib.TI_ERR_CUDA)  # no device, or host memory: never computed on the CPU
    assert lib.ti_last_error_string()
    p.out_dtype = _lib.TI_I8
    assert lib.ti_gemm_i8(ctypes.byref(p)) == _lib.TI_ERR_DTYPE  # raw accumulators are int32


def test_rounding_policy_switch():
    assert config.rounding_mode_name() == "rne_sat"
    with config.rounding("trunc_wrap"):
        assert config.rounding_mode() == _lib.ROUND_TRUNC_WRAP
    assert config.rounding_mode() == _lib.ROUND_RNE_SAT


def test_shard_helpers_partition_exactly():
    w = torch.arange(8 * 12).reshape(8, 12)
    rows = [decoder.shard_rows(w, r, 4) for r in range(4)]
    cols = [decoder.shard_cols(w, r, 4) for r in range(4)]
    assert torch.equal(torch.cat(rows, 0), w) and torch.equal(torch.cat(cols, 1), w)
    with pytest.raises(AssertionError):
        decoder.shard_rows(w, 0, 3)


def test_product_code_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "triton_int_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.replace("# oracle", ""), f"{f} mentions the oracle"


def test_build_flags_target_sm100a_only():
    assert "arch=compute_100a,code=sm_100a" in _build.NVCC_FLAGS
    assert "-lineinfo" in _build.NVCC_FLAGS


def test_reference_import_paths_resolve():
    """Model code written against the reference's package name imports unchanged."""
    from triton_int.functional.bmm import bmm_i8_o8  # noqa: F401
    from triton_int.kernels.linear import linear_a8_w8_b8_o8  # noqa: F401
    from triton_int.nn.bmm import BMM_S8T_S8N_F32T
    from triton_int.nn.fused import DQ_Add_LayerNorm_Q, LayerNormQ  # noqa: F401
    from triton_int.nn.linear import W8A8B8O8Linear, W8A8BFP32OFP32Linear  # noqa: F401
    import triton_int_b200.nn.bmm as impl
    assert BMM_S8T_S8N_F32T is impl.BMM_S8T_S8N_F32T
