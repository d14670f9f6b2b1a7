"""The allocation-free GEMM entry point (ti_gemm_i8_static_scratch).

It exists for hosts that cannot allocate device memory when they call the library (all
HBM already handed to their own pools, a loop that must not hit cudaMalloc's device-wide
synchronisation, a plugin that may not own device memory).  The test drives it through
the C ABI with pre-allocated inputs and outputs, twice in a row, and requires the same
bits as the regular entry point given a caller-provided workspace.  This file sorts last
so that a run stopping at the first failure has already run everything else."""
import ctypes as C

import pytest
import torch

from triton_int_b200 import _lib, synthetic

pytestmark = pytest.mark.gpu


def _params(x, w, out, bias, alpha, beta, out_code, epilogue):
    p = _lib.GemmParams()
    p.a, p.b, p.c = x.data_ptr(), w.data_ptr(), out.data_ptr()
    if bias is not None:
        p.bias, p.bias_dtype = bias.data_ptr(), _lib.DTYPE_CODE[bias.dtype]
    if alpha is not None:
        p.alpha, p.beta = alpha.data_ptr(), beta.data_ptr()
    p.m, p.k = x.shape
    p.n = w.shape[0]
    p.batch = 1
    p.a_stride_m, p.a_stride_k = x.stride(0), 1
    p.b_stride_n, p.b_stride_k = w.stride(0), 1
    p.c_stride_m, p.c_stride_n = out.stride(0), 1
    p.out_dtype, p.epilogue = out_code, epilogue
    p.rounding, p.path = _lib.ROUND_RNE_SAT, _lib.PATH_TCGEN05
    p.stream = torch.cuda.current_stream().cuda_stream
    return p


def test_static_scratch_matches_workspace_entry_point_twice():
    lib = _lib.load()
    cap = lib.ti_static_scratch_bytes()
    assert cap == 8 * 1024 * 1024
    for call in range(2):  # second call reuses the array with the first call's leftovers in it
        c = synthetic.config5_linear(seed=4 + call, m=16, layer="fc1" if call == 0 else "fc2")
        x, w = c["x"].cuda(), c["w"].cuda()
        bias, alpha, beta = c["bias_i8"].cuda(), c["alpha"].cuda(), c["beta"].cuda()
        for out_dtype, code, epi, b in ((torch.int32, _lib.TI_I32, _lib.EPI_I32, None),
                                        (torch.int8, _lib.TI_I8, _lib.EPI_SCALE_BIAS, bias)):
            ref = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device="cuda")
            got = torch.full_like(ref, 7)
            a_, b_ = (alpha, beta) if b is not None else (None, None)
            pr = _params(x, w, ref, b, a_, b_, code, epi)
            need = lib.ti_gemm_workspace_bytes(C.byref(pr))
            assert 0 < need <= cap, "the case must take the split-K path and fit the built-in scratch"
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            pr.workspace, pr.workspace_bytes = ws.data_ptr(), need
            assert lib.ti_gemm_i8(C.byref(pr)) == _lib.TI_OK, lib.ti_last_error_string()
            pg = _params(x, w, got, b, a_, b_, code, epi)
            before = _lib.launch_count()
            assert lib.ti_gemm_i8_static_scratch(C.byref(pg)) == _lib.TI_OK, lib.ti_last_error_string()
            assert _lib.launch_count() - before == 2, "split-K form expected (GEMM into scratch + reduce)"
            torch.cuda.synchronize()
            assert torch.equal(got, ref), f"call {call}, {out_dtype}: static-scratch result differs"
    assert _lib.device_status() == 0


def test_static_scratch_refuses_oversized_problems():
    lib = _lib.load()
    # 128 rows of a 9216-wide output split four ways need 18 MiB of partial sums
    x = torch.zeros((128, 4608), dtype=torch.int8, device="cuda")
    w = torch.zeros((9216, 4608), dtype=torch.int8, device="cuda")
    out = torch.empty((128, 9216), dtype=torch.int32, device="cuda")
    p = _params(x, w, out, None, None, None, _lib.TI_I32, _lib.EPI_I32)
    need = lib.ti_gemm_workspace_bytes(C.byref(p))
    if need <= lib.ti_static_scratch_bytes():
        pytest.skip("this device does not split the probe shape beyond the built-in scratch")
    assert lib.ti_gemm_i8_static_scratch(C.byref(p)) == _lib.TI_ERR_UNSUPPORTED
    msg = lib.ti_last_error_string().decode()
    assert str(need) in msg and str(lib.ti_static_scratch_bytes()) in msg
