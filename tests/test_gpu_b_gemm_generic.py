"""GPU parity of the stride-agnostic GEMM kernel (every epilogue) against the golden
vectors produced by the reference's kernels, through the C ABI."""
import pytest
import torch

from oracle import ops as O
from triton_int_b200 import config, synthetic
from triton_int_b200.kernels import bmm as KB
from triton_int_b200.kernels import fused as KF
from triton_int_b200.kernels import linear as KL
from util import assert_equal, assert_status_clean, assert_within_1lsb, dev, gemm_path

pytestmark = pytest.mark.gpu
T = torch.from_numpy
PATH = "generic"


def run_linear_golden(g, case):
    x, w = dev(T(g[f"{case}/x"])), dev(T(g[f"{case}/w"]))
    b8, b32, bf = (dev(T(g[f"{case}/{k}"])) for k in ("bias8", "bias32", "biasf"))
    a, b = dev(T(g[f"{case}/alpha"])), dev(T(g[f"{case}/beta"]))
    with config.rounding("trunc_wrap"):
        assert_equal(KL.linear_a8_w8_ofp32(x, w, a), T(g[f"{case}/ofp32"]), "ofp32")
        assert_equal(KL.linear_a8_w8_b8_o8(x, w, b8, a, b), T(g[f"{case}/b8_o8"]), "b8_o8")
        assert_equal(KL.linear_relu_a8_w8_b8_o8(x, w, b8, a, b), T(g[f"{case}/relu_b8_o8"]), "relu")
        assert_equal(KL.linear_a8_w8_b32_o32(x, w, b32), T(g[f"{case}/b32_o32"]), "b32_o32")
        assert_equal(KL.linear_a8_w8_b32_o32_with_scaling(x, w, b32, a, b), T(g[f"{case}/b32_o32_scaled"]), "scaled i32")
        assert_equal(KL.linear_a8_w8_bfp32_ofp32(x, w, bf, a, b), T(g[f"{case}/bfp32_ofp32"]), "bfp32")
        assert_equal(KL.linear_a8_w8_bfp32_ofp32(x, w, bf.half(), a, b), T(g[f"{case}/bfp16_ofp16"]), "bfp16")
        y = KF.linear_a8_w8_bfp32_ofp32_GeLu_Q(x, w, bf, a, dev(T(g[f"{case}/gelu_mul"])))
        # tanhf on the GPU and numpy.tanh differ in the last ulp: allow rare one-step differences
        assert_within_1lsb(y, T(g[f"{case}/gelu_q"]), 5e-3, "gelu_q")
    assert_status_clean()


@pytest.mark.parametrize("case", ["ragged", "m1", "lead3d", "ktail"])
def test_linear_golden(golden, case):
    with gemm_path(PATH):
        run_linear_golden(golden["linear"], case)


def test_linear_strided_weight(golden):
    g = golden["linear"]
    w = dev(T(g["strided/wide"]))[:, ::2]
    with config.rounding("trunc_wrap"):
        y = KL.linear_a8_w8_b8_o8(dev(T(g["strided/x"])), w, dev(T(g["strided/bias8"])),
                                  dev(T(g["strided/alpha"])), dev(T(g["strided/beta"])))
    assert_equal(y, T(g["strided/b8_o8"]), "strided weight")


def run_bmm_golden(g, case, nn_too=True):
    a, bn, bt, s = (dev(T(g[f"{case}/{k}"])) for k in ("a", "bn", "bt", "scale"))
    with config.rounding("trunc_wrap"):
        assert_equal(KB.bmm_s8t_s8n_s32t(a, bn), T(g[f"{case}/s8t_s8n_s32t"]), "s8n_s32t")
        assert_equal(KB.bmm_s8t_s8n_f32t(a, bn, s), T(g[f"{case}/s8t_s8n_f32t"]), "s8n_f32t")
        assert_equal(KB.bmm_s8t_s8n_f32t(a, bn, s, dtype=torch.float16), T(g[f"{case}/s8t_s8n_f16t"]), "s8n_f16t")
        assert_equal(KB.bmm_s8t_s8n_s8t(a, bn, s), T(g[f"{case}/s8t_s8n_s8t"]), "s8n_s8t")
        if nn_too:
            assert_equal(KB.bmm_s8t_s8t_s32t(a, bt), T(g[f"{case}/s8t_s8t_s32t"]), "s8t_s32t")
            assert_equal(KB.bmm_s8t_s8t_s8t(a, bt, s), T(g[f"{case}/s8t_s8t_s8t"]), "s8t_s8t")
    assert_status_clean()


@pytest.mark.parametrize("case", ["small", "ragged"])
def test_bmm_golden(golden, case):
    with gemm_path(PATH):
        run_bmm_golden(golden["bmm"], case)


def test_config1_both_policies(golden):
    g = golden["config1"]
    c = synthetic.config1_linear(seed=0)
    x, w, bias = dev(c["x"]), dev(c["w"]), dev(c["bias"])
    with gemm_path(PATH):
        with config.rounding("trunc_wrap"):
            y = KL.linear_a8_w8_b8_o8(x, w, bias, dev(c["alpha"]), dev(c["beta"]))
        assert_equal(y, T(g["y"]), "config1 trunc_wrap vs reference")
        with config.rounding("rne_sat"):
            ys = KL.linear_a8_w8_b8_o8(x, w, bias, dev(c["alpha"]), dev(c["beta"]))
        acc = KL.linear_a8_w8_b32_o32(x, w, None)
    assert_equal(ys, O.linear_a8_w8_b8_o8(c["x"], c["w"], c["bias"], c["alpha"], c["beta"], O.RNE_SAT), "config1 rne_sat")
    assert_equal(acc[:4], T(g["acc_head"]), "config1 accumulators")
    assert_equal(acc, O.acc_linear(c["x"], c["w"]), "config1 accumulators (all)")
    # report the mismatch rate of the saturating policy against the reference on in-range values
    f = O.linear_a8_w8_b8_o8_f32(c["x"], c["w"], c["bias"], c["alpha"], c["beta"])
    inr = (f >= -128) & (f <= 127)
    d = (ys.cpu()[inr].int() - T(g["y"])[inr].int()).abs()
    assert d.max().item() <= 1
    print(f"config1: {1 - inr.float().mean().item():.3f} of values saturate; "
          f"rne_sat vs reference mismatch rate on in-range values {(d != 0).float().mean().item():.3f}")


def test_errors_and_edges():
    x = torch.zeros((4, 32), dtype=torch.int8)
    w = torch.zeros((8, 32), dtype=torch.int8)
    with pytest.raises(RuntimeError):  # no CPU path
        KL.linear_a8_w8_b32_o32(x, w, None)
    with pytest.raises(AssertionError):  # shape mismatch, as the reference asserts
        KL.linear_a8_w8_b32_o32(x.cuda(), torch.zeros((8, 31), dtype=torch.int8).cuda(), None)
    with pytest.raises(AssertionError):
        KB.bmm_s8t_s8n_s32t(x.cuda(), w.cuda())  # BMM wants 3-D
    # empty M
    y = KL.linear_a8_w8_b32_o32(torch.zeros((0, 32), dtype=torch.int8).cuda(), w.cuda(), None)
    assert y.shape == (0, 8)
    # out= is honoured
    out = torch.empty((4, 8), dtype=torch.int32).cuda()
    r = KL.linear_a8_w8_b32_o32(x.cuda() + 1, w.cuda() + 2, None, out=out)
    assert r.data_ptr() == out.data_ptr() and (out == 64).all()
    assert_status_clean()
