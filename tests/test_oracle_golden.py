"""Pins the CPU oracle (oracle/ops.py) to outputs of the reference's own kernels run
under Triton's CPU interpreter (tests/golden/*.npz, made by tests/golden/make_golden.py)."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import ops as O
from triton_int_b200 import synthetic

T = torch.from_numpy


def eq(a, b):
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    assert torch.equal(a, b), f"{(a != b).sum().item()} of {a.numel()} differ"


LINEAR_CASES = ["ragged", "m1", "lead3d", "ktail"]


@pytest.mark.parametrize("case", LINEAR_CASES)
def test_linear_bit_exact(golden, case):
    g = golden["linear"]
    x, w = T(g[f"{case}/x"]), T(g[f"{case}/w"])
    b8, b32, bf = T(g[f"{case}/bias8"]), T(g[f"{case}/bias32"]), T(g[f"{case}/biasf"])
    a, b = T(g[f"{case}/alpha"]), T(g[f"{case}/beta"])
    eq(O.linear_a8_w8_ofp32(x, w, a), T(g[f"{case}/ofp32"]))
    eq(O.linear_a8_w8_b8_o8(x, w, b8, a, b), T(g[f"{case}/b8_o8"]))
    eq(O.linear_relu_a8_w8_b8_o8(x, w, b8, a, b), T(g[f"{case}/relu_b8_o8"]))
    eq(O.linear_a8_w8_b32_o32(x, w, b32), T(g[f"{case}/b32_o32"]))
    eq(O.linear_a8_w8_b32_o32_with_scaling(x, w, b32, a, b), T(g[f"{case}/b32_o32_scaled"]))
    eq(O.linear_a8_w8_bfp32_ofp32(x, w, bf, a, b), T(g[f"{case}/bfp32_ofp32"]))
    eq(O.linear_a8_w8_bfp32_ofp32(x, w, bf.half(), a, b), T(g[f"{case}/bfp16_ofp16"]))
    eq(O.linear_a8_w8_bfp32_ofp32_GeLu_Q(x, w, bf, a, T(g[f"{case}/gelu_mul"])), T(g[f"{case}/gelu_q"]))


def test_linear_strided_weight(golden):
    g = golden["linear"]
    w = T(g["strided/wide"])[:, ::2]
    y = O.linear_a8_w8_b8_o8(T(g["strided/x"]), w, T(g["strided/bias8"]), T(g["strided/alpha"]), T(g["strided/beta"]))
    eq(y, T(g["strided/b8_o8"]))


@pytest.mark.parametrize("case", ["small", "ragged"])
def test_bmm_bit_exact(golden, case):
    g = golden["bmm"]
    a, bn, bt, s = (T(g[f"{case}/{k}"]) for k in ("a", "bn", "bt", "scale"))
    eq(O.bmm_s8t_s8n_s32t(a, bn), T(g[f"{case}/s8t_s8n_s32t"]))
    eq(O.bmm_s8t_s8t_s32t(a, bt), T(g[f"{case}/s8t_s8t_s32t"]))
    eq(O.bmm_s8t_s8n_f32t(a, bn, s), T(g[f"{case}/s8t_s8n_f32t"]))
    eq(O.bmm_s8t_s8n_f32t(a, bn, s, dtype=torch.float16), T(g[f"{case}/s8t_s8n_f16t"]))
    eq(O.bmm_s8t_s8n_s8t(a, bn, s), T(g[f"{case}/s8t_s8n_s8t"]))
    eq(O.bmm_s8t_s8t_s8t(a, bt, s), T(g[f"{case}/s8t_s8t_s8t"]))


def test_config1_full_size(golden):
    g = golden["config1"]
    c = synthetic.config1_linear(seed=0)
    h = hashlib.sha256()
    for t in (c["x"], c["w"], c["bias"]):
        h.update(t.contiguous().numpy().tobytes())
    assert h.hexdigest() == bytes(g["inputs_sha256"]).decode(), "seeded generator drifted; regenerate the golden file"
    acc = O.acc_linear(c["x"], c["w"])
    assert hashlib.sha256(acc.numpy().tobytes()).hexdigest() == bytes(g["acc_sha256"]).decode()
    eq(acc[:4], T(g["acc_head"]))
    y = O.linear_a8_w8_b8_o8(c["x"], c["w"], c["bias"], c["alpha"], c["beta"], mode=O.TRUNC_WRAP)
    eq(y, T(g["y"]))
    # the share of pre-cast values that fall outside int8 at the stated scales
    f = O.linear_a8_w8_b8_o8_f32(c["x"], c["w"], c["bias"], c["alpha"], c["beta"])
    share = ((f < -128) | (f > 127)).float().mean().item()
    assert 0.75 < share < 0.88
    # the saturating policy agrees with the reference within 1 LSB wherever the value is in range
    ys = O.linear_a8_w8_b8_o8(c["x"], c["w"], c["bias"], c["alpha"], c["beta"], mode=O.RNE_SAT)
    inr = (f >= -128) & (f <= 127)
    assert (ys[inr].int() - y[inr].int()).abs().max().item() <= 1


LN_CASES = ["h4096", "n300", "n5000", "f16n256"]


def _ln_inputs(g, case):
    x, skip, w, b = (T(g[f"{case}/{k}"]) for k in ("x", "skip", "w", "b"))
    return x, skip, w, b


@pytest.mark.parametrize("case", LN_CASES)
def test_layernorm_vs_reference(golden, case):
    g = golden["layernorm"]
    x, skip, w, b = _ln_inputs(g, case)
    tol = dict(rtol=0, atol=0)
    # the restatement follows the interpreter's operation order, so it is bit-exact
    eq(O.layer_norm_fwd_fused_single_pass_q(x, w, b, 1e-5), T(g[f"{case}/ln_q"]))
    eq(O.layer_norm_fwd_fused_single_pass_q(x, w, b, 1e-5, True), T(g[f"{case}/ln_q_rms"]))
    eq(O.layer_norm_fwd_fused_single_pass_q(x, w, None, 1e-5), T(g[f"{case}/ln_q_nobias"]))
    eq(O.layer_norm_fwd_fused_single_pass(x, w, b, 1e-5), T(g[f"{case}/ln"]))
    eq(O.skip_layer_norm_fwd_fused_single_pass(x, skip, w, b, 1e-5), T(g[f"{case}/skip_ln"]))
    o0, o1 = O.skip_layer_norm_fwd_fused_single_pass2(x, skip, w, b, 1e-5)
    eq(o0, T(g[f"{case}/skip_ln2_0"]))
    eq(o1, T(g[f"{case}/skip_ln2_1"]))


def test_dq_add_layernorm_q(golden):
    g = golden["layernorm"]
    r, y = O.dq_add_layernorm_q(T(g["dq/acc"]), 1e-4, T(g["dq/res"]), T(g["dq/w"]), T(g["dq/b"]), 1e-5)
    eq(r, T(g["dq/res_out"]))
    eq(y, T(g["dq/y"]))


def test_cast_policies():
    f = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, 126.5, 127.5, 200.0, -128.5, -129.0, 255.9, 256.0, -300.7])
    assert O.cast_i8(f, O.RNE_SAT).tolist() == [0, 2, 2, 0, -2, 126, 127, 127, -128, -128, 127, 127, -128]
    assert O.cast_i8(f, O.TRUNC_WRAP).tolist() == [0, 1, 2, 0, -1, 126, 127, -56, -128, 127, -1, 0, -44]
