"""GPU parity of the row kernels (LayerNorm family, dequant+add+LayerNorm+quant,
int8 GELU, causal softmax -> int8) against the golden vectors and the CPU oracle.
All calls go through the C ABI (ctypes) via the Python wrappers."""
import numpy as np
import pytest
import torch

from oracle import ops as O
from triton_int_b200 import config, synthetic
from triton_int_b200.kernels import fused as K
from util import MODES, assert_close_rel, assert_equal, assert_status_clean, assert_within_1lsb, dev

pytestmark = pytest.mark.gpu
T = torch.from_numpy
LN_CASES = ["h4096", "n300", "n5000", "f16n256"]


@pytest.mark.parametrize("case", LN_CASES)
def test_layernorm_golden(golden, case):
    g = golden["layernorm"]
    x, skip, w, b = (T(g[f"{case}/{k}"]) for k in ("x", "skip", "w", "b"))
    tol = 1e-5 if x.dtype == torch.float32 else 2e-3  # fp16 storage: one half-precision ulp
    with config.rounding("trunc_wrap"):
        q = K.layer_norm_fwd_fused_single_pass_q(dev(x), dev(w), dev(b), 1e-5)
        q_rms = K.layer_norm_fwd_fused_single_pass_q(dev(x), dev(w), dev(b), 1e-5, True)
        q_nb = K.layer_norm_fwd_fused_single_pass_q(dev(x), dev(w), None, 1e-5)
    # reductions run in a different order than numpy's pairwise sum: allow one step
    assert_within_1lsb(q, T(g[f"{case}/ln_q"]), 0.02, "ln_q")
    assert_within_1lsb(q_rms, T(g[f"{case}/ln_q_rms"]), 0.02, "ln_q_rms")
    assert_within_1lsb(q_nb, T(g[f"{case}/ln_q_nobias"]), 0.02, "ln_q_nobias")
    y = K.layer_norm_fwd_fused_single_pass(dev(x), dev(w), dev(b), 1e-5)
    assert y.dtype == x.dtype
    scale = T(g[f"{case}/ln"]).float().abs().max().item()
    assert_close_rel(y.float() / scale, T(g[f"{case}/ln"]).float() / scale, tol, "ln")
    s1 = K.skip_layer_norm_fwd_fused_single_pass(dev(x), dev(skip), dev(w), dev(b), 1e-5)
    o0, o1 = K.skip_layer_norm_fwd_fused_single_pass2(dev(x), dev(skip), dev(w), dev(b), 1e-5)
    assert_close_rel(s1.float() / scale, T(g[f"{case}/skip_ln"]).float() / scale, tol, "skip_ln")
    assert_close_rel(o0.float() / scale, T(g[f"{case}/skip_ln2_0"]).float() / scale, tol, "skip_ln2_0")
    assert_close_rel(o1.float() / scale, T(g[f"{case}/skip_ln2_1"]).float() / scale, tol, "skip_ln2_1")
    assert_status_clean()


def test_layernorm_strided_and_odd_n():
    gen = synthetic.gen(11)
    x = torch.randn((7, 2 * 333), generator=gen)
    w = torch.rand((333,), generator=gen) * 30
    b = torch.randn((333,), generator=gen)
    xs = x[:, ::2]  # column stride 2, odd width: takes the stride-agnostic kernel
    with config.rounding("trunc_wrap"):
        q = K.layer_norm_fwd_fused_single_pass_q(dev(x)[:, ::2], dev(w), dev(b), 1e-5)
    want = O.layer_norm_fwd_fused_single_pass_q(xs.contiguous(), w, b, 1e-5)
    assert_within_1lsb(q, want, 0.02, "strided ln_q")


def test_dq_add_layernorm_q_golden(golden):
    g = golden["layernorm"]
    acc, res, w, b = (T(g[f"dq/{k}"]) for k in ("acc", "res", "w", "b"))
    r, y = K.dq_add_layernorm_q(dev(acc), 1e-4, dev(res), dev(w), dev(b), 1e-5)
    assert_equal(r, T(g["dq/res_out"]), "residual_out")  # one fused multiply-add per element: exact
    assert_within_1lsb(y, T(g["dq/y"]), 0.02, "dq y")
    # scale given as a device tensor
    r2, y2 = K.dq_add_layernorm_q(dev(acc), torch.tensor(1e-4).cuda(), dev(res), dev(w), dev(b), 1e-5)
    assert_equal(r2, T(g["dq/res_out"]), "residual_out (device scale)")
    assert torch.equal(y2, y)
    assert_status_clean()


@pytest.mark.parametrize("rows", [64, 8192])
def test_dq_add_layernorm_q_config2(rows):
    """Config-2 shapes; the full 8192 rows are checked against the oracle too (it takes a second on CPU)."""
    c = synthetic.config2_lnq(seed=1, rows=rows)
    r, y = K.dq_add_layernorm_q(dev(c["acc"]), c["dq_scale"], dev(c["residual"]), dev(c["gamma"]), dev(c["beta"]), c["eps"])
    r_ref, f_ref = O.dq_add_layernorm_q_f32(c["acc"], c["dq_scale"], c["residual"], c["gamma"], c["beta"], c["eps"])
    assert_equal(r, r_ref, "residual_out")
    y_ref = f_ref.clamp(-128, 127).round().to(torch.int8)
    rate = assert_within_1lsb(y, y_ref, 0.01, "config2 ln int8")
    # LayerNorm value itself within 1e-5 relative: recompute it in fp32 from the kernel's residual
    print(f"config2 rows={rows}: int8 mismatch rate vs oracle {rate:.6f}")
    # bias_int32 extension == adding the bias to the accumulators first
    bias = synthetic.int32_normal((c["acc"].shape[1],), 1e3, synthetic.gen(5))
    r3, y3 = K.dq_add_layernorm_q(dev(c["acc"]), c["dq_scale"], dev(c["residual"]), dev(c["gamma"]), dev(c["beta"]),
                                  c["eps"], bias_int32=dev(bias))
    r4, y4 = K.dq_add_layernorm_q(dev(c["acc"] + bias), c["dq_scale"], dev(c["residual"]), dev(c["gamma"]),
                                  dev(c["beta"]), c["eps"])
    assert torch.equal(r3, r4) and torch.equal(y3, y4)
    assert_status_clean()


def test_layernorm_fp32_value_tolerance():
    """fp32 LayerNorm output within 1e-5 * max(1, |ref|) of a float64 evaluation."""
    gen = synthetic.gen(12)
    x = torch.randn((128, 4096), generator=gen) * 3 + 1
    w = torch.rand((4096,), generator=gen) + 0.5
    b = torch.randn((4096,), generator=gen)
    y = K.layer_norm_fwd_fused_single_pass(dev(x), dev(w), dev(b), 1e-5)
    ref = torch.nn.functional.layer_norm(x.double(), (4096,), w.double(), b.double(), 1e-5)
    assert_close_rel(y, ref.float(), 1e-5, "ln fp32")


@pytest.mark.parametrize("mode", ["rne_sat", "trunc_wrap"])
def test_gelu_q(mode):
    c = synthetic.config2_gelu(seed=1, rows=512, cols=4096 + 16)
    x = c["x"].reshape(-1)[: 512 * 4096 + 7]  # odd tail
    with config.rounding(mode):
        y = K.gelu_q(dev(x), c["in_scale"], 1.0 / c["out_scale"])
    want = O.gelu_q(x, c["in_scale"], 1.0 / c["out_scale"], MODES[mode])
    assert_within_1lsb(y, want, 1e-3, "gelu_q")
    # all 256 inputs, unaligned start
    allv = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8).repeat(3)
    buf = torch.zeros(1 + allv.numel(), dtype=torch.int8).cuda()
    buf[1:] = allv.cuda()
    with config.rounding(mode):
        y2 = K.gelu_q(buf[1:], 0.03, 50.0)
    assert_within_1lsb(y2, O.gelu_q(allv, 0.03, 50.0, MODES[mode]), 0.01, "gelu_q all values")
    assert_status_clean()


@pytest.mark.parametrize("shape", [(3, 40, 40), (2, 33, 50), (2, 64, 2048), (1, 5, 7)])
def test_causal_softmax_q(shape):
    gen = synthetic.gen(13)
    s = torch.randn(shape, generator=gen) * 4
    p = K.causal_softmax_q(dev(s), 127.0)
    want = O.causal_softmax_q(s, 127.0, O.RNE_SAT)
    assert_within_1lsb(p, want, 0.01, "softmax_q")
    pn = K.causal_softmax_q(dev(s), 127.0, causal=False)
    wantn = torch.softmax(s, -1).mul(127.0).round().clamp(-128, 127).to(torch.int8)
    assert_within_1lsb(pn, wantn, 0.01, "softmax_q (no mask)")
    # masked positions are exact zeros
    B, M, N = shape
    i, j = torch.arange(M)[:, None], torch.arange(N)[None, :]
    assert (p.cpu()[:, j > i + (N - M)] == 0).all()
    assert_status_clean()
