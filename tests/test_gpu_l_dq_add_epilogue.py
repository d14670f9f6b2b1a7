"""Dequantise + residual-add epilogue of the row-parallel linears (TI_EPI_DQ_ADD): the GEMM
writes residual + dq * (acc + bias) itself, a plain LayerNorm -> int8 follows.  The pair must
return the bits of the two-kernel form it replaces (int32 GEMM, then dq_add_layernorm_q) and
match the oracle (functional/fused.py:6-15 of the reference)."""
import pytest
import torch

from oracle import ops as O
from triton_int_b200 import synthetic
from triton_int_b200.kernels import fused as KF
from triton_int_b200.kernels import linear as KL

from util import assert_status_clean, dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,with_bias", [
    (4096, 4096, 1024, True),    # CTA-pair tiles
    (512, 4096, 1024, False),    # 128 x 256 tiles
    (300, 1000, 256, True),      # ragged rows and a ragged last column chunk
    (200, 128, 512, True),       # 128-column tiles
    (100, 64, 256, False),       # 64-column tiles
    (1, 4096, 4096, True),       # a single token (never split along K with this epilogue)
])
def test_dq_add_matches_two_kernel_form_and_oracle(M, N, K, with_bias):
    g = synthetic.gen(700 + M + N)
    x, w = synthetic.int8_normal((M, K), 40, g), synthetic.int8_normal((N, K), 30, g)
    bias = torch.randint(-5000, 5000, (N,), generator=g, dtype=torch.int32) if with_bias else None
    res = torch.randn((M, N), generator=g)
    gamma, beta = torch.rand((N,), generator=g) + 0.5, torch.randn((N,), generator=g) * 0.1
    dq, eps = 3e-4, 1e-5
    xd, wd, rd, gd, bd = dev(x), dev(w), dev(res), dev(gamma), dev(beta)
    biasd = dev(bias) if with_bias else None

    acc = KL.linear_a8_w8_b32_o32(xd, wd, None)
    r_two, y_two = KF.dq_add_layernorm_q(acc, dq, rd, gd, bd, eps, bias_int32=biasd)
    r_one = KL.linear_a8_w8_b32_dq_add_ofp32(xd, wd, biasd, dq, rd)
    y_one = KF.layer_norm_fwd_fused_single_pass_q(r_one, gd, bd, eps)
    assert_status_clean()
    assert r_one.dtype == torch.float32 and r_one.shape == (M, N)
    assert torch.equal(r_one, r_two), "residual stream differs from dq_add_layernorm_q's"
    assert torch.equal(y_one, y_two), "int8 LayerNorm output differs from dq_add_layernorm_q's"

    acc_ref = O.acc_linear(x, w) + (bias if with_bias else 0)
    r_ref, f_ref = O.dq_add_layernorm_q_f32(acc_ref.to(torch.int32), dq, res, gamma, beta, eps)
    torch.testing.assert_close(r_one.cpu(), r_ref, rtol=1e-5, atol=1e-5)
    y_ref = f_ref.clamp(-128, 127).round().to(torch.int8)
    diff = (y_one.cpu().int() - y_ref.int()).abs()
    assert diff.max().item() <= 1 and (diff != 0).float().mean().item() < 2e-3


def test_dq_add_3d_activation_and_out():
    g = synthetic.gen(801)
    x, w = synthetic.int8_normal((2, 64, 256), 40, g), synthetic.int8_normal((512, 256), 30, g)
    res = torch.randn((2, 64, 512), generator=g)
    out = torch.empty((2, 64, 512), dtype=torch.float32, device="cuda")
    r = KL.linear_a8_w8_b32_dq_add_ofp32(dev(x), dev(w), None, torch.tensor(2e-4).cuda(), dev(res), out=out)
    assert r.shape == (2, 64, 512) and r.data_ptr() == out.data_ptr()
    ref = res + O.acc_linear(x.reshape(-1, 256), w).reshape(2, 64, 512).float() * 2e-4
    torch.testing.assert_close(r.cpu(), ref, rtol=1e-5, atol=1e-5)


def test_dq_add_refuses_what_it_cannot_address():
    x = torch.zeros((4, 50), dtype=torch.int8).cuda()      # K = 50: not addressable by tensor maps
    w = torch.zeros((8, 50), dtype=torch.int8).cuda()
    res = torch.zeros((4, 8)).cuda()
    with pytest.raises(RuntimeError):
        KL.linear_a8_w8_b32_dq_add_ofp32(x, w, None, 1e-3, res)
