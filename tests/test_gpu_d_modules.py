"""Module-level drop-in checks: the nn classes reproduce the functional wrappers,
keep the reference's buffer names, and their from_float constructors work on GPU."""
import pytest
import torch

from oracle import ops as O
from triton_int_b200 import config, synthetic
from triton_int_b200.nn import bmm as NB
from triton_int_b200.nn import fused as NF
from triton_int_b200.nn import linear as NL
from util import assert_equal, assert_status_clean, assert_within_1lsb, dev

pytestmark = pytest.mark.gpu


def test_linear_modules_match_oracle():
    g = synthetic.gen(61)
    x = synthetic.int8_normal((2, 9, 256), 40, g)
    for cls, ref, bias_dtype in [
        (NL.W8A8B8O8Linear, lambda m: O.linear_a8_w8_b8_o8(x, m.weight.cpu(), m.bias.cpu(), m.a.cpu(), m.b.cpu(), O.RNE_SAT), torch.int8),
        (NL.W8A8B8O8LinearReLU, lambda m: O.linear_relu_a8_w8_b8_o8(x, m.weight.cpu(), m.bias.cpu(), m.a.cpu(), m.b.cpu(), O.RNE_SAT), torch.int8),
        (NL.W8A8B32O32Linear, lambda m: O.linear_a8_w8_b32_o32_with_scaling(x, m.weight.cpu(), m.bias.cpu(), m.a.cpu(), m.b.cpu()), torch.int32),
        (NL.W8A8BFP32OFP32Linear, lambda m: O.linear_a8_w8_bfp32_ofp32(x, m.weight.cpu(), m.bias.cpu(), m.a.cpu(), m.b.cpu()), torch.float32),
    ]:
        m = cls(256, 96, alpha=0.002, beta=0.5)
        m.bias = (torch.randn(96, generator=g) * 20).to(bias_dtype)
        assert list(m.state_dict().keys()) == ["weight", "bias", "a", "b"]
        m = m.cuda()
        y = m(dev(x))
        assert y.shape == (2, 9, 96)
        assert_equal(y, ref(m), cls.__name__)
    m = NL.W8A8B32O32LinearWithoutScaling(256, 96).cuda()
    assert_equal(m(dev(x)), O.linear_a8_w8_b32_o32(x, m.weight.cpu(), m.bias.cpu()), "without scaling")
    assert_status_clean()


def test_from_float_and_state_dict_roundtrip():
    torch.manual_seed(0)
    lin = torch.nn.Linear(128, 64)
    q = NL.W8A8B8O8Linear.from_float(lin, 0.05, 0.1).cuda()
    sd = q.state_dict()
    q2 = NL.W8A8B8O8Linear(128, 64).cuda()
    q2.load_state_dict(sd)
    x = synthetic.int8_normal((5, 128), 40, synthetic.gen(62)).cuda()
    assert torch.equal(q(x), q2(x))
    f = NL.W8A8BFP32OFP32Linear.from_float(torch.nn.Linear(128, 64), 0.05).cuda()
    assert f(x).dtype == torch.float32
    d = NL.DynamicW8A8BFP32OFP32Linear.from_float(torch.nn.Linear(128, 64)).cuda()
    assert d(torch.randn(5, 128).cuda()).shape == (5, 64)
    ge = NF.W8A8BFP32OFP32_GeLu_Q.from_float(torch.nn.Linear(128, 64), 0.05, 0.02).cuda()
    assert ge(x).dtype == torch.int8
    assert_status_clean()


def test_layernorm_modules():
    g = synthetic.gen(63)
    ln = torch.nn.LayerNorm(512)
    ln.weight.data = torch.rand(512, generator=g) + 0.5
    ln.bias.data = torch.randn(512, generator=g) * 0.1
    q = NF.LayerNormQ.from_float(ln, 0.05).cuda()
    qt = NF._LayerNormQ.from_float(ln, 0.05)
    x = torch.randn((3, 7, 512), generator=g)
    assert_within_1lsb(q(dev(x)), qt(x), 0.01, "LayerNormQ vs torch form")
    m = NF.DQ_Add_LayerNorm_Q(512).cuda()
    m.weight, m.bias = q.weight, q.bias
    m.input_scale = 1e-4
    acc = synthetic.int32_normal((3, 7, 512), 2e4, g)
    r, y = m(dev(x), dev(acc))
    r_ref, y_ref = O.dq_add_layernorm_q(acc, 1e-4, x, q.weight.cpu(), q.bias.cpu(), 1e-5)
    assert_equal(r, r_ref, "residual")
    assert_within_1lsb(y, y_ref, 0.01, "DQ_Add_LayerNorm_Q")
    gq = NF.GeLu_Q(alpha=50.0, input_scale=0.03).cuda()
    xi = synthetic.int8_normal((4, 1000), 40, g)
    assert_within_1lsb(gq(dev(xi)), O.gelu_q(xi, 0.03, 50.0, O.RNE_SAT), 1e-3, "GeLu_Q")
    assert_status_clean()


def test_bmm_modules():
    g = synthetic.gen(64)
    a = synthetic.int8_normal((2, 40, 64), 30, g)
    b = synthetic.int8_normal((2, 24, 64), 30, g)
    m = NB.BMM_S8T_S8N_S8T.from_scale(0.1, 0.2, 5.0).cuda()
    assert_equal(m(dev(a), dev(b)), O.bmm_s8t_s8n_s8t(a, b, m.a.cpu(), O.RNE_SAT), "BMM_S8T_S8N_S8T")
    f = NB.BMM_S8T_S8N_F32T.from_scale(0.1, 0.2).cuda()
    assert_equal(f(dev(a), dev(b)), O.bmm_s8t_s8n_f32t(a, b, f.a.cpu()), "BMM_S8T_S8N_F32T")
    h = NB.BMM_S8T_S8N_F16T.from_scale(0.1, 0.2).cuda()
    assert h(dev(a), dev(b)).dtype == torch.float16
    bt = b.transpose(1, 2).contiguous()
    t = NB.BMM_S8T_S8T_S8T.from_scale(0.1, 0.2, 5.0).cuda()
    assert_equal(t(dev(a), dev(bt)), O.bmm_s8t_s8t_s8t(a, bt, t.a.cpu(), O.RNE_SAT), "BMM_S8T_S8T_S8T")
    assert_equal(NB.BMM_S8T_S8N_S32T()(dev(a), dev(b)), O.bmm_s8t_s8n_s32t(a, b), "BMM_S8T_S8N_S32T")
    assert_status_clean()
