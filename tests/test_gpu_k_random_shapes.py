"""Seeded random shapes through the automatic path selection (CTA-pair / single-CTA tcgen05,
split-K, NN layout, stride-agnostic fallback) against the CPU oracle, plus the torch.ops
registration under the reference's namespace."""
import random

import pytest
import torch

from oracle import ops as O
from triton_int_b200 import synthetic
from triton_int_b200.kernels import bmm as KB
from triton_int_b200.kernels import fused as KF  # noqa: F401  (registers its torch.ops entries)
from triton_int_b200.kernels import linear as KL
from util import assert_equal, assert_status_clean, dev

pytestmark = pytest.mark.gpu


def test_random_linear_shapes():
    rng = random.Random(7)
    g = synthetic.gen(7)
    for _ in range(24):
        m = rng.choice([1, 3, 17, 64, 130, 257, 300, 513, 1024])
        n = rng.choice([1, 8, 24, 100, 128, 200, 256, 384, 520])
        k = rng.choice([1, 16, 50, 64, 100, 128, 144, 256, 1000, 2048])
        x, w = synthetic.int8_normal((m, k), 40, g), synthetic.int8_normal((n, k), 40, g)
        bias = synthetic.int8_normal((n,), 40, g)
        a, b = torch.tensor(3e-4), torch.tensor(0.05)
        acc = KL.linear_a8_w8_b32_o32(dev(x), dev(w), None)
        y = KL.linear_a8_w8_b8_o8(dev(x), dev(w), dev(bias), dev(a), dev(b))
        assert_equal(acc, O.acc_linear(x, w), f"acc {m}x{n}x{k}")
        assert_equal(y, O.linear_a8_w8_b8_o8(x, w, bias, a, b, O.RNE_SAT), f"b8o8 {m}x{n}x{k}")
    assert_status_clean()


def test_random_bmm_shapes():
    rng = random.Random(8)
    g = synthetic.gen(8)
    for _ in range(12):
        bsz = rng.choice([1, 2, 5])
        m, n, k = rng.choice([7, 64, 129, 300]), rng.choice([16, 48, 130, 256, 272]), rng.choice([16, 64, 112, 160, 1024])
        a = synthetic.int8_normal((bsz, m, k), 30, g)
        bn = synthetic.int8_normal((bsz, n, k), 30, g)
        bt = bn.transpose(1, 2).contiguous()
        s = torch.tensor(1e-3)
        assert_equal(KB.bmm_s8t_s8n_s32t(dev(a), dev(bn)), O.bmm_s8t_s8n_s32t(a, bn), f"NT {bsz}x{m}x{n}x{k}")
        assert_equal(KB.bmm_s8t_s8t_s32t(dev(a), dev(bt)), O.bmm_s8t_s8t_s32t(a, bt), f"NN {bsz}x{m}x{n}x{k}")
        assert_equal(KB.bmm_s8t_s8n_f32t(dev(a), dev(bn), dev(s)), O.bmm_s8t_s8n_f32t(a, bn, s), f"NT f32 {bsz}x{m}x{n}x{k}")
    assert_status_clean()


def test_torch_ops_namespace():
    """The reference registers its wrappers under torch.ops.triton_op (kernels/__init__.py:5-24)."""
    g = synthetic.gen(9)
    x, w = synthetic.int8_normal((32, 128), 40, g), synthetic.int8_normal((64, 128), 40, g)
    bias = synthetic.int8_normal((64,), 40, g)
    a, b = torch.tensor(3e-4), torch.tensor(0.05)
    y = torch.ops.triton_op.linear_a8_w8_b8_o8(dev(x), dev(w), dev(bias), dev(a), dev(b))
    assert_equal(y, O.linear_a8_w8_b8_o8(x, w, bias, a, b, O.RNE_SAT), "torch.ops.triton_op.linear_a8_w8_b8_o8")
    ln = torch.ops.triton_op.layer_norm_fwd_fused_single_pass(torch.randn(4, 256).cuda(), torch.ones(256).cuda(),
                                                              torch.zeros(256).cuda(), 1e-5, False)
    assert ln.shape == (4, 256)
