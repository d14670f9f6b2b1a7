"""GPU parity of the tcgen05 GEMM / BMM kernel: golden vectors from the reference,
oracle comparisons on seeded inputs, and size-independent checks at full size."""
import pytest
import torch

from oracle import ops as O
from triton_int_b200 import config, synthetic
from triton_int_b200.kernels import bmm as KB
from triton_int_b200.kernels import fused as KF
from triton_int_b200.kernels import linear as KL
from test_gpu_b_gemm_generic import run_bmm_golden, run_linear_golden
from util import assert_equal, assert_status_clean, assert_within_1lsb, dev, gemm_path

pytestmark = pytest.mark.gpu
T = torch.from_numpy


def test_first_tile_exact():
    """One 128x256x128 problem: a single tile, a single stage."""
    g = synthetic.gen(21)
    x, w = synthetic.int8_normal((128, 128), 40, g), synthetic.int8_normal((256, 128), 40, g)
    with gemm_path("tcgen05"):
        acc = KL.linear_a8_w8_b32_o32(dev(x), dev(w), None)
    assert_status_clean()
    assert_equal(acc, O.acc_linear(x, w), "single tile")


@pytest.mark.parametrize("case", ["ragged", "m1", "lead3d"])
def test_linear_golden(golden, case):
    with gemm_path("tcgen05"):
        run_linear_golden(golden["linear"], case)


def test_bmm_golden(golden):
    # K = 64 and N = 56... rows: the NT operators take the tensor-map path; the NN ("s8t_s8t")
    # operand of the small case has 56-byte rows and stays on the stride-agnostic kernel
    with gemm_path("tcgen05"):
        run_bmm_golden(golden["bmm"], "small", nn_too=False)


@pytest.mark.parametrize("B,M,N,K", [(3, 200, 256, 320), (2, 130, 48, 112), (1, 128, 384, 2048)])
def test_bmm_nn_layout_on_tensor_cores(B, M, N, K):
    """bmm_s8t_s8t_*: second operand [B, K, N] (N contiguous) read as an MN-major tile."""
    g = synthetic.gen(33 + N)
    a = synthetic.int8_normal((B, M, K), 30, g)
    bt = synthetic.int8_normal((B, K, N), 30, g)
    sc = torch.tensor(2e-3)
    with gemm_path("tcgen05"):
        acc = KB.bmm_s8t_s8t_s32t(dev(a), dev(bt))
        y8 = KB.bmm_s8t_s8t_s8t(dev(a), dev(bt), dev(sc))
    assert_status_clean()
    assert_equal(acc, O.bmm_s8t_s8t_s32t(a, bt), "NN accumulators")
    assert_equal(y8, O.bmm_s8t_s8t_s8t(a, bt, sc, O.RNE_SAT), "NN int8")


def test_unaligned_is_refused_when_forced():
    x = torch.zeros((4, 50), dtype=torch.int8).cuda()
    w = torch.zeros((8, 50), dtype=torch.int8).cuda()
    with gemm_path("tcgen05"):
        with pytest.raises(RuntimeError):
            KL.linear_a8_w8_b32_o32(x, w, None)
    y = KL.linear_a8_w8_b32_o32(x, w, None)  # auto falls back to the stride-agnostic kernel
    assert (y == 0).all()


def test_config1(golden):
    g = golden["config1"]
    c = synthetic.config1_linear(seed=0)
    x, w, bias = dev(c["x"]), dev(c["w"]), dev(c["bias"])
    with gemm_path("tcgen05"):
        with config.rounding("trunc_wrap"):
            y = KL.linear_a8_w8_b8_o8(x, w, bias, dev(c["alpha"]), dev(c["beta"]))
        with config.rounding("rne_sat"):
            ys = KL.linear_a8_w8_b8_o8(x, w, bias, dev(c["alpha"]), dev(c["beta"]))
        acc = KL.linear_a8_w8_b32_o32(x, w, None)
    assert_status_clean()
    assert_equal(acc, O.acc_linear(c["x"], c["w"]), "config1 accumulators")
    assert_equal(y, T(g["y"]), "config1 trunc_wrap vs reference")
    assert_equal(ys, O.linear_a8_w8_b8_o8(c["x"], c["w"], c["bias"], c["alpha"], c["beta"], O.RNE_SAT), "config1 rne_sat")


@pytest.mark.parametrize("m,n,k", [(300, 520, 1040), (1, 4608, 9216), (16, 3456, 9216), (129, 257, 144),
                                   (1024, 64, 4096), (640, 96, 128)])
def test_accumulators_vs_oracle(m, n, k):
    g = synthetic.gen(22 + m)
    x, w = synthetic.int8_normal((m, k), 35, g), synthetic.int8_normal((n, k), 35, g)
    bias = synthetic.int32_normal((n,), 1e4, g)
    with gemm_path("tcgen05"):
        acc = KL.linear_a8_w8_b32_o32(dev(x), dev(w), dev(bias))
    assert_status_clean()
    assert_equal(acc, O.linear_a8_w8_b32_o32(x, w, bias), f"acc {m}x{n}x{k}")


@pytest.mark.parametrize("mode", ["rne_sat", "trunc_wrap"])
def test_epilogues_vs_oracle(mode):
    from util import MODES
    g = synthetic.gen(31)
    m, n, k = 520, 1000, 2048
    x, w = synthetic.int8_normal((m, k), 35, g), synthetic.int8_normal((n, k), 35, g)
    b8 = synthetic.int8_normal((n,), 35, g)
    bf = torch.randn((n,), generator=g)
    a, b = torch.tensor(2e-4), torch.tensor(0.02)
    with gemm_path("tcgen05"), config.rounding(mode):
        y8 = KL.linear_a8_w8_b8_o8(dev(x), dev(w), dev(b8), dev(a), dev(b))
        yr = KL.linear_relu_a8_w8_b8_o8(dev(x), dev(w), dev(b8), dev(a), dev(b))
        yf = KL.linear_a8_w8_bfp32_ofp32(dev(x), dev(w), dev(bf), dev(a), dev(b))
        yb = KL.linear_a8_w8_bfp32_ofp32(dev(x), dev(w), dev(bf).bfloat16(), dev(a), dev(b))
        yg = KF.linear_a8_w8_bfp32_ofp32_GeLu_Q(dev(x), dev(w), dev(bf), dev(a), torch.tensor(1 / 0.02).cuda())
    assert_status_clean()
    assert_equal(y8, O.linear_a8_w8_b8_o8(x, w, b8, a, b, MODES[mode]), "b8_o8")
    assert_equal(yr, O.linear_relu_a8_w8_b8_o8(x, w, b8, a, b, MODES[mode]), "relu")
    assert_equal(yf, O.linear_a8_w8_bfp32_ofp32(x, w, bf, a, b), "bfp32")
    assert_equal(yb, O.linear_a8_w8_bfp32_ofp32(x, w, bf.bfloat16(), a, b), "bbf16")
    assert_within_1lsb(yg, O.linear_a8_w8_bfp32_ofp32_GeLu_Q(x, w, bf, a, torch.tensor(1 / 0.02), MODES[mode]), 2e-3, "gelu_q")


def test_bmm_attention_shapes():
    """Config-3 layout at reduced batch: QK^T -> fp32, causal softmax -> int8, PV -> int8."""
    c = synthetic.config3_attention(seed=2, bh=4, seq=384, head_dim=128)
    q, k, v = c["q"], c["k"], c["v"]
    vt = v.transpose(1, 2).contiguous()
    with gemm_path("tcgen05"):
        s = KB.bmm_s8t_s8n_f32t(dev(q), dev(k), dev(c["alpha_qk"]))
        s_c = KB.bmm_s8t_s8n_f32t(dev(q), dev(k), dev(c["alpha_qk"]), causal=True)
        p = KF.causal_softmax_q(s, c["p_mul"])
        p_c = KF.causal_softmax_q(s_c, c["p_mul"])
        o = KB.bmm_s8t_s8n_s8t(p, dev(vt), dev(c["alpha_pv"]))
        acc = KB.bmm_s8t_s8n_s32t(p, dev(vt))
    assert_status_clean()
    assert_equal(s, O.bmm_s8t_s8n_f32t(q, k, c["alpha_qk"]), "QK^T")
    assert torch.equal(p, p_c), "skipping masked score tiles must not change P"
    p_ref = O.causal_softmax_q(O.bmm_s8t_s8n_f32t(q, k, c["alpha_qk"]), c["p_mul"], O.RNE_SAT)
    assert_within_1lsb(p, p_ref, 0.01, "P")
    # PV from the kernel's own P: exact
    assert_equal(acc, O.bmm_s8t_s8n_s32t(p.cpu(), vt), "PV accumulators")
    assert_equal(o, O.bmm_s8t_s8n_s8t(p.cpu(), vt, c["alpha_pv"], O.RNE_SAT), "PV int8")


def test_strided_batch_and_rows():
    """Row and batch strides larger than the extents (views into wider buffers)."""
    g = synthetic.gen(41)
    big_a = synthetic.int8_normal((3, 200, 256), 30, g)
    big_b = synthetic.int8_normal((3, 150, 256), 30, g)
    a, b = big_a[:, :130, :192], big_b[:, :70, :192]
    with gemm_path("tcgen05"):
        acc = KB.bmm_s8t_s8n_s32t(dev(big_a)[:, :130, :192], dev(big_b)[:, :70, :192])
    assert_status_clean()
    assert_equal(acc, O.bmm_s8t_s8n_s32t(a.contiguous(), b.contiguous()), "strided bmm")


def test_full_size_properties():
    """M = N = K = 4096-class problem: tcgen05 against the stride-agnostic kernel
    bit for bit, plus the column-sum identity sum_n acc[m,n] = x[m,:] . sum_n W[n,:]."""
    g = synthetic.gen(51)
    m, n, k = 4096, 4096, 4096
    x, w = synthetic.int8_normal((m, k), 40, g), synthetic.int8_normal((n, k), 30, g)
    xd, wd = dev(x), dev(w)
    with gemm_path("tcgen05"):
        acc = KL.linear_a8_w8_b32_o32(xd, wd, None)
    with gemm_path("generic"):
        acc_g = KL.linear_a8_w8_b32_o32(xd, wd, None)
    assert_status_clean()
    assert torch.equal(acc, acc_g)
    want = (x.double() @ w.double().sum(0)).to(torch.int64)
    assert torch.equal(acc.sum(dim=1, dtype=torch.int64).cpu(), want)
    # linearity in the activations: acc(x1 + x2) = acc(x1) + acc(x2) for small-range inputs
    x1 = (x // 2)
    x2 = x - x1
    with gemm_path("tcgen05"):
        a1 = KL.linear_a8_w8_b32_o32(dev(x1), wd, None)
        a2 = KL.linear_a8_w8_b32_o32(dev(x2), wd, None)
    assert torch.equal(a1 + a2, acc)


@pytest.mark.parametrize("m", [1, 16, 128])
def test_split_k_small_m(m):
    """Config-5 weight-streaming shapes: K is split over CTAs, partial sums meet in a scratch
    buffer and the second kernel applies the epilogue; results equal the oracle."""
    from triton_int_b200 import _lib
    c = synthetic.config5_linear(seed=4, m=m, layer="fc1")
    x, w = c["x"], c["w"]
    with gemm_path("tcgen05"):
        before = _lib.launch_count()
        acc = KL.linear_a8_w8_b32_o32(dev(x), dev(w), None)
        assert _lib.launch_count() - before == 2, "expected the two-kernel split-K form"
        y8 = KL.linear_a8_w8_b8_o8(dev(x), dev(w), dev(c["bias_i8"]), dev(c["alpha"]), dev(c["beta"]))
        yf = KL.linear_a8_w8_bfp32_ofp32(dev(x), dev(w), dev(c["bias_f32"]), dev(c["alpha"]), dev(c["beta"]))
        yg = KF.linear_a8_w8_bfp32_ofp32_GeLu_Q(dev(x), dev(w), dev(c["bias_f32"]), dev(c["alpha"]), torch.tensor(50.0).cuda())
    assert_status_clean()
    assert_equal(acc, O.acc_linear(x, w), "split-K accumulators")
    assert_equal(y8, O.linear_a8_w8_b8_o8(x, w, c["bias_i8"], c["alpha"], c["beta"], O.RNE_SAT), "split-K b8_o8")
    assert_equal(yf, O.linear_a8_w8_bfp32_ofp32(x, w, c["bias_f32"], c["alpha"], c["beta"]), "split-K bfp32")
    assert_within_1lsb(yg, O.linear_a8_w8_bfp32_ofp32_GeLu_Q(x, w, c["bias_f32"], c["alpha"], torch.tensor(50.0), O.RNE_SAT), 2e-3, "split-K gelu_q")
