"""Fused int8 attention against the three-operator path of this library and the CPU oracle."""
import pytest
import torch

from oracle import ops as O
from triton_int_b200 import config, synthetic
from triton_int_b200.kernels import bmm as KB
from triton_int_b200.kernels import fused as KF
from util import assert_status_clean, dev

pytestmark = pytest.mark.gpu


def oracle_attention(q, k, v, a1, a2, causal, mode=O.RNE_SAT):
    """q [B,Sq,h,D], k/v [B,Sk,h,D] -> o [B,Sq,h,D] through the oracle's operators."""
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    qh = q.permute(0, 2, 1, 3).reshape(B * H, Sq, D)
    kh = k.permute(0, 2, 1, 3).reshape(B * H, Sk, D)
    vt = v.permute(0, 2, 3, 1).reshape(B * H, D, Sk)
    s = O.bmm_s8t_s8n_f32t(qh, kh, a1)
    if causal:
        p = O.causal_softmax_q(s, 127.0, mode)
    else:
        p = O.cast_i8(torch.softmax(s, -1) * 127.0, mode)
    o = O.bmm_s8t_s8n_s8t(p, vt, a2, mode)
    return o.view(B, H, Sq, D).permute(0, 2, 1, 3).contiguous(), p


def compare(o, o_ref, what, max_rate=0.03):
    d = (o.cpu().int() - o_ref.int()).abs()
    rate = (d != 0).float().mean().item()
    print(f"{what}: max |diff| {d.max().item()}, mismatch rate {rate:.5f}")
    # one step of P (1/127 of a probability) moves an output by at most alpha_pv * |v| <= ~1 step
    assert d.max().item() <= 2, f"{what}: max |diff| {d.max().item()}"
    assert rate <= max_rate, f"{what}: mismatch rate {rate}"


@pytest.mark.parametrize("B,H,S", [(1, 1, 128), (2, 3, 384), (1, 2, 200), (1, 1, 130), (2, 2, 1024)])
def test_fused_attention_causal(B, H, S):
    g = synthetic.gen(70 + S)
    q, k, v = (synthetic.int8_normal((B, S, H, 128), 30, g) for _ in range(3))
    a1, a2 = torch.tensor(1e-3), torch.tensor(8e-3)
    o = KF.attention_i8(dev(q), dev(k), dev(v), dev(a1), dev(a2), 127.0, causal=True)
    assert_status_clean()
    o_ref, _ = oracle_attention(q, k, v, a1, a2, True)
    compare(o, o_ref, f"fused vs oracle B{B} H{H} S{S}")
    # against this library's own three-operator path (same exp2-based softmax arithmetic)
    qh = dev(q).permute(0, 2, 1, 3).reshape(B * H, S, 128)
    kh = dev(k).permute(0, 2, 1, 3).reshape(B * H, S, 128)
    vt = dev(v).permute(0, 2, 3, 1).reshape(B * H, 128, S)
    p = KF.causal_softmax_q(KB.bmm_s8t_s8n_f32t(qh, kh, dev(a1)), 127.0)
    o3 = KB.bmm_s8t_s8n_s8t(p, vt, dev(a2)).view(B, H, S, 128).permute(0, 2, 1, 3)
    compare(o, o3.cpu(), f"fused vs three-operator path B{B} H{H} S{S}")


def test_fused_attention_noncausal_and_cross_lengths():
    g = synthetic.gen(77)
    q = synthetic.int8_normal((2, 256, 2, 128), 30, g)
    k = synthetic.int8_normal((2, 384, 2, 128), 30, g)
    v = synthetic.int8_normal((2, 384, 2, 128), 30, g)
    a1, a2 = torch.tensor(1e-3), torch.tensor(8e-3)
    o = KF.attention_i8(dev(q), dev(k), dev(v), dev(a1), dev(a2), 127.0, causal=False)
    assert_status_clean()
    compare(o, oracle_attention(q, k, v, a1, a2, False)[0], "non-causal Sq 256 Sk 384")
    o = KF.attention_i8(dev(q), dev(k), dev(v), dev(a1), dev(a2), 127.0, causal=True)
    assert_status_clean()
    compare(o, oracle_attention(q, k, v, a1, a2, True)[0], "causal with 128 cached keys")


def test_fused_attention_strided_qkv_and_trunc_wrap():
    """q, k, v as slices of one [T, 3H] projection buffer; truncate-and-wrap output cast."""
    g = synthetic.gen(78)
    B, S, H = 2, 256, 2
    qkv = synthetic.int8_normal((B * S, 3 * H * 128), 30, g)
    qkv_d = dev(qkv)
    views = [qkv_d[:, i * H * 128:(i + 1) * H * 128].view(B, S, H, 128) for i in range(3)]
    cpu = [qkv[:, i * H * 128:(i + 1) * H * 128].reshape(B, S, H, 128) for i in range(3)]
    a1, a2 = torch.tensor(1e-3), torch.tensor(2e-2)  # large alpha_pv: exercises saturation / wrap
    for mode, omode in (("rne_sat", O.RNE_SAT), ("trunc_wrap", O.TRUNC_WRAP)):
        with config.rounding(mode):
            o = KF.attention_i8(views[0], views[1], views[2], dev(a1), dev(a2), 127.0, causal=True)
        assert_status_clean()
        # P is quantised round-half-even in both modes; only the output cast follows the policy
        o_ref_p = oracle_attention(cpu[0], cpu[1], cpu[2], a1, a2, True, O.RNE_SAT)[1]
        vt = cpu[2].permute(0, 2, 3, 1).reshape(B * H, 128, S)
        o_ref = O.bmm_s8t_s8n_s8t(o_ref_p, vt, a2, omode).view(B, H, S, 128).permute(0, 2, 1, 3)
        d = (o.cpu().int() - o_ref.int()).abs()
        d = torch.minimum(d, 256 - d)
        rate = (d != 0).float().mean().item()
        print(f"strided qkv, {mode}: max diff {d.max().item()} rate {rate:.5f}")
        assert d.max().item() <= 3 and rate < 0.05
