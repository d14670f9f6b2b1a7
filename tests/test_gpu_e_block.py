"""Decoder block (the benchmark workload) against the CPU oracle composition, and the
tensor-parallel shards emulated on one GPU: partial sums of every rank are added
exactly and must reproduce the single-GPU block bit for bit."""
import pytest
import torch

from oracle import block as OB
from oracle import ops as O
from triton_int_b200 import synthetic
from triton_int_b200.nn.decoder import Int8DecoderBlock
from util import assert_equal, assert_status_clean, assert_within_1lsb

pytestmark = pytest.mark.gpu


def small_params():
    return synthetic.config4_block(seed=3, hidden=256, heads=4, ffn=1024, batch=2, seq=128)


def test_block_stages_vs_oracle():
    p = small_params()
    blk = Int8DecoderBlock(p).cuda()
    stages = {}
    r_ref, a_ref = OB.block_forward(p, p["residual"], p["prev_acc"], 2, 128, stages=stages)
    # stage by stage, each fed with the oracle's input to that stage
    from triton_int_b200.kernels import fused as KF, linear as KL
    res1, x8 = KF.dq_add_layernorm_q(p["prev_acc"].cuda(), blk.prev_scale, p["residual"].cuda(), blk.ln1_w, blk.ln1_b, blk.eps)
    assert_equal(res1, stages["res1"], "res1")
    assert_within_1lsb(x8, stages["x8"], 0.01, "x8")
    attn = blk.attention(stages["x8"].cuda(), 2, 128)
    assert_within_1lsb(attn, stages["attn"], 0.02, "attention output")
    out_acc = KL.linear_a8_w8_b32_o32(stages["attn"].cuda(), blk.out_w, blk.out_bias)
    assert_equal(out_acc, stages["out_acc"], "out_proj accumulators")
    g8 = KF.linear_a8_w8_bfp32_ofp32_GeLu_Q(stages["h8"].cuda(), blk.fc1_w, blk.fc1_bias, blk.fc1_alpha, blk.fc1_mul)
    assert_within_1lsb(g8, stages["g8"], 5e-3, "fc1 gelu-q")
    fc2 = KL.linear_a8_w8_b32_o32(stages["g8"].cuda(), blk.fc2_w, None)
    assert_equal(fc2, a_ref, "fc2 accumulators")
    # end to end
    res2, acc = blk(p["residual"].cuda(), p["prev_acc"].cuda(), 2, 128)
    err = ((res2.cpu() - r_ref).abs() / r_ref.abs().clamp_min(1.0))
    rate = (acc.cpu() != a_ref).float().mean().item()
    print(f"block end to end: residual max scaled err {err.max().item():.2e}, accumulator mismatch rate {rate:.5f}")
    assert err.max().item() < 1e-2 and rate < 0.02
    assert_status_clean()


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_shards_are_exact(world):
    """Run every rank's shard on this GPU in turn; the reduction hook sums the int32
    partials of all ranks (what the NCCL all-reduce does).  Must equal world == 1."""
    p = small_params()
    residual, prev = p["residual"].cuda(), p["prev_acc"].cuda()
    single = Int8DecoderBlock(p).cuda()
    r1, a1 = single(residual, prev, 2, 128)

    # lock-step emulation: stage A on all ranks, reduce, stage B on all ranks, reduce
    from triton_int_b200.kernels import fused as KF, linear as KL
    blocks = [Int8DecoderBlock(p, rank=r, world=world).cuda() for r in range(world)]
    res1, x8 = KF.dq_add_layernorm_q(prev, blocks[0].prev_scale, residual, blocks[0].ln1_w, blocks[0].ln1_b, 1e-5)
    out_acc = sum(KL.linear_a8_w8_b32_o32(b.attention(x8, 2, 128), b.out_w, None) for b in blocks)
    res2, h8 = KF.dq_add_layernorm_q(out_acc, blocks[0].out_scale, res1, blocks[0].ln2_w, blocks[0].ln2_b, 1e-5,
                                     bias_int32=blocks[0].out_bias)
    fc2 = sum(KL.linear_a8_w8_b32_o32(
        KF.linear_a8_w8_bfp32_ofp32_GeLu_Q(h8, b.fc1_w, b.fc1_bias, b.fc1_alpha, b.fc1_mul), b.fc2_w, None)
        for b in blocks)
    assert torch.equal(res2, r1), "residual stream differs between 1 and %d ranks" % world
    assert torch.equal(fc2, a1), "fc2 accumulators differ between 1 and %d ranks" % world
    assert_status_clean()
