"""Tensor-parallel host logic on CPU ranks (gloo, world size 2): each rank computes its
shard of the decoder block with the CPU oracle's operators, int32 partial sums are
all-reduced, and the result must equal the unsharded oracle bit for bit.  This
covers the sharding rules and the exact-integer exchange without a GPU."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import block as OB, ops as O
    from triton_int_b200 import synthetic
    from triton_int_b200.nn.decoder import shard_cols, shard_rows

    p = synthetic.config4_block(seed=3, hidden=128, heads=4, ffn=256, batch=2, seq=32)
    ref_res, ref_acc = OB.block_forward(p, p["residual"], p["prev_acc"], 2, 32)
    meta = p["meta"]
    h_local, d = meta["heads"] // world, meta["hidden"] // meta["heads"]
    res1, x8 = O.dq_add_layernorm_q(p["prev_acc"], p["prev_scale"], p["residual"], p["ln1_w"], p["ln1_b"], meta["eps"])

    def col_linear(name):
        return O.linear_a8_w8_b8_o8(x8, shard_rows(p[f"{name}_w"], rank, world), shard_rows(p[f"{name}_bias"], rank, world),
                                    p[f"{name}_alpha"], p[f"{name}_beta"], O.RNE_SAT)

    q, k, v = col_linear("q"), col_linear("k"), col_linear("v")
    hf = lambda t: t.view(2, 32, h_local, d).transpose(1, 2).reshape(2 * h_local, 32, d)
    vt = v.view(2, 32, h_local, d).permute(0, 2, 3, 1).reshape(2 * h_local, d, 32)
    pq = O.causal_softmax_q(O.bmm_s8t_s8n_f32t(hf(q), hf(k), p["qk_alpha"]), 127.0, O.RNE_SAT)
    o = O.bmm_s8t_s8n_s8t(pq, vt, p["pv_alpha"], O.RNE_SAT)
    attn = o.view(2, h_local, 32, d).transpose(1, 2).reshape(64, h_local * d)
    out_part = O.acc_linear(attn, shard_cols(p["out_w"], rank, world))          # raw int32 partial sums
    dist.all_reduce(out_part, op=dist.ReduceOp.SUM)                              # exact in any order
    out_acc = out_part + p["out_bias"][None, :]                                  # bias once, after the reduction
    res2, h8 = O.dq_add_layernorm_q(out_acc, p["out_scale"], res1, p["ln2_w"], p["ln2_b"], meta["eps"])
    g8 = O.linear_a8_w8_bfp32_ofp32_GeLu_Q(h8, shard_rows(p["fc1_w"], rank, world), shard_rows(p["fc1_bias"], rank, world),
                                           p["fc1_alpha"], p["fc1_mul"], O.RNE_SAT)
    fc2 = O.acc_linear(g8, shard_cols(p["fc2_w"], rank, world))
    dist.all_reduce(fc2, op=dist.ReduceOp.SUM)
    ok = torch.equal(res2, ref_res) and torch.equal(fc2, ref_acc)
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        out.put(int(flag.item()))
    dist.destroy_process_group()


def test_two_rank_block_equals_single_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=240)
        assert pr.exitcode == 0
    assert q.get(timeout=5) == 1
