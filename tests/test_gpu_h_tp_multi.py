"""Two real ranks (two GPUs, NCCL + symmetric memory): the fused tensor-parallel step must
reproduce the single-GPU block bit for bit.  Skipped where fewer than two GPUs are visible."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _rank_main(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from triton_int_b200 import synthetic, tp
    from triton_int_b200.nn.decoder import Int8DecoderBlock

    p = synthetic.config4_block(seed=3, hidden=256, heads=4, ffn=1024, batch=2, seq=128)
    t, h = 256, 256
    single = Int8DecoderBlock(p).to(dev)
    r_ref, a_ref = single(p["residual"].to(dev), p["prev_acc"].to(dev), 2, 128)
    blk = Int8DecoderBlock(p, rank=rank, world=world).to(dev)
    bufs = tp.SymmetricBuffers(dist.group.WORLD, t, h, dev)
    r0, rc = bufs.rank_rows()
    if rank == 0:
        bufs.partial[0][0].copy_(p["prev_acc"].to(dev))
    else:
        bufs.partial[0][0].zero_()
    torch.cuda.synchronize()
    dist.barrier()
    res = blk.forward_tp_fused(p["residual"].to(dev)[r0:r0 + rc].contiguous(), bufs, 2, 128)
    bufs.barrier()
    total = bufs.partial[0][0].clone()
    dist.all_reduce(total)  # sum of the fc2 partial sums
    ok = torch.equal(res, r_ref[r0:r0 + rc]) and torch.equal(total, a_ref)
    # the push form: GEMM tiles scattered into the owners' receive buffers
    bufs2 = tp.SymmetricBuffers(dist.group.WORLD, t, h, dev)
    bufs2.partial[0][0].zero_()
    if rank == 0:  # previous block's slices: everything in slot 0 of each owner
        pass
    bufs2.partial[0][0].view(world, rc, h)[0].copy_(p["prev_acc"].to(dev)[r0:r0 + rc])
    torch.cuda.synchronize()
    dist.barrier()
    res_p = blk.forward_tp_push(p["residual"].to(dev)[r0:r0 + rc].contiguous(), bufs2, 2, 128)
    bufs2.barrier()
    mine = bufs2.partial[0][0].view(world, rc, h).sum(0, dtype=torch.int64).to(torch.int32)  # this rank's rows of fc2
    ok = ok and torch.equal(res_p, r_ref[r0:r0 + rc]) and torch.equal(mine, a_ref[r0:r0 + rc])
    # the copy-engine form
    bufs3 = tp.SymmetricBuffers(dist.group.WORLD, t, h, dev)
    bufs3.partial[0][0].zero_()
    bufs3.partial[0][0].view(world, rc, h)[0].copy_(p["prev_acc"].to(dev)[r0:r0 + rc])
    torch.cuda.synchronize()
    dist.barrier()
    cs = torch.cuda.Stream(dev)
    res_d = blk.forward_tp_dma(p["residual"].to(dev)[r0:r0 + rc].contiguous(), bufs3, 2, 128, cs)
    torch.cuda.current_stream().wait_stream(cs)
    bufs3.barrier()
    mine_d = bufs3.partial[0][0].view(world, rc, h).sum(0, dtype=torch.int64).to(torch.int32)
    ok = ok and torch.equal(res_d, r_ref[r0:r0 + rc]) and torch.equal(mine_d, a_ref[r0:r0 + rc])
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        out.put(int(flag.item()))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_tp_step_equals_single_gpu():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() % 200)
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=240)
        assert pr.exitcode == 0
    assert q.get(timeout=5) == 1
