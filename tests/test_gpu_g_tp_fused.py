"""The fused exchange kernel on one GPU: the "ranks" are buffers on the same device, each
rank's launch covers its slice of the rows, and the result must equal the unfused
operator applied to the exact integer sum of the partial sums."""
import pytest
import torch

from triton_int_b200 import synthetic, tp
from triton_int_b200.kernels import fused as KF
from util import assert_status_clean

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,rows,n", [(1, 64, 1024), (2, 256, 4096), (4, 64, 768), (8, 128, 4096)])
def test_reduce_layernorm_q_matches_unfused(world, rows, n):
    g = synthetic.gen(90 + world)
    parts = [synthetic.int32_normal((rows, n), 2e4 / world, g).cuda() for _ in range(world)]
    residual = torch.randn((rows, n), generator=g).cuda()
    gamma = (torch.rand((n,), generator=g) * 20 + 5).cuda()
    beta = (torch.randn((n,), generator=g) * 2).cuda()
    bias = synthetic.int32_normal((n,), 1e3, g).cuda()
    outs = [torch.full((rows, n), 77, dtype=torch.int8, device="cuda") for _ in range(world)]
    res_out = torch.empty_like(residual)
    per = rows // world
    for r in range(world):  # one launch per emulated rank
        ro = tp.reduce_layernorm_q([p.data_ptr() for p in parts], [o.data_ptr() for o in outs], (r * per, per), n,
                                   residual[r * per:(r + 1) * per], gamma, beta, 1e-5, 1e-4, bias_int32=bias)
        res_out[r * per:(r + 1) * per] = ro
    total = parts[0].clone()
    for p in parts[1:]:
        total += p
    r_ref, y_ref = KF.dq_add_layernorm_q(total, 1e-4, residual, gamma, beta, 1e-5, bias_int32=bias)
    assert torch.equal(res_out, r_ref)
    for o in outs:  # every rank's copy of the gathered rows
        assert torch.equal(o, y_ref)
    assert_status_clean()


@pytest.mark.parametrize("world,rows,n,k", [(2, 256, 512, 256), (4, 512, 4096, 1024)])
def test_scatter_gemm_then_local_reduce(world, rows, n, k):
    """Emulated ranks on one GPU: every rank's K-shard GEMM scatters its tiles into the owners'
    receive buffers; each owner's reduce+LayerNorm over its slots equals the unsharded result."""
    from oracle import ops as O
    g = synthetic.gen(95 + world)
    x = synthetic.int8_normal((rows, k), 40, g)
    w = synthetic.int8_normal((n, k), 30, g)
    per, ks = rows // world, k // world
    recv = [torch.full((world, per, n), -5, dtype=torch.int32, device="cuda") for _ in range(world)]
    ptrs = [t.data_ptr() for t in recv]
    for r in range(world):
        tp.gemm_scatter(x[:, r * ks:(r + 1) * ks].contiguous().cuda(), w[:, r * ks:(r + 1) * ks].contiguous().cuda(),
                        ptrs, r, per)
    torch.cuda.synchronize()
    acc = O.acc_linear(x, w)
    for owner in range(world):
        total = recv[owner].sum(0, dtype=torch.int64).to(torch.int32)
        assert torch.equal(total.cpu(), acc[owner * per:(owner + 1) * per]), f"owner {owner}"
    residual = torch.randn((rows, n), generator=g).cuda()
    gamma = (torch.rand((n,), generator=g) * 20 + 5).cuda()
    outs = [torch.zeros((rows, n), dtype=torch.int8, device="cuda") for _ in range(world)]
    for owner in range(world):
        slots = [recv[owner][s].data_ptr() for s in range(world)]
        tp.reduce_layernorm_q(slots, [o.data_ptr() for o in outs], (owner * per, per), n,
                              residual[owner * per:(owner + 1) * per], gamma, None, 1e-5, 1e-4,
                              parts_row_begin=0, rank=owner)
    _, y_ref = KF.dq_add_layernorm_q(acc.cuda(), 1e-4, residual, gamma, None, 1e-5)
    for o in outs:
        assert torch.equal(o, y_ref)
    assert_status_clean()
