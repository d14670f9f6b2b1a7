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
