"""GPU activation quantisers against the reference's torch helpers (functional/quantization.py)."""
import pytest
import torch

from triton_int_b200.functional import quantization as Q
from util import assert_status_clean

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(37, 768), (4, 9, 4096), (3, 20)])
def test_per_token_matches_torch_helper(dtype, shape):
    g = torch.Generator().manual_seed(5)
    t = (torch.randn(shape, generator=g) * 3).to(dtype).cuda()
    t[0, ..., :] = 0  # an all-zero row exercises the 1e-8 floor
    q, s = Q.dynamic_quantize_activation_per_token_absmax_cuda(t)
    q_ref, s_ref = Q.dynamic_quantize_activation_per_token_absmax(t.clone())  # the helper overwrites its input
    assert s.dtype == dtype and s.shape == s_ref.shape
    assert torch.equal(s, s_ref), (s - s_ref).abs().max()
    assert torch.equal(q, q_ref), f"{(q != q_ref).sum().item()} of {q.numel()} differ"
    assert_status_clean()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_per_tensor_matches_torch_helpers(dtype):
    g = torch.Generator().manual_seed(6)
    t = (torch.randn((513, 1031), generator=g) * 2).to(dtype).cuda()
    q, s = Q.dynamic_quantize_activation_per_tensor_absmax_cuda(t)
    q_ref, s_ref = Q.dynamic_quantize_activation_per_tensor_absmax(t.clone())
    assert torch.equal(s.float(), s_ref.float()) and torch.equal(q, q_ref)
    q2, s2 = Q.quantize_per_tensor_absmax_cuda(t)
    q2_ref, s2_ref = Q.quantize_per_tensor_absmax(t.clone())
    assert torch.equal(s2.float(), s2_ref.float()) and torch.equal(q2, q2_ref)
    assert_status_clean()
