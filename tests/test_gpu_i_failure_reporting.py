"""Failure detection without a GPU fault: a bounded device-side wait that nothing satisfies
expires after its (short) limit, the kernel returns, the status word reports it, and the
context keeps working."""
import pytest
import torch

from triton_int_b200 import _lib, synthetic
from triton_int_b200.kernels import linear as KL

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_and_context_survives():
    lib = _lib.load()
    assert _lib.device_status() == 0
    rc = lib.ti_debug_expire_wait(2000, torch.cuda.current_stream().cuda_stream)  # 2 ms limit
    assert rc == _lib.TI_OK
    st = _lib.device_status()          # synchronises, reads and clears the word
    assert st & 4, f"status word {st:#x} does not report the expired wait"
    with pytest.raises(RuntimeError):
        lib.ti_debug_expire_wait(1000, torch.cuda.current_stream().cuda_stream)
        _lib.check(lib.ti_device_status(None), "status")     # TI_ERR_TIMEOUT maps to RuntimeError
    assert _lib.device_status() == 0   # cleared
    # the context is still usable: a real kernel runs and is correct
    x = synthetic.int8_normal((128, 128), 40, synthetic.gen(1)).cuda()
    w = synthetic.int8_normal((256, 128), 40, synthetic.gen(2)).cuda()
    acc = KL.linear_a8_w8_b32_o32(x, w, None)
    assert torch.equal(acc, (x.int().cpu() @ w.int().cpu().t()).cuda())
    assert _lib.device_status() == 0
