"""Helpers shared by the GPU parity tests."""
import torch

from oracle import ops as O
from triton_int_b200 import _lib, config

MODES = {"trunc_wrap": O.TRUNC_WRAP, "rne_sat": O.RNE_SAT}


def dev(t):
    return None if t is None else t.cuda()


def assert_status_clean():
    assert _lib.device_status() == 0, "a bounded device-side wait expired"


def assert_equal(got, want, what=""):
    got = got.cpu()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert got.dtype == want.dtype, (what, got.dtype, want.dtype)
    if not torch.equal(got, want):
        bad = (got != want)
        idx = bad.nonzero()[:5].tolist()
        raise AssertionError(f"{what}: {bad.sum().item()} of {got.numel()} differ, first at {idx}: "
                             f"got {got[bad][:5].tolist()} want {want[bad][:5].tolist()}")


def assert_within_1lsb(got, want, max_rate, what=""):
    """int8 results that may differ by one step where a transcendental or a
    reduction order moved a value across a rounding boundary."""
    got = got.cpu().to(torch.int32)
    want = want.to(torch.int32)
    diff = (got - want).abs()
    # wrap-around neighbours (127 <-> -128) count as one step in trunc_wrap mode
    diff = torch.minimum(diff, 256 - diff)
    rate = (diff != 0).float().mean().item()
    assert diff.max().item() <= 1, f"{what}: max |diff| {diff.max().item()}"
    assert rate <= max_rate, f"{what}: mismatch rate {rate:.5f} > {max_rate}"
    return rate


def assert_close_rel(got, want, tol=1e-5, what=""):
    """|got - want| <= tol * max(1, |want|), the tolerance used for fp32 outputs."""
    got = got.detach().cpu().float()
    want = want.float()
    err = (got - want).abs() / want.abs().clamp_min(1.0)
    assert err.max().item() <= tol, f"{what}: max scaled error {err.max().item():.3e} > {tol}"


class gemm_path:
    def __init__(self, name):
        self.name = name

    def __enter__(self):
        self.prev = config.gemm_path()
        config.set_gemm_path(self.name)

    def __exit__(self, *exc):
        config._gemm_path = self.prev
