"""Tensor-parallel plumbing for one node: peer-mapped buffers and the fused
reduce-scatter -> dequant+bias+residual+LayerNorm+quant -> all-gather launch.

One process per GPU.  ``torch.distributed`` (NCCL) is the control plane;
the int32 partial sums and the gathered int8 activations live in symmetric
memory (``torch.distributed._symmetric_memory``), which gives every rank a device
pointer to every peer's buffer over NVLink.  The data path is this library's own
kernel (``ti_tp_reduce_layernorm_q``): plain peer loads and stores, no TMA, no
multicast.  Ordering between ranks is a device-side barrier on the current stream.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib, config
from .kernels._gemm import scale_tensor


def reduce_layernorm_q(parts_ptrs, outs_ptrs, rank_rows, n, residual_in, gamma, beta, eps, dq_scale,
                       bias_int32=None, want_residual_out=True):
    """Launch the fused kernel for this rank's rows.

    parts_ptrs / outs_ptrs: device pointers (ints), one per rank, of the [rows, n]
    int32 partial-sum buffers and the [rows, n] int8 output buffers as mapped in
    this process.  rank_rows = (row_begin, row_count).  residual_in: fp32
    [row_count, n] (this rank's slice).  Returns residual_out (fp32 [row_count, n])."""
    _lib.require_cuda(residual_in, gamma, beta, bias_int32)
    world = len(parts_ptrs)
    assert world == len(outs_ptrs) and 1 <= world <= 8
    row_begin, row_count = rank_rows
    dev = residual_in.device
    residual_in = residual_in.contiguous()
    assert residual_in.dtype == torch.float32 and residual_in.shape == (row_count, n)
    res_out = torch.empty_like(residual_in) if want_residual_out else None
    p = _lib.TpReduceLnParams()
    for r in range(world):
        p.parts[r] = parts_ptrs[r]
        p.outs[r] = outs_ptrs[r]
    p.residual_in = residual_in.data_ptr()
    p.residual_out = res_out.data_ptr() if res_out is not None else None
    keep = [gamma.contiguous()]
    p.gamma = keep[0].data_ptr()
    if beta is not None:
        keep.append(beta.contiguous())
        p.beta = keep[-1].data_ptr()
    if bias_int32 is not None:
        keep.append(bias_int32.contiguous())
        p.bias_i32 = keep[-1].data_ptr()
    if torch.is_tensor(dq_scale):
        keep.append(scale_tensor(dq_scale, dev))
        p.dq_scale_dev = keep[-1].data_ptr()
    else:
        p.dq_scale = float(dq_scale)
    p.row_begin, p.row_count, p.n = row_begin, row_count, n
    p.eps = float(eps)
    p.world = world
    p.rounding = config.rounding_mode()
    with torch.cuda.device(dev):
        p.stream = _lib.current_stream_ptr(dev)
        rc = _lib.load().ti_tp_reduce_layernorm_q(C.byref(p))
    _lib.check(rc, "ti_tp_reduce_layernorm_q")
    return res_out


class SymmetricBuffers:
    """[rows, n] int32 partial-sum buffers and int8 activation buffers that every
    rank of ``group`` can address, plus a stream-ordered barrier."""

    def __init__(self, group, rows, n, device, num_partial=2, num_act=2):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.group, self.rows, self.n = group, rows, n
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert rows % self.world == 0, "rows must divide evenly over the ranks"
        self.partial, self.act, self._handles = [], [], []
        for _ in range(num_partial):
            t = symm.empty((rows, n), dtype=torch.int32, device=device)
            h = symm.rendezvous(t, group)
            self.partial.append((t, [int(x) for x in h.buffer_ptrs]))
            self._handles.append(h)
        for _ in range(num_act):
            t = symm.empty((rows, n), dtype=torch.int8, device=device)
            h = symm.rendezvous(t, group)
            self.act.append((t, [int(x) for x in h.buffer_ptrs]))
            self._handles.append(h)
        # pad of flags for this library's own bounded barrier
        pad = symm.empty((8,), dtype=torch.int32, device=device)
        pad.zero_()
        ph = symm.rendezvous(pad, group)
        self._pad, self._pad_ptrs = pad, (C.c_void_p * 8)(*[int(x) for x in ph.buffer_ptrs])
        self._handles.append(ph)
        self._epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every pad is zeroed before anyone's first device barrier

    def rank_rows(self):
        per = self.rows // self.world
        return self.rank * per, per

    def barrier(self):
        """All ranks' streams have reached this point before any proceeds (bounded wait on
        the device; an expired wait shows up in ``triton_int_b200.device_status()``)."""
        self._epoch += 1
        dev = self._pad.device
        with torch.cuda.device(dev):
            rc = _lib.load().ti_tp_barrier(self._pad_ptrs, self.world, self.rank, self._epoch & 0xFFFFFFFF,
                                           _lib.current_stream_ptr(dev))
        _lib.check(rc, "ti_tp_barrier")
