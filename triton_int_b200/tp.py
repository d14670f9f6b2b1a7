"""Tensor-parallel plumbing for one node: peer-mapped buffers and the fused
reduce-scatter -> dequant+bias+residual+LayerNorm+quant -> all-gather launch.

One process per GPU.  ``torch.distributed`` (NCCL) is the control plane;
the int32 partial sums and the gathered int8 activations live in symmetric
memory (``torch.distributed._symmetric_memory``), which gives every rank a device
pointer to every peer's buffer over NVLink.  The data path is this library's own
kernel (``ti_tp_reduce_layernorm_q``): plain peer loads and stores only.
Ordering between ranks is a device-side barrier on the current stream.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib, config
from .kernels._gemm import scale_tensor


def reduce_layernorm_q(parts_ptrs, outs_ptrs, rank_rows, n, residual_in, gamma, beta, eps, dq_scale,
                       bias_int32=None, want_residual_out=True, parts_row_begin=None, rank=None):
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
    p.parts_row_begin = row_begin if parts_row_begin is None else parts_row_begin
    p.eps = float(eps)
    p.world = world
    p.rank = (row_begin // row_count if row_count else 0) if rank is None else rank
    p.rounding = config.rounding_mode()
    with torch.cuda.device(dev):
        p.stream = _lib.current_stream_ptr(dev)
        rc = _lib.load().ti_tp_reduce_layernorm_q(C.byref(p))
    _lib.check(rc, "ti_tp_reduce_layernorm_q")
    return res_out


def gemm_scatter(a2d, w, recv_ptrs, rank, rows_per_rank):
    """Row-parallel linear whose raw int32 tiles are stored, as they finish, into the receive
    buffers of the ranks owning their rows (``ti_gemm_i8_scatter``).  a2d int8 [M, K_local],
    w int8 [N, K_local]; recv_ptrs: one device pointer per rank to an int32 buffer laid out
    [world][rows_per_rank][N] (rank r's tile rows land in slot ``rank`` of their owner)."""
    _lib.require_cuda(a2d, w)
    assert a2d.dim() == 2 and w.dim() == 2 and a2d.shape[1] == w.shape[1]
    world = len(recv_ptrs)
    p = _lib.GemmParams()
    p.a, p.b = a2d.data_ptr(), w.data_ptr()
    p.m, p.k = a2d.shape
    p.n = w.shape[0]
    p.batch = 1
    p.a_stride_m, p.a_stride_k = a2d.stride(0), a2d.stride(1)
    p.b_stride_n, p.b_stride_k = w.stride(0), w.stride(1)
    p.out_dtype, p.epilogue = _lib.TI_I32, _lib.EPI_I32
    p.rounding = config.rounding_mode()
    sc = _lib.GemmScatter()
    for r in range(world):
        sc.recv[r] = recv_ptrs[r]
    sc.world, sc.rank, sc.rows_per_rank = world, rank, rows_per_rank
    dev = a2d.device
    with torch.cuda.device(dev):
        p.stream = _lib.current_stream_ptr(dev)
        rc = _lib.load().ti_gemm_i8_scatter(C.byref(p), C.byref(sc))
    _lib.check(rc, "ti_gemm_i8_scatter")


class SymmetricBuffers:
    """[rows, n] int32 partial-sum buffers and int8 activation buffers that every
    rank of ``group`` can address, plus a stream-ordered barrier."""

    def __init__(self, group, rows, n, device, num_partial=2, num_act=2):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.group, self.rows, self.n = group, rows, n
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert rows % self.world == 0, "rows must divide evenly over the ranks"
        self.partial, self.act, self._handles, self._partial_handles = [], [], [], []
        for _ in range(num_partial):
            t = symm.empty((rows, n), dtype=torch.int32, device=device)
            h = symm.rendezvous(t, group)
            self.partial.append((t, [int(x) for x in h.buffer_ptrs]))
            self._handles.append(h)
            self._partial_handles.append(h)
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

    def staging(self, i):
        """Local (not peer-mapped) [rows, n] int32 matrix a row-parallel GEMM writes before its row
        slices are pushed to their owners; allocated on first use and kept."""
        if not hasattr(self, "_staging"):
            self._staging = {}
        if i not in self._staging:
            self._staging[i] = torch.empty((self.rows, self.n), dtype=torch.int32, device=self.partial[0][0].device)
        return self._staging[i]

    def peer_slot(self, i, peer):
        """Tensor view [rows/world, n] of slot `self.rank` inside rank `peer`'s receive buffer i
        (peer-mapped memory): the destination of this rank's copy-engine push to `peer`."""
        per = self.rows // self.world
        return self._partial_handles[i].get_buffer(peer, (per, self.n), torch.int32, self.rank * per * self.n)

    def push_slices(self, i, partial):
        """Copy rows [r*per, (r+1)*per) of this rank's [rows, n] int32 partial sums into slot
        `rank` of rank r's receive buffer i, for every r, with asynchronous device-to-device
        copies on the current stream (they run on the copy engines, not on SMs)."""
        per = self.rows // self.world
        for s in range(self.world):
            r = (self.rank + 1 + s) % self.world   # staggered: every rank starts with a different peer
            self.peer_slot(i, r).copy_(partial[r * per:(r + 1) * per], non_blocking=True)

    def local_slots(self, i):
        """Pointers to the `world` slices [rows/world, n] of this rank's receive buffer i."""
        t, _ = self.partial[i]
        step = (self.rows // self.world) * self.n * 4
        return [t.data_ptr() + s * step for s in range(self.world)]

    def barrier(self):
        """All ranks' streams have reached this point before any proceeds (bounded wait on
        the device; an expired wait shows up in ``triton_int_b200.device_status()``)."""
        self._epoch += 1
        dev = self._pad.device
        with torch.cuda.device(dev):
            rc = _lib.load().ti_tp_barrier(self._pad_ptrs, self.world, self.rank, self._epoch & 0xFFFFFFFF,
                                           _lib.current_stream_ptr(dev))
        _lib.check(rc, "ti_tp_barrier")
