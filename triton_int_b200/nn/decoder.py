"""An OPT-shape SmoothQuant decoder block assembled from the modules of this
package, with optional tensor parallelism.

The reference ships operators and modules but no model file; this block is the
composition its modules were written for (int8 q/k/v projections, int8 BMM
attention, row-parallel out_proj / fc2 that keep int32 accumulators, two fused
dequant -> residual-add -> LayerNorm -> quant steps, fc1 with fused GELU-quant).

Data flow for T = batch * seq tokens, hidden H, P tensor-parallel ranks:

    (residual fp32 [T,H], acc int32 [T,H] of the previous block's fc2)
      -> DQ_Add_LayerNorm_Q          -> residual1 fp32 [T,H], x int8 [T,H]
      -> q/k/v W8A8B8O8Linear        -> int8 [T,H/P] each       (column parallel)
      -> BMM_S8T_S8N_F32T, causal softmax -> int8, BMM_S8T_S8N_S8T over H/P/D heads
         (one fused attention kernel when head_dim is 128; the three-operator form otherwise)
      -> out_proj, raw int32 [T,H]   -> sum over ranks (exact)  (row parallel)
      -> DQ_Add_LayerNorm_Q          -> residual2 fp32 [T,H], h int8 [T,H]
      -> fc1 W8A8BFP32OFP32_GeLu_Q   -> int8 [T,F/P]            (column parallel)
      -> fc2, raw int32 [T,H]        -> sum over ranks (exact)  (row parallel)
    returns (residual2, fc2 accumulators); the next block's first step dequantises them.

Row-parallel shards emit raw int32 partial sums and the int32 bias is added
after the reduction, inside the LayerNorm kernel; integer addition is
associative, so every rank count produces the same bits as one GPU.
"""
from __future__ import annotations

import torch

from ..kernels.bmm import bmm_s8t_s8n_f32t, bmm_s8t_s8n_s8t
from ..kernels.fused import (attention_i8, causal_softmax_q, dq_add_layernorm_q, layer_norm_fwd_fused_single_pass_q,
                             linear_a8_w8_bfp32_ofp32_GeLu_Q)
from ..kernels.linear import linear_a8_w8_b8_o8, linear_a8_w8_b32_dq_add_ofp32, linear_a8_w8_b32_o32


def shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Column-parallel slice: rows [rank*N/P, (rank+1)*N/P) of a [N, ...] weight or bias."""
    n = t.shape[0]
    assert n % world == 0
    return t[rank * (n // world):(rank + 1) * (n // world)].contiguous()


def shard_cols(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Row-parallel slice: columns [rank*K/P, (rank+1)*K/P) of a [N, K] weight."""
    k = t.shape[1]
    assert k % world == 0
    return t[:, rank * (k // world):(rank + 1) * (k // world)].contiguous()


class Int8DecoderBlock(torch.nn.Module):
    """One decoder block; ``params`` is the dict made by ``synthetic.config4_block``
    (full, unsharded tensors).  ``rank``/``world`` select this process's shard;
    ``reduce_fn(int32_tensor) -> int32_tensor`` performs the sum over ranks (identity
    when world == 1)."""

    def __init__(self, params, rank: int = 0, world: int = 1, reduce_fn=None, causal_skip: bool = True,
                 fused_attention: bool = True, fuse_dq_add: bool = True):
        super().__init__()
        meta = params["meta"]
        self.hidden, self.heads, self.ffn = meta["hidden"], meta["heads"], meta["ffn"]
        self.eps = meta["eps"]
        self.rank, self.world = rank, world
        assert self.heads % world == 0 and self.ffn % world == 0
        self.local_heads = self.heads // world
        self.head_dim = self.hidden // self.heads
        self.reduce_fn = reduce_fn if reduce_fn is not None else (lambda t: t)
        self.causal_skip = causal_skip
        # fused attention keeps S and P on chip; the unfused form (three operators of the
        # reference interface) is kept for comparison
        self.fused_attention = fused_attention and self.head_dim == 128
        # one rank: out_proj's epilogue does the dequantise + residual add of the LayerNorm step that follows
        self.fuse_dq_add = fuse_dq_add and world == 1 and self.hidden % 16 == 0
        reg = self.register_buffer
        reg("ln1_w", params["ln1_w"].clone()); reg("ln1_b", params["ln1_b"].clone())
        reg("ln2_w", params["ln2_w"].clone()); reg("ln2_b", params["ln2_b"].clone())
        for name in ("q", "k", "v"):
            reg(f"{name}_w", shard_rows(params[f"{name}_w"], rank, world))
            reg(f"{name}_bias", shard_rows(params[f"{name}_bias"], rank, world))
            reg(f"{name}_alpha", params[f"{name}_alpha"].clone())
            reg(f"{name}_beta", params[f"{name}_beta"].clone())
        reg("out_w", shard_cols(params["out_w"], rank, world))
        reg("out_bias", params["out_bias"].clone())
        reg("fc1_w", shard_rows(params["fc1_w"], rank, world))
        reg("fc1_bias", shard_rows(params["fc1_bias"], rank, world))
        reg("fc2_w", shard_cols(params["fc2_w"], rank, world))
        reg("fc2_bias", params["fc2_bias"].clone())
        # per-tensor scales of the attention and the dequantisation steps
        for name in ("prev_scale", "out_scale", "fc1_alpha", "fc1_mul", "qk_alpha", "pv_alpha"):
            reg(name, params[name].clone().to(torch.float32))

    def _heads_first(self, x, batch, seq):
        # [T, h*D] -> [B*h, S, D]
        return x.view(batch, seq, self.local_heads, self.head_dim).transpose(1, 2).reshape(
            batch * self.local_heads, seq, self.head_dim)

    @torch.no_grad()
    def attention(self, x8, batch, seq):
        q = linear_a8_w8_b8_o8(x8, self.q_w, self.q_bias, self.q_alpha, self.q_beta)
        k = linear_a8_w8_b8_o8(x8, self.k_w, self.k_bias, self.k_alpha, self.k_beta)
        v = linear_a8_w8_b8_o8(x8, self.v_w, self.v_bias, self.v_alpha, self.v_beta)
        if self.fused_attention:
            shape = (batch, seq, self.local_heads, self.head_dim)
            o = attention_i8(q.view(shape), k.view(shape), v.view(shape), self.qk_alpha, self.pv_alpha, 127.0, causal=True)
            return o.view(batch * seq, self.local_heads * self.head_dim)
        qh, kh = self._heads_first(q, batch, seq), self._heads_first(k, batch, seq)
        # V^T: [B*h, D, S], the "s8n" operand of the second BMM
        vt = v.view(batch, seq, self.local_heads, self.head_dim).permute(0, 2, 3, 1).reshape(
            batch * self.local_heads, self.head_dim, seq)
        s = bmm_s8t_s8n_f32t(qh, kh, self.qk_alpha, causal=self.causal_skip)
        p = causal_softmax_q(s, 127.0)
        del s
        o = bmm_s8t_s8n_s8t(p, vt, self.pv_alpha)
        # [B*h, S, D] -> [T, h*D]
        return o.view(batch, self.local_heads, seq, self.head_dim).transpose(1, 2).reshape(
            batch * seq, self.local_heads * self.head_dim)

    @torch.no_grad()
    def forward(self, residual, prev_acc, batch, seq, prev_bias=None):
        res1, x8 = dq_add_layernorm_q(prev_acc, self.prev_scale, residual, self.ln1_w, self.ln1_b, self.eps,
                                      bias_int32=prev_bias)
        attn = self.attention(x8, batch, seq)
        if self.world == 1 and self.fuse_dq_add:
            # one rank: nothing to sum across ranks, so out_proj's epilogue dequantises and adds the
            # residual itself and the LayerNorm kernel reads 4 bytes per element instead of 8 (same bits)
            res2 = linear_a8_w8_b32_dq_add_ofp32(attn, self.out_w, self.out_bias, self.out_scale, res1)
            h8 = layer_norm_fwd_fused_single_pass_q(res2, self.ln2_w, self.ln2_b, self.eps)
        else:
            out_acc = self.reduce_fn(linear_a8_w8_b32_o32(attn, self.out_w, None))
            res2, h8 = dq_add_layernorm_q(out_acc, self.out_scale, res1, self.ln2_w, self.ln2_b, self.eps,
                                          bias_int32=self.out_bias)
        g8 = linear_a8_w8_bfp32_ofp32_GeLu_Q(h8, self.fc1_w, self.fc1_bias, self.fc1_alpha, self.fc1_mul)
        fc2_acc = self.reduce_fn(linear_a8_w8_b32_o32(g8, self.fc2_w, None))
        return res2, fc2_acc

    @torch.no_grad()
    def forward_tp_fused(self, residual_shard, bufs, batch, seq, prev_bias=None):
        """Tensor-parallel step with the exchange fused into the LayerNorm kernels.

        ``bufs`` is a ``triton_int_b200.tp.SymmetricBuffers``.  On entry ``bufs.partial[0]``
        holds every rank's int32 partial sums of the previous block's fc2 and
        ``residual_shard`` this rank's rows of the fp32 residual stream.  On return
        ``bufs.partial[0]`` holds this block's fc2 partial sums (unreduced: the next
        block's first kernel adds them) and the new residual shard is returned."""
        from ..kernels._gemm import gemm
        from .. import _lib, tp
        rows = bufs.rank_rows()
        (p0, p0_ptrs), (p1, p1_ptrs) = bufs.partial[0], bufs.partial[1]
        (x8, x8_ptrs), (h8, h8_ptrs) = bufs.act[0], bufs.act[1]
        bufs.barrier()  # every rank's partial sums in partial[0] are complete
        res1 = tp.reduce_layernorm_q(p0_ptrs, x8_ptrs, rows, self.hidden, residual_shard, self.ln1_w, self.ln1_b,
                                     self.eps, self.prev_scale, bias_int32=prev_bias)
        bufs.barrier()  # x8 is complete everywhere; partial[0] may be overwritten
        attn = self.attention(x8, batch, seq)
        linear_a8_w8_b32_o32(attn, self.out_w, None, out=p1)
        bufs.barrier()
        res2 = tp.reduce_layernorm_q(p1_ptrs, h8_ptrs, rows, self.hidden, res1, self.ln2_w, self.ln2_b,
                                     self.eps, self.out_scale, bias_int32=self.out_bias)
        bufs.barrier()
        g8 = linear_a8_w8_bfp32_ofp32_GeLu_Q(h8, self.fc1_w, self.fc1_bias, self.fc1_alpha, self.fc1_mul)
        linear_a8_w8_b32_o32(g8, self.fc2_w, None, out=p0)
        return res2

    @torch.no_grad()
    def forward_tp_push(self, residual_shard, bufs, batch, seq, prev_bias=None):
        """Tensor-parallel step in which the row-parallel GEMMs push their int32 tiles into
        the owners' receive buffers while they run (``ti_gemm_i8_scatter``) and the owner adds
        the slices locally inside the dequant+LayerNorm kernel, which also pushes its int8
        rows to every rank.  ``bufs.partial[0]`` is used as this rank's receive buffer for the
        fc2 slices (filled by the previous block), ``bufs.partial[1]`` for out_proj's.  Returns
        the new residual shard; the fc2 slices of this block sit in the peers' buffers."""
        from .. import tp
        r0, rc = bufs.rank_rows()
        p0_ptrs, p1_ptrs = bufs.partial[0][1], bufs.partial[1][1]
        (x8, x8_ptrs), (h8, h8_ptrs) = bufs.act[0], bufs.act[1]
        bufs.barrier()  # every rank's fc2 slices have landed in this rank's buffer 0
        res1 = tp.reduce_layernorm_q(bufs.local_slots(0), x8_ptrs, (r0, rc), self.hidden, residual_shard, self.ln1_w,
                                     self.ln1_b, self.eps, self.prev_scale, bias_int32=prev_bias, parts_row_begin=0,
                                     rank=bufs.rank)
        bufs.barrier()  # x8 is complete everywhere
        attn = self.attention(x8, batch, seq)
        tp.gemm_scatter(attn, self.out_w, p1_ptrs, bufs.rank, rc)
        bufs.barrier()
        res2 = tp.reduce_layernorm_q(bufs.local_slots(1), h8_ptrs, (r0, rc), self.hidden, res1, self.ln2_w, self.ln2_b,
                                     self.eps, self.out_scale, bias_int32=self.out_bias, parts_row_begin=0,
                                     rank=bufs.rank)
        bufs.barrier()
        g8 = linear_a8_w8_bfp32_ofp32_GeLu_Q(h8, self.fc1_w, self.fc1_bias, self.fc1_alpha, self.fc1_mul)
        tp.gemm_scatter(g8, self.fc2_w, p0_ptrs, bufs.rank, rc)
        return res2

    @torch.no_grad()
    def forward_tp_dma(self, residual_shard, bufs, batch, seq, comm_stream, prev_bias=None):
        """Tensor-parallel step whose reduce-scatter traffic rides the copy engines: each
        row-parallel GEMM writes a local [T, H] int32 matrix, its row slices are pushed to the
        owners' receive buffers with asynchronous peer copies on ``comm_stream`` (no SM is
        involved, so another group of sequences can compute meanwhile), and the owner adds the
        slices locally inside the dequant+LayerNorm kernel.  Buffer roles as in forward_tp_push;
        on return the pushes of this block's fc2 slices are in flight on ``comm_stream``."""
        from .. import tp
        r0, rc = bufs.rank_rows()
        (x8, x8_ptrs), (h8, h8_ptrs) = bufs.act[0], bufs.act[1]
        comp = torch.cuda.current_stream(residual_shard.device)
        comp.wait_stream(comm_stream)   # the previous block's pushes from this rank are done
        bufs.barrier()                  # ... and so are everybody else's
        res1 = tp.reduce_layernorm_q(bufs.local_slots(0), x8_ptrs, (r0, rc), self.hidden, residual_shard, self.ln1_w,
                                     self.ln1_b, self.eps, self.prev_scale, bias_int32=prev_bias, parts_row_begin=0,
                                     rank=bufs.rank)
        bufs.barrier()
        attn = self.attention(x8, batch, seq)
        part = bufs.staging(1)
        linear_a8_w8_b32_o32(attn, self.out_w, None, out=part)
        comm_stream.wait_stream(comp)
        with torch.cuda.stream(comm_stream):
            bufs.push_slices(1, part)
        comp.wait_stream(comm_stream)
        bufs.barrier()
        res2 = tp.reduce_layernorm_q(bufs.local_slots(1), h8_ptrs, (r0, rc), self.hidden, res1, self.ln2_w, self.ln2_b,
                                     self.eps, self.out_scale, bias_int32=self.out_bias, parts_row_begin=0,
                                     rank=bufs.rank)
        bufs.barrier()
        g8 = linear_a8_w8_bfp32_ofp32_GeLu_Q(h8, self.fc1_w, self.fc1_bias, self.fc1_alpha, self.fc1_mul)
        part2 = bufs.staging(0)
        linear_a8_w8_b32_o32(g8, self.fc2_w, None, out=part2)
        comm_stream.wait_stream(comp)
        with torch.cuda.stream(comm_stream):
            bufs.push_slices(0, part2)
        return res2
