"""CPU restatement of the decoder block (triton_int_b200/nn/decoder.py) from the
oracle's operator restatements.  TEST INFRASTRUCTURE ONLY.

The block is a composition, so its oracle is the same composition of
oracle/ops.py functions on full (unsharded) tensors; the tensor-parallel
product path must reproduce it for every rank count.
"""
from __future__ import annotations

import torch

from . import ops as O


def block_forward(params, residual, prev_acc, batch, seq, prev_bias=None, mode=O.RNE_SAT, stages=None):
    """Returns (residual2 fp32, fc2 accumulators int32).  The per-tensor scales
    (prev_scale, qk_alpha, pv_alpha, out_scale, fc1_alpha, fc1_mul) come from
    ``params``.  When ``stages`` is a dict the intermediate tensors are stored in it."""
    meta = params["meta"]
    scales = params
    h, d = meta["heads"], meta["hidden"] // meta["heads"]
    acc = prev_acc if prev_bias is None else prev_acc + prev_bias[None, :]
    res1, x8 = O.dq_add_layernorm_q(acc, scales["prev_scale"], residual, params["ln1_w"], params["ln1_b"], meta["eps"])
    q = O.linear_a8_w8_b8_o8(x8, params["q_w"], params["q_bias"], params["q_alpha"], params["q_beta"], mode)
    k = O.linear_a8_w8_b8_o8(x8, params["k_w"], params["k_bias"], params["k_alpha"], params["k_beta"], mode)
    v = O.linear_a8_w8_b8_o8(x8, params["v_w"], params["v_bias"], params["v_alpha"], params["v_beta"], mode)

    def heads_first(t):
        return t.view(batch, seq, h, d).transpose(1, 2).reshape(batch * h, seq, d)

    qh, kh = heads_first(q), heads_first(k)
    vt = v.view(batch, seq, h, d).permute(0, 2, 3, 1).reshape(batch * h, d, seq)
    s = O.bmm_s8t_s8n_f32t(qh, kh, scales["qk_alpha"])
    p = O.causal_softmax_q(s, 127.0, mode)
    o = O.bmm_s8t_s8n_s8t(p, vt, scales["pv_alpha"], mode)
    attn = o.view(batch, h, seq, d).transpose(1, 2).reshape(batch * seq, h * d)
    out_acc = O.linear_a8_w8_b32_o32(attn, params["out_w"], params["out_bias"])
    res2, h8 = O.dq_add_layernorm_q(out_acc, scales["out_scale"], res1, params["ln2_w"], params["ln2_b"], meta["eps"])
    g8 = O.linear_a8_w8_bfp32_ofp32_GeLu_Q(h8, params["fc1_w"], params["fc1_bias"], scales["fc1_alpha"], scales["fc1_mul"], mode)
    fc2_acc = O.acc_linear(g8, params["fc2_w"])
    if stages is not None:
        stages.update(res1=res1, x8=x8, q=q, k=k, v=v, p=p, attn=attn, out_acc=out_acc, res2=res2, h8=h8, g8=g8)
    return res2, fc2_acc
