"""Generate the golden vectors in this directory by running the reference's own
kernels (unmodified) on the CPU under Triton's interpreter.

Usage (development container only; needs the reference checkout):

    TRITON_INT_REFERENCE=/path/to/reference python tests/golden/make_golden.py

Writes ``linear.npz``, ``bmm.npz``, ``layernorm.npz`` and ``config1.npz`` next to
this script.  Small cases store inputs and outputs; the config-1 case stores the
output plus a SHA-256 of its seed-generated inputs (``triton_int_b200.synthetic``)
so that a generator drift is detected rather than silently compared.
"""
from __future__ import annotations

import hashlib
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import numpy as np  # noqa: E402
import torch  # noqa: E402

from oracle import ref_interp  # noqa: E402
from triton_int_b200 import synthetic  # noqa: E402


def npy(t):
    if t.dtype == torch.bfloat16:
        return t.float().numpy()
    return t.numpy()


def sha(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().numpy().tobytes())
    return h.hexdigest()


def i8(shape, sigma, g):
    return synthetic.int8_normal(shape, sigma, g)


def linear_cases(ref):
    g = synthetic.gen(100)
    out = {}
    shapes = {
        "ragged": ((37, 96), (100, 96)),
        "m1": ((1, 128), (256, 128)),
        "lead3d": ((2, 5, 64), (48, 64)),
        "ktail": ((16, 200), (24, 200)),
    }
    a = torch.tensor(0.004, dtype=torch.float32)
    b = torch.tensor(0.3, dtype=torch.float32)
    for name, (xs, ws) in shapes.items():
        x, w = i8(xs, 40.0, g), i8(ws, 40.0, g)
        n = ws[0]
        bias8 = i8((n,), 40.0, g)
        bias32 = synthetic.int32_normal((n,), 3.0e4, g)
        biasf = torch.randn((n,), generator=g)
        pre = f"{name}/"
        out.update({pre + "x": npy(x), pre + "w": npy(w), pre + "bias8": npy(bias8),
                    pre + "bias32": npy(bias32), pre + "biasf": npy(biasf),
                    pre + "alpha": npy(a), pre + "beta": npy(b)})
        L = ref.linear
        out[pre + "ofp32"] = npy(L.linear_a8_w8_ofp32(x, w, a))
        out[pre + "b8_o8"] = npy(L.linear_a8_w8_b8_o8(x, w, bias8, a, b))
        out[pre + "relu_b8_o8"] = npy(L.linear_relu_a8_w8_b8_o8(x, w, bias8, a, b))
        out[pre + "b32_o32"] = npy(L.linear_a8_w8_b32_o32(x, w, bias32))
        out[pre + "b32_o32_scaled"] = npy(L.linear_a8_w8_b32_o32_with_scaling(x, w, bias32, a, b))
        out[pre + "bfp32_ofp32"] = npy(L.linear_a8_w8_bfp32_ofp32(x, w, biasf, a, b))
        out[pre + "bfp16_ofp16"] = npy(L.linear_a8_w8_bfp32_ofp32(x, w, biasf.half(), a, b))
        gel_b = torch.tensor(1.0 / 0.02, dtype=torch.float32)
        out[pre + "gelu_mul"] = npy(gel_b)
        out[pre + "gelu_q"] = npy(ref.fused.linear_a8_w8_bfp32_ofp32_GeLu_Q(x, w, biasf, a, gel_b))
    # non-contiguous weight (a column slice of a wider matrix)
    x = i8((9, 64), 40.0, g)
    wide = i8((20, 128), 40.0, g)
    w = wide[:, ::2]
    bias8 = i8((20,), 40.0, g)
    out["strided/x"], out["strided/wide"], out["strided/bias8"] = npy(x), npy(wide), npy(bias8)
    out["strided/alpha"], out["strided/beta"] = npy(a), npy(b)
    out["strided/b8_o8"] = npy(ref.linear.linear_a8_w8_b8_o8(x, w, bias8, a, b))
    return out


def bmm_cases(ref):
    g = synthetic.gen(200)
    out = {}
    s = torch.tensor(0.0021, dtype=torch.float32)
    for name, (B, M, N, K) in {"small": (3, 40, 56, 64), "ragged": (2, 33, 17, 50)}.items():
        a = i8((B, M, K), 30.0, g)
        bn = i8((B, N, K), 30.0, g)   # "s8n": [B,N,K]
        bt = i8((B, K, N), 30.0, g)   # "s8t": [B,K,N]
        pre = f"{name}/"
        out.update({pre + "a": npy(a), pre + "bn": npy(bn), pre + "bt": npy(bt), pre + "scale": npy(s)})
        R = ref.bmm
        out[pre + "s8t_s8n_s32t"] = npy(R.bmm_s8t_s8n_s32t(a, bn))
        out[pre + "s8t_s8t_s32t"] = npy(R.bmm_s8t_s8t_s32t(a, bt))
        out[pre + "s8t_s8n_f32t"] = npy(R.bmm_s8t_s8n_f32t(a, bn, s))
        out[pre + "s8t_s8n_f16t"] = npy(R.bmm_s8t_s8n_f32t(a, bn, s, dtype=torch.float16))
        out[pre + "s8t_s8n_s8t"] = npy(R.bmm_s8t_s8n_s8t(a, bn, s))
        out[pre + "s8t_s8t_s8t"] = npy(R.bmm_s8t_s8t_s8t(a, bt, s))
    return out


def layernorm_cases(ref):
    g = synthetic.gen(300)
    out = {}
    F = ref.fused
    for name, (rows, n, dt) in {"h4096": (4, 4096, torch.float32), "n300": (5, 300, torch.float32),
                                "n5000": (3, 5000, torch.float32), "f16n256": (4, 256, torch.float16)}.items():
        x = (torch.randn((rows, n), generator=g) * 1.7 + 0.3).to(dt)
        skip = torch.randn((rows, n), generator=g).to(dt)
        w = (synthetic.uniform((n,), 0.5, 1.5, g) / 0.05).to(dt)
        b = (torch.randn((n,), generator=g) * 2.0).to(dt)
        pre = f"{name}/"
        out.update({pre + "x": npy(x), pre + "skip": npy(skip), pre + "w": npy(w), pre + "b": npy(b)})
        out[pre + "ln_q"] = npy(F.layer_norm_fwd_fused_single_pass_q(x, w, b, 1e-5))
        out[pre + "ln_q_rms"] = npy(F.layer_norm_fwd_fused_single_pass_q(x, w, b, 1e-5, True))
        out[pre + "ln_q_nobias"] = npy(F.layer_norm_fwd_fused_single_pass_q(x, w, None, 1e-5))
        out[pre + "ln"] = npy(F.layer_norm_fwd_fused_single_pass(x, w, b, 1e-5))
        out[pre + "skip_ln"] = npy(F.skip_layer_norm_fwd_fused_single_pass(x, skip, w, b, 1e-5))
        o0, o1 = F.skip_layer_norm_fwd_fused_single_pass2(x, skip, w, b, 1e-5)
        out[pre + "skip_ln2_0"], out[pre + "skip_ln2_1"] = npy(o0), npy(o1)
    # the torch definition of the fused dequant+add+LN+quant op (functional/fused.py:6-15)
    acc = synthetic.int32_normal((6, 512), 2.0e4, g)
    res = torch.randn((6, 512), generator=g)
    w = synthetic.uniform((512,), 0.5, 1.5, g) / 0.05
    b = torch.randn((512,), generator=g) * 2.0
    r, y = ref.ffused.dq_add_layernorm_q_py(acc, 1e-4, res, w, b, 1e-5)
    out.update({"dq/acc": npy(acc), "dq/res": npy(res), "dq/w": npy(w), "dq/b": npy(b),
                "dq/res_out": npy(r), "dq/y": npy(y)})
    return out


def config1_case(ref):
    c = synthetic.config1_linear(seed=0)
    y = ref.linear.linear_a8_w8_b8_o8(c["x"], c["w"], c["bias"], c["alpha"], c["beta"])
    acc = ref.linear.linear_a8_w8_b32_o32(c["x"], c["w"], torch.zeros(c["w"].shape[0], dtype=torch.int32))
    return {"inputs_sha256": np.frombuffer(sha(c["x"], c["w"], c["bias"]).encode(), dtype=np.uint8),
            "y": npy(y), "acc_sha256": np.frombuffer(sha(acc).encode(), dtype=np.uint8),
            "acc_head": npy(acc[:4])}


def main():
    ref = ref_interp.load()
    np.savez_compressed(os.path.join(HERE, "linear.npz"), **linear_cases(ref))
    np.savez_compressed(os.path.join(HERE, "bmm.npz"), **bmm_cases(ref))
    np.savez_compressed(os.path.join(HERE, "layernorm.npz"), **layernorm_cases(ref))
    np.savez_compressed(os.path.join(HERE, "config1.npz"), **config1_case(ref))
    for f in ("linear", "bmm", "layernorm", "config1"):
        p = os.path.join(HERE, f + ".npz")
        print(f, os.path.getsize(p), "bytes")


if __name__ == "__main__":
    main()
