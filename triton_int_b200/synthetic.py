"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations (no datasets or checkpoints are involved anywhere).

"int8 ~ round(N(0, sigma)) clipped" is ``randn * sigma -> round -> clamp(-127, 127)``.
All generators draw on the CPU from ``torch.Generator().manual_seed(seed)`` so a
given (config, seed) produces the same bytes on every host; callers move the
tensors to the GPU themselves.
"""
from __future__ import annotations

import torch


def gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def int8_normal(shape, sigma: float, g: torch.Generator) -> torch.Tensor:
    return (torch.randn(shape, generator=g) * sigma).round().clamp(-127, 127).to(torch.int8)


def int32_normal(shape, sigma: float, g: torch.Generator) -> torch.Tensor:
    return (torch.randn(shape, generator=g) * sigma).round().to(torch.int32)


def uniform(shape, lo: float, hi: float, g: torch.Generator) -> torch.Tensor:
    return torch.rand(shape, generator=g) * (hi - lo) + lo


def config1_linear(seed: int = 0, m: int = 64, n: int = 3072, k: int = 768):
    """Single W8A8B8O8 linear: x [m,k], W [n,k], bias [n] ~ round(N(0,40)); alpha 0.0125, beta 0.02."""
    g = gen(seed)
    return dict(
        x=int8_normal((m, k), 40.0, g),
        w=int8_normal((n, k), 40.0, g),
        bias=int8_normal((n,), 40.0, g),
        alpha=torch.tensor(0.0125, dtype=torch.float32),
        beta=torch.tensor(0.02, dtype=torch.float32),
    )


def config2_lnq(seed: int = 1, rows: int = 8192, hidden: int = 4096):
    """Fused dequant -> residual add -> LayerNorm -> quant inputs.  The output scale
    0.05 is folded into gamma and beta the way LayerNormQ.from_float does."""
    g = gen(seed)
    out_scale = 0.05
    acc = int32_normal((rows, hidden), 2.0e4, g)
    residual = torch.randn((rows, hidden), generator=g)
    gamma = uniform((hidden,), 0.5, 1.5, g)
    beta = torch.randn((hidden,), generator=g) * 0.1
    return dict(acc=acc, dq_scale=1.0e-4, residual=residual,
                gamma=gamma / out_scale, beta=beta / out_scale, eps=1e-5, out_scale=out_scale)


def config2_gelu(seed: int = 1, rows: int = 16384, cols: int = 16384):
    """Stand-alone int8 GELU input: int8 ~ round(N(0,40)); in scale 0.03, out scale 0.02."""
    g = gen(seed + 1000)
    return dict(x=int8_normal((rows, cols), 40.0, g), in_scale=0.03, out_scale=0.02)


def config3_attention(seed: int = 2, bh: int = 256, seq: int = 2048, head_dim: int = 128):
    """Q, K, V int8 ~ round(N(0,30)); alpha1 1e-3; P scale 1/127; alpha2 8e-3."""
    g = gen(seed)
    return dict(
        q=int8_normal((bh, seq, head_dim), 30.0, g),
        k=int8_normal((bh, seq, head_dim), 30.0, g),
        v=int8_normal((bh, seq, head_dim), 30.0, g),
        alpha_qk=torch.tensor(1e-3, dtype=torch.float32),
        p_mul=127.0,
        alpha_pv=torch.tensor(8e-3, dtype=torch.float32),
    )


def config4_block(seed: int = 3, hidden: int = 4096, heads: int = 32, ffn: int = 16384,
                  batch: int = 8, seq: int = 2048):
    """OPT-6.7B-shape decoder block: int8 weights ~ round(N(0,30)), per-layer
    alpha/beta ~ U(1e-3,1e-2), LayerNorm parameters as in config 2, and the two
    block inputs (fp32 residual stream, int32 accumulators of the previous
    block's fc2).  Weight tensors are the full (unsharded) ones."""
    g = gen(seed)
    t = batch * seq
    out_scale = 0.05

    def ln():
        gamma = uniform((hidden,), 0.5, 1.5, g)
        beta = torch.randn((hidden,), generator=g) * 0.1
        return gamma / out_scale, beta / out_scale

    def scale():
        return uniform((), 1e-3, 1e-2, g).to(torch.float32)

    p = {}
    p["ln1_w"], p["ln1_b"] = ln()
    p["ln2_w"], p["ln2_b"] = ln()
    for name in ("q", "k", "v"):
        p[f"{name}_w"] = int8_normal((hidden, hidden), 30.0, g)
        p[f"{name}_bias"] = int8_normal((hidden,), 30.0, g)
        p[f"{name}_alpha"], p[f"{name}_beta"] = scale(), scale()
    p["out_w"] = int8_normal((hidden, hidden), 30.0, g)
    p["out_bias"] = int32_normal((hidden,), 1.0e3, g)
    p["fc1_w"] = int8_normal((ffn, hidden), 30.0, g)
    p["fc1_bias"] = torch.randn((ffn,), generator=g) * 0.1
    p["fc2_w"] = int8_normal((hidden, ffn), 30.0, g)
    p["fc2_bias"] = int32_normal((hidden,), 1.0e3, g)
    # dequantisation scales of the int32-emitting linears and fc1's alpha: drawn from the
    # same U(1e-3,1e-2) and divided by a power of two so dequantised values stay O(1)
    p["prev_scale"] = scale() / 64.0
    p["out_scale"] = scale() / 256.0
    p["fc1_alpha"] = scale() / 128.0
    p["fc1_mul"] = torch.tensor(1.0 / 0.02, dtype=torch.float32)
    p["qk_alpha"] = torch.tensor(1e-3, dtype=torch.float32)
    p["pv_alpha"] = torch.tensor(8e-3, dtype=torch.float32)
    p["residual"] = torch.randn((t, hidden), generator=g)
    p["prev_acc"] = int32_normal((t, hidden), 2.0e4, g)
    p["meta"] = dict(hidden=hidden, heads=heads, ffn=ffn, batch=batch, seq=seq, eps=1e-5)
    return p


def config5_linear(seed: int, m: int, layer: str, shard: int = 8):
    """OPT-66B-shape W8A8 linear shard (hidden 9216, FFN 36864, 8-way tensor
    parallel): layer in {"fc1", "fc2", "qkv"}; values ~ round(N(0,35))."""
    hidden, ffn = 9216, 36864
    n, k = {"fc1": (ffn // shard, hidden), "fc2": (hidden, ffn // shard),
            "qkv": (3 * hidden // shard, hidden)}[layer]
    g = gen(seed)
    return dict(
        x=int8_normal((m, k), 35.0, g),
        w=int8_normal((n, k), 35.0, g),
        bias_i8=int8_normal((n,), 35.0, g),
        bias_f32=torch.randn((n,), generator=g),
        alpha=torch.tensor(2.0e-4, dtype=torch.float32),
        beta=torch.tensor(0.02, dtype=torch.float32),
    )
