"""Seeded synthetic MoE layers and token batches.

The reference ships no weights, so every test and benchmark runs on tensors with
the shapes, layouts and value distributions of a GPT-OSS MoE layer:

* expert weights as packed MXFP4: two 4-bit e2m1 codes per byte (low nibble =
  even element), one E8M0 scale byte per 32 consecutive elements along the
  input dimension (layout of getp-csrc/memory/mxfp4.hpp:20-57 and of the
  upstream checkpoint read by
  export_model_bin/gpt-oss-120b/export_model_bin.py:100-137); codes uniform,
  scale exponents uniform in [-8, -4];
* MLP1 weight [E, 2*D, H] with gate rows even / up rows odd (run.cpp:700-704),
  MLP2 weight [E, H, D], bf16 biases ~ N(0, 0.02);
* fp32 router weight [E, H] ~ N(0, 0.02) with a bias;
* token rows ~ N(0, 1), RMS-normalised (eps 1e-5, unit gain) and rounded to
  bf16, i.e. what the block receives after its RMSNorm.

bf16 tensors are carried as uint16 bit patterns so that numpy, ctypes and the
device see identical bytes.
"""
from __future__ import annotations

import numpy as np


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bf16 bit pattern (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rnd = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + rnd) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


E2M1_VALUES = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6],
                       dtype=np.float32)


def dequant_mxfp4(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """[..., n/2] codes + [..., n/32] scales -> float32 [..., n] (small tensors only)."""
    lo = E2M1_VALUES[codes & 0xF]
    hi = E2M1_VALUES[codes >> 4]
    vals = np.stack([lo, hi], axis=-1).reshape(*codes.shape[:-1], codes.shape[-1] * 2)
    sc = np.ldexp(np.float32(1.0), scales.astype(np.int32) - 127).astype(np.float32)
    return vals * np.repeat(sc, 32, axis=-1)


def zipf_router_bias(n_experts: int, s: float = 1.2) -> np.ndarray:
    """Router bias that skews expert popularity towards Zipf(s): log of the target
    probability of each expert, largest shifted to 0."""
    p = 1.0 / np.arange(1, n_experts + 1, dtype=np.float64) ** s
    p /= p.sum()
    return np.log(p / p.max()).astype(np.float32)


def make_layer(n_experts: int, hidden: int, inter: int, seed: int = 0,
               zipf_s: float | None = None) -> dict:
    assert hidden % 32 == 0 and inter % 32 == 0
    rng = np.random.Generator(np.random.Philox(seed))
    E, H, D = n_experts, hidden, inter
    layer = {
        "E": E, "H": H, "D": D,
        "w1_codes": rng.integers(0, 256, size=(E, 2 * D, H // 2), dtype=np.uint8),
        "w1_scales": (127 + rng.integers(-8, -3, size=(E, 2 * D, H // 32))).astype(np.uint8),
        "w2_codes": rng.integers(0, 256, size=(E, H, D // 2), dtype=np.uint8),
        "w2_scales": (127 + rng.integers(-8, -3, size=(E, H, D // 32))).astype(np.uint8),
        "b1": f32_to_bf16_bits(rng.normal(0.0, 0.02, size=(E, 2 * D)).astype(np.float32)),
        "b2": f32_to_bf16_bits(rng.normal(0.0, 0.02, size=(E, H)).astype(np.float32)),
        "router_w": rng.normal(0.0, 0.02, size=(E, H)).astype(np.float32),
        "router_b": rng.normal(0.0, 0.02, size=(E,)).astype(np.float32),
    }
    if zipf_s is not None:
        layer["router_b"] = zipf_router_bias(E, zipf_s)
    return layer


def make_tokens(n_tokens: int, hidden: int, seed: int = 0) -> np.ndarray:
    """bf16 bit patterns [T, H] of RMS-normalised N(0,1) rows."""
    rng = np.random.Generator(np.random.Philox([seed, 0x746F6B]))
    x = rng.normal(0.0, 1.0, size=(n_tokens, hidden)).astype(np.float32)
    ms = (x.astype(np.float64) ** 2).mean(axis=1, keepdims=True)
    t = (x / np.sqrt(ms + 1e-5)).astype(np.float32)
    return f32_to_bf16_bits(t)


def make_residual(n_tokens: int, hidden: int, seed: int = 0) -> tuple[np.ndarray, np.ndarray]:
    """Residual-stream rows x [T, H] (row scales spread over two decades, a few outlier channels, as a
    residual stream has) and an RMSNorm gain [H] around 1, both as bf16 bit patterns."""
    rng = np.random.Generator(np.random.Philox([seed, 0x726573]))
    x = rng.normal(0.0, 1.0, size=(n_tokens, hidden)).astype(np.float32)
    x *= np.exp(rng.uniform(np.log(0.2), np.log(20.0), size=(n_tokens, 1))).astype(np.float32)
    hot = rng.choice(hidden, size=max(hidden // 64, 1), replace=False)
    x[:, hot] *= 8.0
    gain = rng.normal(1.0, 0.25, size=hidden).astype(np.float32)
    return f32_to_bf16_bits(x), f32_to_bf16_bits(gain)


def make_quantizer_inputs(seed: int = 0) -> np.ndarray:
    """fp32 values that exercise the MXFP4 quantiser: wide-range random blocks, an all-zero block, values
    exactly midway between two E2M1 magnitudes, signed zeros, denormals, values near the float maximum,
    block maxima that are exact powers of two or just below one, values above 6 x scale, and a ragged
    tail (the length is not a multiple of 32)."""
    rng = np.random.Generator(np.random.Philox([seed, 0x717561]))
    parts = []
    body = rng.standard_normal(32 * 64).astype(np.float32)
    body *= np.repeat(np.exp2(rng.integers(-30, 30, size=64)).astype(np.float32), 32)
    parts.append(body)
    parts.append(np.zeros(32, dtype=np.float32))
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, 7.99], dtype=np.float32)
    for k in (-3, 0, 5):
        blk = np.zeros(32, dtype=np.float32)
        blk[:9] = mids * np.float32(2.0 ** k)
        blk[9:18] = -mids * np.float32(2.0 ** k)
        blk[18] = np.float32(4.0 * 2.0 ** k)          # fixes the block exponent at k
        blk[19] = np.float32(-0.0)
        parts.append(blk)
    tiny = np.full(32, np.float32(1e-41), dtype=np.float32)     # denormals
    tiny[5] = np.float32(3e-39)
    parts.append(tiny)
    huge = rng.uniform(-3e38, 3e38, size=32).astype(np.float32)
    parts.append(huge)
    pow2 = rng.uniform(-1, 1, size=32).astype(np.float32)
    pow2[7] = np.float32(8.0)
    parts.append(pow2)
    below = rng.uniform(-1, 1, size=32).astype(np.float32)
    below[3] = np.nextafter(np.float32(8.0), np.float32(0.0))
    parts.append(below)
    parts.append(rng.standard_normal(13).astype(np.float32))    # ragged tail
    return np.concatenate(parts)


def weight_bytes_per_expert(hidden: int, inter: int) -> int:
    """MXFP4 codes + E8M0 scales + bf16 biases of one expert (both MLPs)."""
    w1 = 2 * inter * hidden
    w2 = hidden * inter
    return (w1 + w2) // 2 + (w1 + w2) // 32 + 2 * (2 * inter + hidden)


def algorithmic_work(n_tokens: int, hidden: int, inter: int, n_experts: int, top_k: int,
                     active_experts: int) -> tuple[int, int]:
    """(flops, bytes) of one block: 2*MACs of router + both MLPs; bytes = weights of
    the experts that receive at least one token + bf16 rows in and out + router."""
    flops = n_tokens * (top_k * (2 * hidden * 2 * inter + 2 * inter * hidden)
                        + 2 * hidden * n_experts)
    nbytes = (active_experts * weight_bytes_per_expert(hidden, inter)
              + n_tokens * hidden * 2 * 2 + n_experts * hidden * 4)
    return flops, nbytes
