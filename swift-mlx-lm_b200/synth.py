"""Seeded synthetic tensors with the shapes and value distributions of the benchmark configurations.

Linear weights: nibbles uniform 0..15 packed 8 per uint32 along K, per-group bf16 scale ~ U(0.005, 0.02)
and bf16 bias ~ N(0, 0.01). Embeddings bf16 ~ N(0, 0.02); norm weights bf16 ~ 1 + N(0, 0.02);
conv weights bf16 ~ N(0, 0.02). There are no checkpoints involved: weights are random-init.
"""
from __future__ import annotations

import zlib
from typing import Dict

import numpy as np

from .formats import f32_to_bf16


def synth_q4(n: int, k: int, seed: int, centered: bool = False, group: int = 64):
    """(weight u32 [n, k/8], scales bf16 [n, k/group], biases bf16 [n, k/group]) as uint arrays; group = 64 or 128.

    centered=True moves every group's bias by -7.5 * scale, so that the dequantised weights have zero mean instead of
    the benchmark distribution's common mean of 7.5 * scale: products are then well conditioned (no output is a small
    difference of large sums), which is what a test of numerical equivalence between two code paths wants."""
    rng = np.random.default_rng(seed)
    w = rng.integers(0, 1 << 32, size=(n, k // 8), dtype=np.uint32)  # every nibble uniform on 0..15
    scale_f = rng.uniform(0.005, 0.02, size=(n, k // group)).astype(np.float32)
    bias_f = rng.normal(0.0, 0.01, size=(n, k // group)).astype(np.float32)
    if centered:
        bias_f = bias_f - 7.5 * scale_f
    return w, f32_to_bf16(scale_f), f32_to_bf16(bias_f)


def _seed(base: int, name: str) -> int:
    return (base * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFF


def synth_model_weights(builder, seed: int = 3, centered: bool = False, group: int = 64) -> Dict[str, object]:
    """name -> (w, scales, biases) for quantized tensors, bf16 uint16 array for dense ones."""
    out: Dict[str, object] = {}
    for name, kind, shape, _shard in builder.tensors():
        rng = np.random.default_rng(_seed(seed, name))
        if kind == "q4":
            out[name] = synth_q4(shape[0], shape[1], _seed(seed, name), centered=centered, group=group)
        elif kind == "norm":
            out[name] = f32_to_bf16((1.0 + rng.normal(0.0, 0.02, size=shape)).astype(np.float32))
        elif kind == "f32":   # recurrent layers: norm weight ~ 1, A_log ~ U(-1, 1); kept in fp32
            out[name] = (rng.uniform(-1.0, 1.0, size=shape) if name.endswith("A_log") else 1.0 + rng.normal(0.0, 0.02, size=shape)).astype(np.float32)
        elif name.endswith("dt_bias"):
            out[name] = f32_to_bf16(rng.normal(0.0, 0.5, size=shape).astype(np.float32))
        elif name.endswith("conv1d.weight"):
            out[name] = f32_to_bf16(rng.normal(0.0, 0.3, size=shape).astype(np.float32))
        else:  # embedding table, conv weights
            out[name] = f32_to_bf16(rng.normal(0.0, 0.02, size=shape).astype(np.float32))
    return out
