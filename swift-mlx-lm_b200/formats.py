"""Format constants and host-side byte shuffling of the Q4 group-64 path (NumPy, integer/byte work only).

Mirrors, on the host: `AffineQ4Group64Format` (Sources/MetalCompiler/STAF/QuantizationFormat.swift:463-528),
`STAFPayloadConverter.repackMLXQuantized` (Sources/MetalCompiler/STAF/STAFPayloadConverter.swift:209-282)
and `KVCacheSpecification` sizing (Sources/MetalCompiler/Buffer/MetalGraphAllocator.swift:15-223).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


class AffineQ4Group64Format:
    """w = scale * q + zero, q in [0, 15]; 64 weights per block; STAF block = 36 bytes."""

    bits = 4
    group_size = 64
    weights_per_block = 64
    bytes_per_block = 36  # fp16 scale | fp16 zero | 32 payload bytes
    is_quantized = True
    scheme_identifier = "q4Group64ScaleF16"   # QuantizationSchemeIdentifier, STAF/STAFFormat.swift (0x40)

    @staticmethod
    def bytes_per_weight() -> float:
        return 36.0 / 64.0


class AffineQ4Group128Format:
    """The same arithmetic with one scale / zero pair per 128 weights; STAF block = 68 bytes
    (STAF/QuantizationFormat.swift:539-604)."""

    bits = 4
    group_size = 128
    weights_per_block = 128
    bytes_per_block = 68  # fp16 scale | fp16 zero | 64 payload bytes
    is_quantized = True
    scheme_identifier = "q4Group128ScaleF16"  # 0x41

    @staticmethod
    def bytes_per_weight() -> float:
        return 68.0 / 128.0


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (Sources/MetalCompiler/BFloat16.swift:25-32)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    return ((bits + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def pack_mlx_q4(q: np.ndarray) -> np.ndarray:
    """uint8 nibbles [n, k] -> MLX words u32 [n, k/8]; element j in bits [4(j%8), 4(j%8)+4) of word j/8."""
    q = np.ascontiguousarray(q, dtype=np.uint32)
    n, k = q.shape
    assert k % 8 == 0 and int(q.max(initial=0)) < 16
    shifts = (np.arange(8, dtype=np.uint32) * np.uint32(4))[None, None, :]
    return (q.reshape(n, k // 8, 8) << shifts).sum(axis=2, dtype=np.uint64).astype(np.uint32)


def unpack_mlx_q4(w: np.ndarray, k: int) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint32)
    shifts = (np.arange(8, dtype=np.uint32) * np.uint32(4))[None, None, :]
    return ((w[:, :, None] >> shifts) & np.uint32(0xF)).reshape(w.shape[0], k).astype(np.uint8)


def repack_mlx_to_staf(w: np.ndarray, scales_bf16: np.ndarray, biases_bf16: np.ndarray, group: int = 64) -> np.ndarray:
    """MLX triple -> STAF blocks, [n, k/group, 4 + group/2] uint8: 36 bytes for groups of 64 weights, 68 bytes for
    groups of 128 (AffineQ4Group128Format, STAF/QuantizationFormat.swift:539-604).

    Per (row, group): fp16(scale), fp16(bias), then the group's payload bytes verbatim — the MLX
    LSB-first bit stream already is the block's `qs` order (STAFPayloadConverter.swift:268-274); scale and
    bias are narrowed bf16 -> fp16 (:326-368).
    """
    n, words = w.shape
    groups = words * 8 // group
    out = np.zeros((n, groups, 4 + group // 2), dtype=np.uint8)
    s16 = bf16_to_f32(scales_bf16).astype(np.float16).view(np.uint16).reshape(n, groups)
    z16 = bf16_to_f32(biases_bf16).astype(np.float16).view(np.uint16).reshape(n, groups)
    out[:, :, 0:2] = s16[:, :, None].view(np.uint8).reshape(n, groups, 2)
    out[:, :, 2:4] = z16[:, :, None].view(np.uint8).reshape(n, groups, 2)
    out[:, :, 4:] = np.ascontiguousarray(w, dtype=np.uint32).view(np.uint8).reshape(n, groups, group // 2)
    return out


def _align_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


@dataclass(frozen=True)
class KVCacheSpecification:
    """Sizing contract of the reference's dense bf16 KV cache (scheme 0x01, sequence-major layout).

    The device layout of this build packs head slots without the 256-byte padding (it only matters for
    head_dim < 128); the figures below are the reference's, kept for the sizing contract tests.
    """

    layer_count: int
    kv_head_count: int
    head_dimension: int
    maximum_sequence_length: int

    token_slot_alignment = 256  # dense formats (MetalGraphAllocator.swift:90-114)

    def bytes_per_head_slot(self) -> int:
        return _align_up(self.head_dimension * 2, self.token_slot_alignment)

    def bytes_per_token_slot(self) -> int:
        return self.kv_head_count * self.bytes_per_head_slot()

    def bytes_per_layer(self) -> int:
        return self.maximum_sequence_length * self.bytes_per_token_slot()

    def total_bytes(self) -> int:
        """K plus V over all layers for one sequence."""
        return 2 * self.layer_count * self.bytes_per_layer()

    def sequence_major_offset(self, layer: int, head: int, position: int) -> int:
        head_stride = self.maximum_sequence_length * self.bytes_per_head_slot()
        return layer * self.kv_head_count * head_stride + head * head_stride + position * self.bytes_per_head_slot()
