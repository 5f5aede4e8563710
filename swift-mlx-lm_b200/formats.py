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


# KV scheme identifier -> (values per block, bytes per block); dense schemes are one value per "block"
# (QuantizationFormatRegistry as KVCacheSpecification.resolveBlockLayout uses it, MetalGraphAllocator.swift:71-79)
KV_BLOCK_LAYOUTS = {0x00: (1, 2), 0x01: (1, 2), 0x02: (1, 4), 0x10: (32, 36), 0x11: (64, 68), 0x12: (128, 132),
                    0x40: (64, 36), 0x41: (128, 68), 0x42: (128, 68)}
KV_ROTOR_BASE = {0x70: 0x10, 0x71: 0x40}   # the rotated schemes store the block layout of their base scheme


@dataclass(frozen=True)
class KVCacheSpecification:
    """Sizing contract of the reference's KV cache (sequence-major layout; dense bf16 = scheme 0x01 by default).

    The device layout of this build packs head slots without the reference's padding (256 bytes for dense, 64 bytes
    for block-quantized slots); the figures below are the reference's, kept for the sizing contract tests.
    """

    layer_count: int
    kv_head_count: int
    head_dimension: int
    maximum_sequence_length: int
    scheme: int = 0x01

    token_slot_alignment = 256  # dense formats (MetalGraphAllocator.swift:90-114)

    @property
    def uses_rotor_quant(self) -> bool:
        return self.scheme in KV_ROTOR_BASE

    def slot_alignment(self) -> int:
        weights_per_block, _ = KV_BLOCK_LAYOUTS[KV_ROTOR_BASE.get(self.scheme, self.scheme)]
        return 64 if weights_per_block > 1 else self.token_slot_alignment

    def bytes_per_head_slot(self) -> int:
        weights_per_block, bytes_per_block = KV_BLOCK_LAYOUTS[KV_ROTOR_BASE.get(self.scheme, self.scheme)]
        blocks = (self.head_dimension + weights_per_block - 1) // weights_per_block
        return _align_up(blocks * bytes_per_block, self.slot_alignment())

    def bytes_per_token_slot(self) -> int:
        return self.kv_head_count * self.bytes_per_head_slot()

    def bytes_per_layer(self) -> int:
        return self.maximum_sequence_length * self.bytes_per_token_slot()

    def total_bytes(self) -> int:
        """K plus V over all layers for one sequence."""
        return 2 * self.layer_count * self.bytes_per_layer()

    # rotated schemes (MetalGraphAllocator.swift:177-216): one rotor (s, b12, b13, b23) of fp16 per KV head and group of
    # three values; with a projection dimension m > 0 a shared [head_dim][m] fp16 matrix and m fp16 values per cached K row
    def num_rotor_groups(self) -> int:
        return (self.head_dimension + 2) // 3

    def rotor_parameters_bytes_per_layer(self) -> int:
        return self.kv_head_count * self.num_rotor_groups() * 4 * 2

    def total_rotor_parameters_size(self) -> int:
        return self.layer_count * self.rotor_parameters_bytes_per_layer()

    def qjl_matrix_size(self, qjl_dimension: int) -> int:
        return self.head_dimension * qjl_dimension * 2 if qjl_dimension > 0 else 0

    def qjl_residual_bytes_per_layer(self, qjl_dimension: int) -> int:
        return self.maximum_sequence_length * self.kv_head_count * qjl_dimension * 2 if qjl_dimension > 0 else 0

    def total_qjl_residual_size(self, qjl_dimension: int) -> int:
        return self.layer_count * self.qjl_residual_bytes_per_layer(qjl_dimension)

    def sequence_major_offset(self, layer: int, head: int, position: int) -> int:
        head_stride = self.maximum_sequence_length * self.bytes_per_head_slot()
        return layer * self.kv_head_count * head_stride + head * head_stride + position * self.bytes_per_head_slot()
