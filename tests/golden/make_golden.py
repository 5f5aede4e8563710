"""Regenerates tests/golden/reference_kat.json: the known-answer vectors of the reference's kernel tests.

The reference's tests build their inputs from closed-form patterns and compute the expected value with
a scalar Swift loop in Float (fp32). This script reproduces both, pattern for pattern, in pure Python with
NumPy fp32 scalars, so the committed file holds inputs AND expected outputs that do not come from this
repository's oracle or kernels. Sources (paths relative to the reference project root):

  gemv_single_block   Tests/MetalCompilerTests/Core/UnifiedGEMVBitLevelTests.swift:114-122, 205-208, 247-255
  gemv_multi_row      Tests/MetalCompilerTests/Core/UnifiedGEMVMultiRowTests.swift:108-176 and
                      Tests/MetalCompilerTests/Core/STAFEndToEndGEMVTests.swift:137-160, 252-255, 295-320
  gemv_multi_block_*  Tests/MetalCompilerTests/Core/UnifiedGEMVMultiBlockTests.swift:51-60, 108-215 (Q4G64, Q4G128)
  dequant_block       Tests/MetalCompilerTests/Core/UnifiedDequantBitLevelTests.swift:129-137
  rotor_defaults      Sources/MetalCompiler/Buffer/MetalGraphAllocator.swift:349-411 (the deterministic rotors and sign
                      matrix of the rotated KV schemes; the reference's tests check their properties, not their values)
  staf_roundtrip_*    Tests/MetalCompilerTests/Core/STAFQuantizedRoundtripTests.swift:133-143, 159-171, 187-198, 225-240
  attention_pattern   Tests/MetalCompilerTests/Core/AttentionSequenceEquivalenceTests.swift:21-43, 94-103
  conv_pattern        Tests/MetalCompilerTests/Core/Conv1dSequenceEquivalenceTests.swift:21-30

Run: python tests/golden/make_golden.py
"""
import base64
import json
import os
import struct

import numpy as np

F = np.float32


def f32_bits(x) -> int:
    return struct.unpack("<I", struct.pack("<f", float(F(x))))[0]


def bf16_round(x) -> F:
    b = f32_bits(x)
    b = (b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFFFFFF
    return F(struct.unpack("<f", struct.pack("<I", (b >> 16) << 16))[0])


def bf16_bits(x) -> int:
    return f32_bits(bf16_round(x)) >> 16


def f16_bits(x) -> int:
    return int(np.float16(F(x)).view(np.uint16))


def gemv_single_block():
    q = [k % 16 for k in range(64)]
    scale, zero = F(0.0625), F(-0.5)
    x = [F(np.float16(F(k % 10) * F(0.125) - F(0.5))) for k in range(64)]
    expected = F(0)
    for k in range(64):
        w = scale * F(q[k]) + zero
        expected = F(expected + F(w * x[k]))
    return {"q": q, "scale": float(scale), "zero": float(zero), "x": [float(v) for v in x],
            "expected": float(expected), "abs_tol": 0.01, "rel_tol": 0.02}


def gemv_multi_row(rows=4, blocks=4):
    k_total = 64 * blocks
    x = [F(np.float16(F(k % 13) * F(0.046875) - F(0.25))) for k in range(k_total)]
    q, scales, zeros, expected = [], [], [], []
    for r in range(rows):
        qr, sr, zr = [], [], []
        e = F(0)
        for b in range(blocks):
            scale = F(F(0.0625) * F(b + 1) + F(0.015625) * F(r))
            zero = F(F(-0.25) + F(0.125) * F(b) + F(0.03125) * F(r))
            qb = [(k + b * 7 + r * 3) % 16 for k in range(64)]
            for k in range(64):
                w = F(scale * F(qb[k]) + zero)
                e = F(e + F(w * x[b * 64 + k]))
            qr += qb
            sr.append(float(scale))
            zr.append(float(zero))
        q.append(qr); scales.append(sr); zeros.append(zr); expected.append(float(e))
    return {"rows": rows, "blocks": blocks, "q": q, "scales": scales, "zeros": zeros,
            "x": [float(v) for v in x], "expected": expected, "abs_tol": 0.03, "rel_tol": 0.03}


def gemv_multi_block(weights_per_block, blocks=4):
    """One output row over `blocks` consecutive blocks with their own scale and zero; fp32 expectation in block order."""
    total = weights_per_block * blocks
    x = [F(np.float16(F(F(k % 11) * F(0.0625)) - F(0.3))) for k in range(total)]
    q, scales, zeros = [], [], []
    e = F(0)
    for b in range(blocks):
        scale, zero = F(F(0.0625) * F(b + 1)), F(F(-0.25) + F(0.125) * F(b))
        qb = [(k + b * 7) % 16 for k in range(weights_per_block)]
        for k in range(weights_per_block):
            e = F(e + F(F(scale * F(qb[k]) + zero) * x[b * weights_per_block + k]))
        q += qb; scales.append(float(scale)); zeros.append(float(zero))
    return {"group": weights_per_block, "blocks": blocks, "q": q, "scales": scales, "zeros": zeros,
            "x": [float(v) for v in x], "expected": float(e), "abs_tol": 0.03, "rel_tol": 0.03}


def rotor_defaults(rotors=12, head_dim=8, qjl=4):
    """fp16 bit patterns of the first `rotors` unit rotors (four LCG draws each, mapped to [-1, 1), normalised in fp32) and
    of a head_dim x qjl sign matrix (+-1/sqrt(qjl) by bit 33 of the first draw of each index)."""
    a, c, mask = 6364136223846793005, 1442695040888963407, (1 << 64) - 1
    out = []
    for i in range(rotors):
        h, comp = i, []
        for _ in range(4):
            h = (h * a + c) & mask
            comp.append(F(F((h >> 33) - (1 << 30)) * F(1.0 / (1 << 30))))
        norm = F(np.sqrt(F(F(F(comp[0] * comp[0] + comp[1] * comp[1]) + comp[2] * comp[2]) + comp[3] * comp[3])))
        comp = [F(1), F(0), F(0), F(0)] if norm < 1e-8 else [F(v * F(F(1.0) / norm)) for v in comp]
        out.append([f16_bits(v) for v in comp])
    scale = F(F(1.0) / F(np.sqrt(F(qjl))))
    signs = [f16_bits(scale) if ((((i * a + c) & mask) >> 33) & 1) == 0 else f16_bits(-scale) for i in range(head_dim * qjl)]
    return {"rotors_f16_bits": out, "head_dim": head_dim, "qjl": qjl, "matrix_f16_bits": signs}


def dequant_block():
    q = [k % 16 for k in range(64)]
    scale, zero = F(0.0625), F(-0.5)
    return {"q": q, "scale": float(scale), "zero": float(zero),
            "expected_bf16_bits": [bf16_bits(F(scale * F(v) + zero)) for v in q]}


def pack_stream_bytes(q):
    """LSB-first 4-bit stream: weight k in byte k>>1, low nibble when k is even."""
    out = []
    for i in range(0, len(q), 2):
        out.append((q[i] & 0xF) | ((q[i + 1] & 0xF) << 4))
    return out


def staf_block(q, scale, zero):
    s, z = f16_bits(scale), f16_bits(zero)
    return [s & 0xFF, s >> 8, z & 0xFF, z >> 8] + pack_stream_bytes(q)


def staf_roundtrip_single():
    q = [k % 16 for k in range(64)]
    return {"rows": 1, "blocks": 1, "q": [q], "scales": [[0.0625]], "zeros": [[-0.5]],
            "expected_blocks": [staf_block(q, 0.0625, -0.5)]}


def staf_roundtrip_multi():
    rows, blocks = 2, 2
    q, scales, zeros, exp = [], [], [], []
    for r in range(rows):
        qr, sr, zr = [], [], []
        for b in range(blocks):
            seed = r * 37 + b * 11
            qb = [(seed + i) & 0xF for i in range(64)]
            scale = F(0.0625) * F(b + 1)
            zero = F(-0.5) + F(r) * F(0.125)
            qr += qb; sr.append(float(scale)); zr.append(float(zero))
            exp.append(staf_block(qb, scale, zero))
        q.append(qr); scales.append(sr); zeros.append(zr)
    return {"rows": rows, "blocks": blocks, "q": q, "scales": scales, "zeros": zeros, "expected_blocks": exp}


def pattern_bf16(count, mult, mod, scale):
    return [float(bf16_round(F(F((i * mult) % mod - mod // 2) * F(scale)))) for i in range(count)]


def attention_pattern(heads=8, kv_heads=2, head_dim=256, max_seq=8, seq_len=5):
    """Inputs of the reference's attention equivalence test plus an fp64 softmax-attention result for every
    position (no RoPE; the K/V rows of earlier positions are the bf16 patterns themselves, exact in bf16)."""
    qv = pattern_bf16(seq_len * heads * head_dim, 17, 29, 0.03125)
    kv = pattern_bf16(seq_len * kv_heads * head_dim, 13, 23, 0.03125)
    vv = pattern_bf16(seq_len * kv_heads * head_dim, 19, 31, 0.03125)
    q = np.array(qv, dtype=np.float64).reshape(seq_len, heads, head_dim)
    k = np.array(kv, dtype=np.float64).reshape(seq_len, kv_heads, head_dim)
    v = np.array(vv, dtype=np.float64).reshape(seq_len, kv_heads, head_dim)
    scale = 1.0 / np.sqrt(head_dim)
    out = np.zeros((seq_len, heads, head_dim))
    for p in range(seq_len):
        for h in range(heads):
            g = h * kv_heads // heads
            s = (k[: p + 1, g] @ q[p, h]) * scale
            w = np.exp(s - s.max())
            w /= w.sum()
            out[p, h] = w @ v[: p + 1, g]
    # inputs are regenerated from the (multiplier, modulus, scale) patterns by the tests; the expected
    # result is stored as little-endian fp32, base64
    return {"heads": heads, "kv_heads": kv_heads, "head_dim": head_dim, "max_seq": max_seq, "seq_len": seq_len,
            "q_pattern": [17, 29, 0.03125], "k_pattern": [13, 23, 0.03125], "v_pattern": [19, 31, 0.03125],
            "expected_f32_b64": base64.b64encode(out.astype("<f4").tobytes()).decode(), "tol": 2e-2}


def conv_pattern(dim=8, kernel=4, seq_len=6):
    """Inputs of the reference's conv equivalence test; expected output and final state from the causal
    sequence formula with its rounding rule (Sources/MetalCompiler/Generator/MetalSourceGenerator+ConvAndState.swift
    :162-177, :209-216): past taps are rounded through bf16, the current one is not."""
    in_dim = 3 * dim
    x = [F(np.float16(F((i * 19) % 23 - 11) * F(0.0625))) for i in range(seq_len * in_dim)]
    w = [bf16_round(F((i * 7) % 17 - 8) * F(0.03125)) for i in range(dim * kernel)]
    out_bits, state_bits = [], [[0] * dim for _ in range(kernel)]
    for pos in range(seq_len):
        for ch in range(dim):
            acc = F(0)
            for kk in range(kernel):
                src = pos - (kernel - 1) + kk
                if src >= 0:
                    bx = F(x[src * in_dim + ch] * x[src * in_dim + 2 * dim + ch])
                    if src != pos:
                        bx = bf16_round(bx)
                    acc = F(acc + F(bx * w[ch * kernel + kk]))
            c = x[pos * in_dim + dim + ch]
            out_bits.append(bf16_bits(F(c * acc)))
    for kk in range(kernel):
        src = seq_len - kernel + kk
        for ch in range(dim):
            if 0 <= src < seq_len:
                state_bits[kk][ch] = bf16_bits(F(x[src * in_dim + ch] * x[src * in_dim + 2 * dim + ch]))
    return {"dim": dim, "kernel": kernel, "seq_len": seq_len, "x": [float(v) for v in x],
            "w_bf16_bits": [bf16_bits(v) for v in w], "expected_out_bf16_bits": out_bits,
            "expected_state_bf16_bits": state_bits}


def main():
    data = {
        "gemv_single_block": gemv_single_block(),
        "gemv_multi_row": gemv_multi_row(),
        "gemv_multi_block_g64": gemv_multi_block(64),
        "gemv_multi_block_g128": gemv_multi_block(128),
        "dequant_block": dequant_block(),
        "rotor_defaults": rotor_defaults(),
        "staf_roundtrip_single": staf_roundtrip_single(),
        "staf_roundtrip_multi": staf_roundtrip_multi(),
        "attention_pattern": attention_pattern(),
        "attention_pattern_hd128": attention_pattern(head_dim=128),
        "conv_pattern": conv_pattern(),
    }
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kat.json")
    with open(path, "w") as f:
        json.dump(data, f)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
