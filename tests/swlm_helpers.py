"""Small helpers shared by the tests."""
import numpy as np


def pattern_bf16(count, mult, mod, scale):
    """bf16(((i*mult) % mod - mod/2) * scale) — the input generator of the reference's sequence-equivalence
    tests (Tests/MetalCompilerTests/Core/AttentionSequenceEquivalenceTests.swift:94-103); exact in bf16."""
    i = np.arange(count, dtype=np.int64)
    return (((i * mult) % mod - mod // 2).astype(np.float32) * np.float32(scale)).astype(np.float32)


def rel_err(got, ref):
    """Per-output relative error with the denominator floored at 2 % of the vector's largest magnitude, so
    that outputs which cancel to nearly zero are judged on the scale of the vector."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    floor = 0.02 * max(float(np.max(np.abs(ref))), 1e-30)
    return np.abs(got - ref) / np.maximum(np.abs(ref), floor)
