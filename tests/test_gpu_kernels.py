"""Kernel-level parity on a B200: every CUDA kernel of the path against the CPU oracle, through the C ABI.

Tolerance for floating-point results: relative error <= 1e-2 per bf16 output (helper `rel_err`, denominator
floored at 2 % of the vector's largest magnitude). Integer / byte results (re-tiling, cache bytes, conv state,
argmax indices) are compared exactly.
"""
import base64
import ctypes as C

import numpy as np
import pytest

from swlm_helpers import pattern_bf16, rel_err

pytestmark = pytest.mark.gpu

RTOL = 1e-2


@pytest.fixture(scope="module")
def store(pkg):
    s = pkg.WeightStore(0)
    yield s
    s.close()


def _bf(pkg, a):
    return pkg.f32_to_bf16(np.asarray(a, dtype=np.float32))


# ---- qGEMV / small-M qGEMM --------------------------------------------------------------------------------

def test_qgemv_reference_known_answers(pkg, store, golden):
    g = golden["gemv_single_block"]
    w = pkg.pack_mlx_q4(np.array([g["q"]], dtype=np.uint8))
    store.add_q4_mlx("kat.single", w, _bf(pkg, [[g["scale"]]]), _bf(pkg, [[g["zero"]]]))
    y = pkg.bf16_to_f32(store.qgemm("kat.single", _bf(pkg, [g["x"]]), 1))
    assert abs(float(y[0, 0]) - g["expected"]) < max(g["abs_tol"], g["rel_tol"] * abs(g["expected"]))

    g = golden["gemv_multi_row"]
    w = pkg.pack_mlx_q4(np.array(g["q"], dtype=np.uint8))
    s, z = _bf(pkg, g["scales"]), _bf(pkg, g["zeros"])
    store.add_q4_mlx("kat.multi", w, s, z)
    # same tensor through the STAF execution-block format (fp16 headers), as the reference's end-to-end test does
    store.add_q4_staf("kat.multi.staf", pkg.formats.repack_mlx_to_staf(w, s, z), g["rows"], 64 * g["blocks"])
    for name in ("kat.multi", "kat.multi.staf"):
        y = pkg.bf16_to_f32(store.qgemm(name, _bf(pkg, [g["x"]]), g["rows"]))[0]
        for r in range(g["rows"]):
            assert abs(float(y[r]) - g["expected"][r]) < max(g["abs_tol"], g["rel_tol"] * abs(g["expected"][r]))


@pytest.mark.parametrize("n,k,m", [
    (4096, 4096, 1),      # the op-level benchmark shape
    (1, 64, 1), (17, 128, 1), (100, 320, 3), (33, 64 * 5, 2),   # ragged: padding rows and k-tiles
    (1024, 4096, 8), (4096, 14336, 1), (256, 14336, 16),        # batch columns; split-K through scratch
    (128, 512, 16), (6144, 4096, 4), (2048, 1792, 1),
])
def test_qgemm_matches_oracle(pkg, store, oracle, n, k, m):
    w, s, b = pkg.synth_q4(n, k, seed=n * 31 + k)
    rng = np.random.default_rng(m * 7 + 1)
    x = _bf(pkg, rng.normal(size=(m, k)))
    name = f"t.{n}x{k}"
    store.add_q4_mlx(name, w, s, b)
    got = pkg.bf16_to_f32(store.qgemm(name, x, n))
    oracle.set_threads(0)
    ref_bf16, ref64 = oracle.qgemm(x, w, s, b, want_f64=True)
    ref = pkg.bf16_to_f32(ref_bf16)
    for row in range(m):
        assert rel_err(got[row], ref[row]).max() <= RTOL
        # against the fp64 accumulation the kernel must be as close as bf16 rounding allows
        assert rel_err(got[row], ref64[row]).max() <= RTOL


@pytest.mark.parametrize("n,k,m", [(4096, 4096, 1), (100, 384, 3), (1024, 14336, 1), (512, 4096, 16), (768, 2048, 40), (1024, 4096, 128)])
def test_qgemm_group128_matches_oracle(pkg, store, oracle, n, k, m):
    """One scale / bias pair per 128 weights (AffineQ4Group128Format): through the MLX entry point and through 68-byte
    STAF blocks, in the single-sequence kernel, the 2..16-sequence kernel and the tensor-core product. The oracle
    dequantises with the group-128 parameters natively."""
    w, s, b = pkg.synth_q4(n, k, seed=n * 13 + k, group=128)
    assert s.shape == (n, k // 128)
    rng = np.random.default_rng(m * 5 + 2)
    x = _bf(pkg, rng.normal(size=(m, k)))
    store.add_q4_mlx(f"g128.{n}x{k}", w, s, b)
    store.add_q4_staf(f"g128s.{n}x{k}", pkg.formats.repack_mlx_to_staf(w, s, b, group=128), n, k, group=128)
    oracle.set_threads(0)
    for name, fp16 in ((f"g128.{n}x{k}", False), (f"g128s.{n}x{k}", True)):
        got = pkg.bf16_to_f32(store.qgemm(name, x, n))
        ref_bf16, ref64 = oracle.qgemm(x, w, s, b, staf_fp16=fp16, want_f64=True)
        ref = pkg.bf16_to_f32(ref_bf16)
        for row in range(m):
            assert rel_err(got[row], ref[row]).max() <= RTOL
            assert rel_err(got[row], ref64[row]).max() <= RTOL
    # the dequantised matrix, bit for bit
    if n * k <= 4096 * 4096:
        ref = pkg.f32_to_bf16(oracle.dequant_staf_group(oracle.staf_repack_group(w, s, b, 128), n, k, 128))
        assert np.array_equal(store.dequant_bf16(f"g128s.{n}x{k}", n, k), ref)
    with pytest.raises(ValueError):
        store.add_q4_mlx("g128.bad", w, s[:, :-1], b[:, :-1])


@pytest.mark.parametrize("m", [17, 40, 63])
def test_qgemm_17_to_63_rows_ride_in_one_tensor_core_tile(pkg, store, oracle, m):
    """Between 17 and 63 token rows the product runs once over the weights, in a 64-token tensor-core tile whose
    remaining rows are zero (the reference's gemm_q4_g64 re-reads the weights for every row,
    Generator/MetalSourceGenerator+Quantized.swift:88-156)."""
    n, k = 512, 1024
    w, s, b = pkg.synth_q4(n, k, seed=5)
    x = _bf(pkg, np.random.default_rng(2).normal(size=(m, k)))
    store.add_q4_mlx(f"t.mid{m}", w, s, b)
    got = pkg.bf16_to_f32(store.qgemm(f"t.mid{m}", x, n))
    ref = pkg.bf16_to_f32(oracle.qgemm(x, w, s, b))
    assert rel_err(got, ref).max() <= RTOL


@pytest.mark.parametrize("n,k,m", [
    (128, 64, 64),        # one tile, one group
    (256, 256, 64),
    (192, 512, 100),      # ragged in both the weight rows and the tokens
    (512, 4096, 128),     # 128-token tile
    (1000, 1024, 300),    # several token tiles, last one partial
])
def test_qgemm_tensor_core_matches_oracle(pkg, store, oracle, n, k, m):
    """More than 16 token rows run on the tcgen05 kernel. Its operands are exact (scale * (q - 8) in fp16, the
    group constants and group sums as fp16 pairs, activations scaled by a power of two per token), so the result
    differs from the oracle's fp32-weight product (gemm_q4_g64, Generator/MetalSourceGenerator+Quantized.swift:126-153,
    the route the reference actually runs) only by the order of the fp32 sums: 1e-2 per output against it and
    against an fp64 product of the exactly dequantised weights."""
    w, s, b = pkg.synth_q4(n, k, seed=n * 17 + k + m)
    x = _bf(pkg, np.random.default_rng(m).normal(size=(m, k)))
    name = f"tc.{n}x{k}x{m}"
    store.add_q4_mlx(name, w, s, b)
    got = pkg.bf16_to_f32(store.qgemm(name, x, n))
    wq = oracle.dequant_mlx(w, s, b).astype(np.float64)
    ref = pkg.bf16_to_f32(pkg.f32_to_bf16((pkg.bf16_to_f32(x).astype(np.float64) @ wq.T).astype(np.float32)))
    oracle.set_threads(0)
    ref32 = pkg.bf16_to_f32(oracle.qgemm(x, w, s, b))
    for r in range(m):
        assert rel_err(got[r], ref[r]).max() <= RTOL
        assert rel_err(got[r], ref32[r]).max() <= RTOL
    # and much closer than that on the whole: no 16-bit rounding of the weights is left in the path
    assert np.linalg.norm(got - ref) <= 3e-3 * np.linalg.norm(ref)


@pytest.mark.parametrize("n,m", [(14336, 64), (14336, 256), (14336, 512), (4096, 512)])
def test_qgemm_prefill_sweep_shapes_against_oracle(pkg, store, oracle, n, m):
    """The prefill sweep's shapes (K = 4096, N = 14336 and 4096, M = 64 / 256 / 512) against the oracle's
    fp32-weight product (gemm_q4_g64, Generator/MetalSourceGenerator+Quantized.swift:126-153), per output."""
    k = 4096
    w, s, b = pkg.synth_q4(n, k, seed=n + m)
    x = _bf(pkg, np.random.default_rng(m).normal(size=(m, k)))
    name = f"sweep.{n}x{m}"
    store.add_q4_mlx(name, w, s, b)
    got = pkg.bf16_to_f32(store.qgemm(name, x, n))
    oracle.set_threads(0)
    ref = pkg.bf16_to_f32(oracle.qgemm(x, w, s, b))
    err = np.array([rel_err(got[r], ref[r]).max() for r in range(m)])
    assert err.max() <= RTOL, f"worst token row {int(err.argmax())}: {err.max():.4f}"


@pytest.mark.parametrize("n,k,m", [(384, 1024, 64), (130, 128, 128)])
def test_qgemm_tensor_core_one_hot_is_bit_exact(pkg, store, oracle, n, k, m):
    """One-hot tokens pick single columns of the dequantised matrix: the tensor-core path must return
    bf16(scale * q + zero) bit for bit, which pins the nibble order, the shared-memory swizzle, the split into
    scale * (q - 8) plus the group constant, and the accumulator read-out at once."""
    w, s, b = pkg.synth_q4(n, k, seed=n + k)
    cols = (np.arange(m) * 37 + 5) % k
    x = np.zeros((m, k), dtype=np.float32)
    x[np.arange(m), cols] = 1.0
    store.add_q4_mlx(f"tc1h.{n}", w, s, b)
    got = store.qgemm(f"tc1h.{n}", _bf(pkg, x), n)
    want = oracle.dequant_bf16(w, s, b)
    assert np.array_equal(got, want[:, cols].T)


def test_device_layout_dequantises_bit_exactly(pkg, store, oracle):
    for n, k in [(48, 256), (37, 64 * 7), (512, 4096)]:
        w, s, b = pkg.synth_q4(n, k, seed=n + k)
        store.add_q4_mlx(f"dq.{n}", w, s, b)
        assert np.array_equal(store.dequant_bf16(f"dq.{n}", n, k), oracle.dequant_bf16(w, s, b))


def test_dequant_known_answer_bits(pkg, store, golden):
    g = golden["dequant_block"]
    w = pkg.pack_mlx_q4(np.array([g["q"]], dtype=np.uint8))
    store.add_q4_mlx("kat.dq", w, _bf(pkg, [[g["scale"]]]), _bf(pkg, [[g["zero"]]]))
    assert store.dequant_bf16("kat.dq", 1, 64)[0].tolist() == g["expected_bf16_bits"]


def test_one_hot_probes_at_full_size(pkg, store, oracle):
    """Size-independent property at the full 14336 x 4096 shape: a one-hot activation returns the
    dequantised column, so every probed weight is checked without a CPU GEMV."""
    n, k = 14336, 4096
    w, s, b = pkg.synth_q4(n, k, seed=99)
    store.add_q4_mlx("probe", w, s, b)
    cols = [0, 63, 64, 1000, 4095]
    x = np.zeros((len(cols), k), dtype=np.float32)
    for i, c in enumerate(cols):
        x[i, c] = 1.0
    got = pkg.bf16_to_f32(store.qgemm("probe", _bf(pkg, x), n))
    deq = oracle.dequant_mlx(w, s, b)
    for i, c in enumerate(cols):
        want = pkg.bf16_to_f32(pkg.f32_to_bf16(deq[:, c]))
        assert np.max(np.abs(got[i] - want) / np.maximum(np.abs(want), 1e-3)) <= 2.0 ** -7  # one bf16 ulp


# ---- glue kernels through single plan steps -----------------------------------------------------------------

def _mini(pkg, store, oracle, *, batch=1, hidden=256, slot=1024, vocab=512, max_seq=64, kv_layers=1, kv_heads=2,
          head_dim=128, conv_layers=0, conv_dim=0, conv_kernel=0):
    desc = pkg.BuffersDesc(hidden=hidden, slot_dim=slot, vocab=vocab, max_seq=max_seq, max_batch=batch,
                           kv_layers=kv_layers, kv_heads=kv_heads, head_dim=head_dim, conv_layers=conv_layers,
                           conv_dim=conv_dim, conv_kernel=conv_kernel)
    table = _bf(pkg, np.random.default_rng(0).normal(0, 0.02, size=(vocab, hidden)))
    if not getattr(store, "_mini_table", None) == (vocab, hidden):
        store.add_dense("mini.embed", table)
        store._mini_table = (vocab, hidden)
    step = pkg.plan._step(pkg.plan.STEP_EMBED, out_buf=0, n=hidden, weight="mini.embed")
    gm = pkg.InferenceModel(store, [step], desc)
    om = oracle.model(desc)
    om.add_dense("mini.embed", table)
    return gm, om


@pytest.mark.parametrize("kind_name", ["STEP_COPY_RMSNORM", "STEP_RESADD_COPY_RMSNORM", "STEP_RESADD_RMSNORM"])
@pytest.mark.parametrize("batch", [1, 3])
def test_rmsnorm_family(pkg, store, oracle, kind_name, batch):
    P = pkg.plan
    hidden = 4096
    gm, om = _mini(pkg, store, oracle, batch=batch, hidden=hidden, slot=4096)
    rng = np.random.default_rng(3)
    wn = _bf(pkg, 1.0 + rng.normal(0, 0.02, size=hidden))
    store.add_dense("n.w", wn)
    om.add_dense("n.w", wn)
    h = _bf(pkg, rng.normal(size=(batch, hidden)))
    r = _bf(pkg, rng.normal(size=(batch, hidden)))
    for mdl in (gm, om):
        mdl.write_buffer(P.BUF_HIDDEN, h)
        mdl.write_buffer(P.BUF_RESIDUAL, r)
    step = P._step(getattr(P, kind_name), in_buf=P.BUF_HIDDEN, out_buf=P.BUF_S0, n=hidden, eps=1e-5, weight_bias=0.0, weight="n.w")
    gm.run_step(step)
    om.run_step(step)
    got, ref = pkg.bf16_to_f32(gm.read_buffer(P.BUF_S0, hidden)), pkg.bf16_to_f32(om.read_buffer(P.BUF_S0, hidden))
    assert rel_err(got, ref).max() <= RTOL
    # the residual stream is a sum of two bf16 values rounded once: exact
    assert np.array_equal(gm.read_buffer(P.BUF_RESIDUAL, hidden), om.read_buffer(P.BUF_RESIDUAL, hidden))
    gm.close()


def test_qk_norm_swiglu_embed_argmax(pkg, store, oracle):
    P = pkg.plan
    batch, heads, kvh, hd = 2, 8, 2, 64
    gm, om = _mini(pkg, store, oracle, batch=batch, hidden=256, slot=1024, vocab=512, head_dim=hd)
    rng = np.random.default_rng(4)
    wq, wk = _bf(pkg, 1 + rng.normal(0, 0.1, size=hd)), _bf(pkg, 1 + rng.normal(0, 0.1, size=hd))
    for mdl in (store, om):
        mdl.add_dense("qn", wq)
        mdl.add_dense("kn", wk)
    q, k = _bf(pkg, rng.normal(size=(batch, heads * hd))), _bf(pkg, rng.normal(size=(batch, kvh * hd)))
    step = P._step(P.STEP_QK_NORM, in_buf=P.BUF_S1, in2_buf=P.BUF_S2, heads=heads, kv_heads=kvh, head_dim=hd, eps=1e-5,
                   weight_bias=0.0, weight="qn", weight2="kn")
    for mdl in (gm, om):
        mdl.write_buffer(P.BUF_S1, q)
        mdl.write_buffer(P.BUF_S2, k)
        mdl.run_step(step)
    for buf, cnt in ((P.BUF_S1, heads * hd), (P.BUF_S2, kvh * hd)):
        assert rel_err(pkg.bf16_to_f32(gm.read_buffer(buf, cnt)), pkg.bf16_to_f32(om.read_buffer(buf, cnt))).max() <= RTOL

    g, u = _bf(pkg, rng.normal(size=(batch, 1000)) * 3), _bf(pkg, rng.normal(size=(batch, 1000)))
    step = P._step(P.STEP_SWIGLU, in_buf=P.BUF_S1, in2_buf=P.BUF_S2, out_buf=P.BUF_S0, n=1000)
    for mdl in (gm, om):
        mdl.write_buffer(P.BUF_S1, g)
        mdl.write_buffer(P.BUF_S2, u)
        mdl.run_step(step)
    assert rel_err(pkg.bf16_to_f32(gm.read_buffer(P.BUF_S0, 1000)), pkg.bf16_to_f32(om.read_buffer(P.BUF_S0, 1000))).max() <= RTOL

    step = P._step(P.STEP_EMBED, out_buf=P.BUF_HIDDEN, n=256, weight="mini.embed")
    toks = np.array([511, 7], dtype=np.int32)
    gm.run_step(step, toks)
    om.run_step(step, toks)
    assert np.array_equal(gm.read_buffer(P.BUF_HIDDEN, 256), om.read_buffer(P.BUF_HIDDEN, 256))

    # argmax: ties resolve to the lowest index; -inf rows and a maximum in the last element
    logits = rng.normal(size=(batch, 512)).astype(np.float32)
    logits[0, [100, 37, 400]] = 9.0
    logits[1, 511] = 50.0
    step = P._step(P.STEP_ARGMAX, in_buf=P.BUF_LOGITS, n=512)
    for mdl in (gm, om):
        mdl.write_buffer(P.BUF_LOGITS, _bf(pkg, logits))
    assert gm.run_step(step).tolist() == om.run_step(step).tolist() == [37, 511]
    assert gm.position == 0  # single-step runs leave the position alone
    gm.close()


def test_argmax_full_vocab(pkg, store, oracle):
    P = pkg.plan
    vocab = 128256
    gm, om = _mini(pkg, store, oracle, batch=2, hidden=256, slot=1024, vocab=vocab)
    rng = np.random.default_rng(5)
    logits = _bf(pkg, rng.normal(size=(2, vocab)))  # bf16 rounding creates plenty of exact ties
    step = P._step(P.STEP_ARGMAX, in_buf=P.BUF_LOGITS, n=vocab)
    for mdl in (gm, om):
        mdl.write_buffer(P.BUF_LOGITS, logits)
    assert gm.run_step(step).tolist() == om.run_step(step).tolist()
    gm.close()


def test_conv_state_update_known_answer_bits(pkg, store, oracle, golden):
    g = golden["conv_pattern"]
    D, K, T = g["dim"], g["kernel"], g["seq_len"]
    P = pkg.plan
    gm, _ = _mini(pkg, store, oracle, hidden=256, slot=1024, conv_layers=1, conv_dim=D, conv_kernel=K)
    store.add_dense("kat.conv", np.array(g["w_bf16_bits"], dtype=np.uint16).reshape(D, K))
    step = P._step(P.STEP_CONV_STATE_UPDATE, layer=0, in_buf=P.BUF_S1, out_buf=P.BUF_S0, n=D, conv_kernel=K, weight="kat.conv")
    x = np.array(g["x"], dtype=np.float32).reshape(T, 3 * D)
    out_bits = []
    for t in range(T):
        row = np.zeros((1, 1024), dtype=np.float32)
        row[0, : 3 * D] = x[t]
        gm.write_buffer(P.BUF_S1, _bf(pkg, row))
        gm.run_step(step)
        out_bits += gm.read_buffer(P.BUF_S0, D)[0].tolist()
    assert out_bits == g["expected_out_bf16_bits"]
    assert gm.read_conv(0, 0).tolist() == g["expected_state_bf16_bits"]
    gm.close()


# ---- attention --------------------------------------------------------------------------------------------

def test_attention_reference_pattern(pkg, store, oracle, golden):
    g = golden["attention_pattern_hd128"]
    H, KV, D, T = g["heads"], g["kv_heads"], g["head_dim"], g["seq_len"]
    P = pkg.plan
    q = pattern_bf16(T * H * D, *g["q_pattern"]).reshape(T, H * D)
    k = pattern_bf16(T * KV * D, *g["k_pattern"]).reshape(T, KV * D)
    v = pattern_bf16(T * KV * D, *g["v_pattern"]).reshape(T, KV * D)
    expected = np.frombuffer(base64.b64decode(g["expected_f32_b64"]), dtype="<f4").reshape(T, H * D)
    gm, _ = _mini(pkg, store, oracle, hidden=256, slot=H * D, max_seq=g["max_seq"], kv_heads=KV, head_dim=D)
    step = P._step(P.STEP_ATTN_DECODE, layer=0, in_buf=P.BUF_S1, in2_buf=P.BUF_S2, in3_buf=P.BUF_S3, out_buf=P.BUF_S0,
                   heads=H, kv_heads=KV, head_dim=D, rope_dim=0, rope_base=0.0, scale=1.0 / np.sqrt(D))
    pad = lambda a: np.pad(a, (0, H * D - a.size))[None, :]
    for t in range(T):
        gm.set_position(t)
        gm.write_buffer(P.BUF_S1, _bf(pkg, pad(q[t])))
        gm.write_buffer(P.BUF_S2, _bf(pkg, pad(k[t])))
        gm.write_buffer(P.BUF_S3, _bf(pkg, pad(v[t])))
        gm.run_step(step)
        out = pkg.bf16_to_f32(gm.read_buffer(P.BUF_S0, H * D))[0]
        assert np.max(np.abs(out - expected[t])) < g["tol"] * max(1.0, np.max(np.abs(expected[t])))
    # cache bytes equal the (bf16-exact) inputs, as the reference asserts between its two fill paths
    for h in range(KV):
        assert np.array_equal(pkg.bf16_to_f32(gm.read_kv(0, 0, 0, h, T)), k.reshape(T, KV, D)[:, h])
        assert np.array_equal(pkg.bf16_to_f32(gm.read_kv(1, 0, 0, h, T)), v.reshape(T, KV, D)[:, h])
    gm.close()


@pytest.mark.parametrize("hd,heads,kvh", [(128, 32, 8), (64, 32, 8), (128, 8, 8)])
@pytest.mark.parametrize("batch,ctx", [(1, 0), (1, 1), (1, 63), (1, 64), (1, 65), (1, 1000), (1, 4095), (3, 300)])
def test_attention_decode_matches_oracle(pkg, store, oracle, hd, heads, kvh, batch, ctx):
    """RoPE(q, k_new), KV append, attention over [0, ctx] with the cache pre-filled with random bf16 rows."""
    P = pkg.plan
    max_seq = 4096
    gm, om = _mini(pkg, store, oracle, batch=batch, hidden=256, slot=heads * hd, max_seq=max_seq, kv_heads=kvh, head_dim=hd)
    rng = np.random.default_rng(ctx * 13 + hd + batch)
    if ctx:
        for b in range(batch):
            for h in range(kvh):
                kr, vr = _bf(pkg, rng.normal(size=(ctx, hd))), _bf(pkg, rng.normal(size=(ctx, hd)))
                for mdl in (gm, om):
                    mdl.write_kv(0, 0, b, h, kr)
                    mdl.write_kv(1, 0, b, h, vr)
    q = _bf(pkg, rng.normal(size=(batch, heads * hd)))
    k = _bf(pkg, np.pad(rng.normal(size=(batch, kvh * hd)), ((0, 0), (0, (heads - kvh) * hd))))
    v = _bf(pkg, np.pad(rng.normal(size=(batch, kvh * hd)), ((0, 0), (0, (heads - kvh) * hd))))
    step = P._step(P.STEP_ATTN_DECODE, layer=0, in_buf=P.BUF_S1, in2_buf=P.BUF_S2, in3_buf=P.BUF_S3, out_buf=P.BUF_S0,
                   heads=heads, kv_heads=kvh, head_dim=hd, rope_dim=hd, rope_base=500000.0, scale=1.0 / np.sqrt(hd))
    for mdl in (gm, om):
        mdl.set_position(ctx)
        mdl.write_buffer(P.BUF_S1, q)
        mdl.write_buffer(P.BUF_S2, k)
        mdl.write_buffer(P.BUF_S3, v)
        mdl.run_step(step)
    got = pkg.bf16_to_f32(gm.read_buffer(P.BUF_S0, heads * hd))
    ref = pkg.bf16_to_f32(om.read_buffer(P.BUF_S0, heads * hd))
    assert rel_err(got, ref).max() <= RTOL
    # the appended K row (RoPE in fp32, rounded once) and V row
    for b in range(batch):
        for h in range(kvh):
            gk, ok = gm.read_kv(0, 0, b, h, ctx + 1)[ctx], om.read_kv(0, 0, b, h, ctx + 1)[ctx]
            assert rel_err(pkg.bf16_to_f32(gk), pkg.bf16_to_f32(ok)).max() <= RTOL
            assert np.array_equal(gm.read_kv(1, 0, b, h, ctx + 1)[ctx], om.read_kv(1, 0, b, h, ctx + 1)[ctx])
    gm.close()


@pytest.mark.parametrize("window,ctx", [(1, 300), (16, 5), (16, 15), (16, 16), (16, 17), (64, 200), (100, 1000), (1000, 4095),
                                        (4096, 700), (63, 2111), (129, 4000)])
@pytest.mark.parametrize("hd,heads,kvh,batch", [(128, 32, 8, 1), (64, 16, 4, 2)])
def test_attention_decode_sliding_window_matches_oracle(pkg, store, oracle, hd, heads, kvh, batch, window, ctx):
    """windowLeft: the new token attends itself and the window - 1 cached rows before it, wherever the window's
    left edge falls relative to the 64-row blocks the splits walk (inside the first block, on a block boundary,
    whole splits below it), and a window wider than the context changes nothing."""
    P = pkg.plan
    max_seq = 4096
    gm, om = _mini(pkg, store, oracle, batch=batch, hidden=256, slot=heads * hd, max_seq=max_seq, kv_heads=kvh, head_dim=hd)
    rng = np.random.default_rng(ctx * 7 + window)
    for b in range(batch):
        for h in range(kvh):
            kr, vr = _bf(pkg, rng.normal(size=(ctx, hd))), _bf(pkg, rng.normal(size=(ctx, hd)))
            for mdl in (gm, om):
                mdl.write_kv(0, 0, b, h, kr)
                mdl.write_kv(1, 0, b, h, vr)
    q = _bf(pkg, rng.normal(size=(batch, heads * hd)))
    k = _bf(pkg, np.pad(rng.normal(size=(batch, kvh * hd)), ((0, 0), (0, (heads - kvh) * hd))))
    v = _bf(pkg, np.pad(rng.normal(size=(batch, kvh * hd)), ((0, 0), (0, (heads - kvh) * hd))))
    outs = {}
    for w in (window, 0):
        step = P._step(P.STEP_ATTN_DECODE, layer=0, in_buf=P.BUF_S1, in2_buf=P.BUF_S2, in3_buf=P.BUF_S3, out_buf=P.BUF_S0,
                       heads=heads, kv_heads=kvh, head_dim=hd, rope_dim=hd, rope_base=500000.0, scale=1.0 / np.sqrt(hd),
                       window_left=w)
        for mdl in (gm, om):
            mdl.set_position(ctx)
            mdl.write_buffer(P.BUF_S1, q)
            mdl.write_buffer(P.BUF_S2, k)
            mdl.write_buffer(P.BUF_S3, v)
            mdl.run_step(step)
        outs[w] = (pkg.bf16_to_f32(gm.read_buffer(P.BUF_S0, heads * hd)), pkg.bf16_to_f32(om.read_buffer(P.BUF_S0, heads * hd)))
    got, ref = outs[window]
    assert rel_err(got, ref).max() <= RTOL
    if window > ctx:
        assert np.array_equal(outs[window][0], outs[0][0])       # the window covers everything
    else:
        assert not np.array_equal(outs[window][1], outs[0][1])   # ... or it really leaves rows out
    gm.close()


@pytest.mark.parametrize("B,ctx", [(4, 8192), (1, 32768), (8, 32768), (64, 1024)])
def test_flash_decode_op_long_context(pkg, store, B, ctx):
    """Config-2 shapes (32 query / 8 KV heads of 128, contexts up to 32768, batches up to 64) through the
    device-pointer entry point, against a PyTorch fp32 reference of the same op."""
    import torch

    lib = store.lib
    H, KV, D = 32, 8, 128
    gen = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(B, H, D, device="cuda", generator=gen).bfloat16()
    k = torch.randn(B, KV, ctx, D, device="cuda", generator=gen).bfloat16()
    v = torch.randn(B, KV, ctx, D, device="cuda", generator=gen).bfloat16()
    out = torch.empty(B, H, D, device="cuda", dtype=torch.bfloat16)
    scratch = torch.empty(lib.swlm_op_flash_decode_scratch_bytes(B, H, KV, D, ctx), device="cuda", dtype=torch.uint8)
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    lib.check(lib.swlm_op_flash_decode_dev(store.handle, B, H, KV, D, ctx, ctx, 1.0 / np.sqrt(D), q.data_ptr(), k.data_ptr(),
                                           v.data_ptr(), out.data_ptr(), scratch.data_ptr(), C.c_void_p(stream)))
    torch.cuda.synchronize()
    qf = q.float().view(B, KV, H // KV, D)
    s = torch.einsum("bgrd,bgtd->bgrt", qf, k.float()) / np.sqrt(D)
    ref = torch.einsum("bgrt,bgtd->bgrd", torch.softmax(s, dim=-1), v.float()).reshape(B, H, D)
    err = rel_err(out.float().cpu().numpy().reshape(B * H, D), ref.cpu().numpy().reshape(B * H, D))
    assert err.max() <= RTOL


# ---- recurrent (gated delta rule) step ---------------------------------------------------------------------

@pytest.mark.parametrize("heads,groups,dk,dv,K,batch", [(4, 2, 16, 16, 4, 1), (32, 16, 128, 128, 4, 1), (8, 8, 64, 128, 3, 2),
                                                        (6, 2, 32, 64, 4, 3)])
def test_ssm_recurrence_matches_oracle_over_steps(pkg, store, oracle, heads, groups, dk, dv, K, batch):
    """ssm_recurrence (the DeltaNet / Qwen3.5 linear-attention step): 5 steps with the conv state and the fp32 recurrent
    state carried, outputs against the oracle per step, states at the end; (32, 16, 128, 128) is the full-size layer."""
    from test_oracle_golden import ssm_case, ssm_step_and_desc
    c = ssm_case(pkg, heads=heads, groups=groups, dk=dk, dv=dv, K=K, batch=batch, seed=heads + dk)
    desc, step, width = ssm_step_and_desc(pkg, c, max_batch=batch)
    tag = f"ssm{heads}x{dk}x{dv}b{batch}"
    for name in ("weight", "weight2", "weight3", "weight4"):
        setattr(step, name, getattr(step, name).replace(b"l0.", tag.encode() + b"."))
    P = pkg.plan
    store.add_dense(tag + ".conv1d.weight", _bf(pkg, c["conv_w"]))
    store.add_dense_f32(tag + ".norm.weight", c["norm_w"])
    store.add_dense(tag + ".dt_bias", _bf(pkg, c["dt_bias"]))
    store.add_dense_f32(tag + ".A_log", c["a_log"])
    store.add_dense("ssm.embed", np.zeros((8, 256), dtype=np.uint16))
    steps = [P._step(P.STEP_EMBED, out_buf=P.BUF_HIDDEN, n=256, weight="ssm.embed"), step]
    gm = pkg.InferenceModel(store, steps, desc)
    om = oracle.model(desc)
    om.add_dense(tag + ".conv1d.weight", _bf(pkg, c["conv_w"]))
    om.add_dense_f32(tag + ".norm.weight", c["norm_w"])
    om.add_dense(tag + ".dt_bias", _bf(pkg, c["dt_bias"]))
    om.add_dense_f32(tag + ".A_log", c["a_log"])
    rng = c["rng"]
    pad = lambda a: np.pad(a, ((0, 0), (0, width - a.shape[1])))
    for t in range(5):
        ins = {P.BUF_S1: rng.normal(size=(batch, c["conv_dim"])), P.BUF_S2: rng.normal(size=(batch, heads * dv)),
               P.BUF_S3: rng.normal(size=(batch, heads)), P.BUF_S4: rng.normal(size=(batch, heads))}
        for buf, v in ins.items():
            for mdl in (gm, om):
                mdl.write_buffer(buf, _bf(pkg, pad(v)))
        gm.run_step(step)
        om.run_step(step)
        got = pkg.bf16_to_f32(gm.read_buffer(P.BUF_S0, heads * dv))
        ref = pkg.bf16_to_f32(om.read_buffer(P.BUF_S0, heads * dv))
        assert rel_err(got, ref).max() <= RTOL, t
    for b in range(batch):
        gs, os_ = gm.read_ssm_state(0, b), om.read_ssm_state(0, b)
        assert np.max(np.abs(gs - os_)) <= 1e-4 * max(1.0, np.max(np.abs(os_)))
    # a sequence that is reset starts from an empty state again
    gm.reset_sequence(0)
    assert not gm.read_ssm_state(0, 0).any()
    gm.close()


# ---- 8-bit KV cache ----------------------------------------------------------------------------------------

KV_SCHEMES = {0x10: (8, 32), 0x11: (8, 64), 0x12: (8, 128), 0x40: (4, 64), 0x41: (4, 128), 0x42: (4, 128)}


@pytest.mark.parametrize("scheme", sorted(KV_SCHEMES))
@pytest.mark.parametrize("hd,heads,kvh", [(128, 32, 8), (64, 16, 4), (128, 8, 8)])
@pytest.mark.parametrize("batch,ctx,window", [(1, 0, 0), (1, 1, 0), (1, 65, 0), (1, 1000, 0), (1, 4095, 0), (3, 300, 0), (1, 900, 100)])
def test_attention_decode_over_q8_group32_cache(pkg, store, oracle, hd, heads, kvh, batch, ctx, window, scheme):
    """KV rows as blocks of 8- or 4-bit values (36 bytes per 32 8-bit values, and the other four schemes): the cache is
    filled through the probe (quantised on the host by both sides with the reference's rule, so both start from the
    same bytes), one decode step appends the new token's row and attends; output and the appended (dequantised) rows
    against the oracle."""
    bits, group = KV_SCHEMES[scheme]
    if group > hd:
        pytest.skip("a group wider than the head dimension is refused")
    levels = 255.0 if bits == 8 else 15.0
    P = pkg.plan
    max_seq = 4096
    desc = pkg.BuffersDesc(hidden=256, slot_dim=heads * hd, vocab=512, max_seq=max_seq, max_batch=batch, kv_layers=1, kv_heads=kvh,
                           head_dim=hd, conv_layers=0, conv_dim=0, conv_kernel=0, kv_scheme=scheme)
    table = _bf(pkg, np.zeros((512, 256)))
    store.add_dense("q8.embed", table)
    gm = pkg.InferenceModel(store, [P._step(P.STEP_EMBED, out_buf=0, n=256, weight="q8.embed")], desc)
    om = oracle.model(desc)
    rng = np.random.default_rng(ctx * 3 + hd + batch)
    if ctx:
        for b in range(batch):
            for h in range(kvh):
                kr, vr = _bf(pkg, rng.normal(size=(ctx, hd))), _bf(pkg, rng.normal(size=(ctx, hd)))
                for mdl in (gm, om):
                    mdl.write_kv(0, 0, b, h, kr)
                    mdl.write_kv(1, 0, b, h, vr)
        assert np.array_equal(gm.read_kv(0, 0, 0, 0, ctx), om.read_kv(0, 0, 0, 0, ctx))   # same bytes, same dequantisation
    q = _bf(pkg, rng.normal(size=(batch, heads * hd)))
    k = _bf(pkg, np.pad(rng.normal(size=(batch, kvh * hd)), ((0, 0), (0, (heads - kvh) * hd))))
    v = _bf(pkg, np.pad(rng.normal(size=(batch, kvh * hd)), ((0, 0), (0, (heads - kvh) * hd))))
    step = P._step(P.STEP_ATTN_DECODE, layer=0, in_buf=P.BUF_S1, in2_buf=P.BUF_S2, in3_buf=P.BUF_S3, out_buf=P.BUF_S0,
                   heads=heads, kv_heads=kvh, head_dim=hd, rope_dim=hd, rope_base=500000.0, scale=1.0 / np.sqrt(hd), window_left=window)
    for mdl in (gm, om):
        mdl.set_position(ctx)
        mdl.write_buffer(P.BUF_S1, q)
        mdl.write_buffer(P.BUF_S2, k)
        mdl.write_buffer(P.BUF_S3, v)
        mdl.run_step(step)
    got = pkg.bf16_to_f32(gm.read_buffer(P.BUF_S0, heads * hd))
    ref = pkg.bf16_to_f32(om.read_buffer(P.BUF_S0, heads * hd))
    assert rel_err(got, ref).max() <= RTOL
    for b in range(batch):
        for h in range(kvh):
            for which in (0, 1):
                g = pkg.bf16_to_f32(gm.read_kv(which, 0, b, h, ctx + 1)[ctx])
                o = pkg.bf16_to_f32(om.read_kv(which, 0, b, h, ctx + 1)[ctx])
                # the same row quantised on the device and by the oracle: at most one step apart (RoPE in fp32 may
                # differ in the last bit, which can move a value across a rounding boundary)
                step_size = (o.reshape(-1, group).max(-1) - o.reshape(-1, group).min(-1)) / levels
                assert np.all(np.abs(g - o).reshape(-1, group).max(-1) <= 1.5 * step_size + 2.0 ** -7 * np.abs(o).max())
    gm.close()


# ---- rotated KV schemes (rotors + projected K residuals) --------------------------------------------------------------

ROTOR_SCHEMES = {0x70: (8, 32), 0x71: (4, 64)}


@pytest.mark.parametrize("scheme,qjl", [(0x70, 0), (0x71, 0), (0x70, 64), (0x71, 16), (0x71, 64)])
@pytest.mark.parametrize("hd,heads,kvh", [(128, 32, 8), (64, 16, 4)])
@pytest.mark.parametrize("batch,ctx,window", [(1, 0, 0), (1, 65, 0), (1, 1000, 0), (3, 300, 0), (1, 900, 100)])
def test_attention_decode_over_rotated_cache(pkg, store, oracle, hd, heads, kvh, batch, ctx, window, scheme, qjl):
    """Rows turned by the KV head's rotors before they are quantised, q turned likewise, the output turned back, and with
    qjl > 0 the projected K residuals in the scores (Generator/MetalSourceGenerator+Attention.swift:694-930). The cache
    is filled through the probe (turned, quantised and projected on the host by both sides), then three decode steps
    append and attend: outputs, appended rows and their residual rows against the oracle; the default rotors are the
    oracle's (the reference's deterministic rule)."""
    bits, group = ROTOR_SCHEMES[scheme]
    levels = 255.0 if bits == 8 else 15.0
    P = pkg.plan
    desc = pkg.BuffersDesc(hidden=256, slot_dim=heads * hd, vocab=512, max_seq=2048, max_batch=batch, kv_layers=1, kv_heads=kvh,
                           head_dim=hd, conv_layers=0, conv_dim=0, conv_kernel=0, kv_scheme=scheme, kv_qjl_dim=qjl)
    store.add_dense("rotor.embed", _bf(pkg, np.zeros((512, 256))))
    gm = pkg.InferenceModel(store, [P._step(P.STEP_EMBED, out_buf=0, n=256, weight="rotor.embed")], desc)
    om = oracle.model(desc)
    assert np.array_equal(gm.rotors().reshape(-1), om.rotors())
    rng = np.random.default_rng(ctx * 3 + hd + batch + qjl)
    if ctx:
        for b in range(batch):
            for h in range(kvh):
                kr, vr = _bf(pkg, rng.normal(size=(ctx, hd))), _bf(pkg, rng.normal(size=(ctx, hd)))
                for mdl in (gm, om):
                    mdl.write_kv(0, 0, b, h, kr)
                    mdl.write_kv(1, 0, b, h, vr)
        assert np.array_equal(gm.read_kv(0, 0, 0, 0, ctx), om.read_kv(0, 0, 0, 0, ctx))
        if qjl:
            assert np.array_equal(gm.read_qjl(0, batch - 1, kvh - 1, ctx), om.read_qjl(0, batch - 1, kvh - 1, ctx))
    step = P._step(P.STEP_ATTN_DECODE, layer=0, in_buf=P.BUF_S1, in2_buf=P.BUF_S2, in3_buf=P.BUF_S3, out_buf=P.BUF_S0,
                   heads=heads, kv_heads=kvh, head_dim=hd, rope_dim=hd, rope_base=500000.0, scale=1.0 / np.sqrt(hd), window_left=window)
    steps = 3
    for i in range(steps):
        q = _bf(pkg, rng.normal(size=(batch, heads * hd)))
        k = _bf(pkg, np.pad(rng.normal(size=(batch, kvh * hd)), ((0, 0), (0, (heads - kvh) * hd))))
        v = _bf(pkg, np.pad(rng.normal(size=(batch, kvh * hd)), ((0, 0), (0, (heads - kvh) * hd))))
        for mdl in (gm, om):
            mdl.set_position(ctx + i)
            mdl.write_buffer(P.BUF_S1, q)
            mdl.write_buffer(P.BUF_S2, k)
            mdl.write_buffer(P.BUF_S3, v)
            mdl.run_step(step)
        got = pkg.bf16_to_f32(gm.read_buffer(P.BUF_S0, heads * hd))
        ref = pkg.bf16_to_f32(om.read_buffer(P.BUF_S0, heads * hd))
        assert rel_err(got, ref).max() <= RTOL, (i, rel_err(got, ref).max())
    n = ctx + steps
    for b in range(batch):
        for h in range(kvh):
            for which in (0, 1):
                g = pkg.bf16_to_f32(gm.read_kv(which, 0, b, h, n)[ctx:]).reshape(steps, hd)
                o = pkg.bf16_to_f32(om.read_kv(which, 0, b, h, n)[ctx:]).reshape(steps, hd)
                # the rows the device appended, turned back by the probe: a value may sit one quantisation step from the
                # oracle's (RoPE in fp32 differs in the last bit), and the turn spreads a step over the three values of a group
                span = np.abs(o).max() * 2.0 / levels
                assert np.abs(g - o).max() <= 3.0 * span + 2.0 ** -6 * np.abs(o).max()
                assert np.median(np.abs(g - o)) <= 2.0 ** -7 * np.abs(o).max()
            if qjl:
                g = gm.read_qjl(0, b, h, n)[ctx:].view(np.float16).astype(np.float64)
                o = om.read_qjl(0, b, h, n)[ctx:].view(np.float16).astype(np.float64)
                assert np.all(np.isfinite(g))
                assert np.median(np.abs(g - o)) <= 4e-3 * max(np.abs(o).max(), 1e-3)
                assert np.abs(g - o).max() <= 0.5 * max(np.abs(o).max(), 1e-3) + 1e-3
    gm.close()


def test_identity_rotors_give_the_base_scheme(pkg, store, oracle):
    """'Identity rotor preserves vector' (RotorQuantCorrectnessTests:500-518) end to end: with every rotor (1, 0, 0, 0) and
    no residuals the rotated 8-bit scheme computes what the plain 8-bit group-32 scheme computes."""
    P = pkg.plan
    hd, heads, kvh, ctx = 128, 8, 2, 200
    rng = np.random.default_rng(4)
    kr = [[_bf(pkg, rng.normal(size=(ctx, hd))) for _ in range(2)] for _ in range(kvh)]
    q = _bf(pkg, rng.normal(size=(1, heads * hd)))
    k = _bf(pkg, np.pad(rng.normal(size=(1, kvh * hd)), ((0, 0), (0, (heads - kvh) * hd))))
    v = _bf(pkg, np.pad(rng.normal(size=(1, kvh * hd)), ((0, 0), (0, (heads - kvh) * hd))))
    step = P._step(P.STEP_ATTN_DECODE, layer=0, in_buf=P.BUF_S1, in2_buf=P.BUF_S2, in3_buf=P.BUF_S3, out_buf=P.BUF_S0,
                   heads=heads, kv_heads=kvh, head_dim=hd, rope_dim=hd, rope_base=10000.0, scale=1.0 / np.sqrt(hd))
    store.add_dense("rotor.embed", _bf(pkg, np.zeros((512, 256))))
    outs, rows = [], []
    for scheme in (0x70, 0x10):
        desc = pkg.BuffersDesc(hidden=256, slot_dim=heads * hd, vocab=512, max_seq=256, max_batch=1, kv_layers=1, kv_heads=kvh,
                               head_dim=hd, conv_layers=0, conv_dim=0, conv_kernel=0, kv_scheme=scheme)
        gm = pkg.InferenceModel(store, [P._step(P.STEP_EMBED, out_buf=0, n=256, weight="rotor.embed")], desc)
        if scheme == 0x70:
            ident = np.zeros(gm.rotors().shape, dtype=np.float16)
            ident[..., 0] = 1.0
            gm.set_rotors(ident.view(np.uint16))
        for h in range(kvh):
            gm.write_kv(0, 0, 0, h, kr[h][0])
            gm.write_kv(1, 0, 0, h, kr[h][1])
        gm.set_position(ctx)
        gm.write_buffer(P.BUF_S1, q); gm.write_buffer(P.BUF_S2, k); gm.write_buffer(P.BUF_S3, v)
        gm.run_step(step)
        outs.append(pkg.bf16_to_f32(gm.read_buffer(P.BUF_S0, heads * hd)))
        rows.append(gm.read_kv(0, 0, 0, 1, ctx + 1))
        gm.close()
    assert np.array_equal(rows[0], rows[1])
    assert rel_err(outs[0], outs[1]).max() <= 2.0 ** -7
