"""Pins the CPU oracle on the known-answer vectors of the reference's own kernel tests (tests/golden)."""
import base64

import numpy as np
import pytest

from swlm_helpers import pattern_bf16


def _pack(pkg, q_rows):
    return pkg.pack_mlx_q4(np.array(q_rows, dtype=np.uint8))


def _bf(pkg, a):
    return pkg.f32_to_bf16(np.array(a, dtype=np.float32))


def test_gemv_single_block(pkg, oracle, golden):
    g = golden["gemv_single_block"]
    w = _pack(pkg, [g["q"]])
    s, z = _bf(pkg, [[g["scale"]]]), _bf(pkg, [[g["zero"]]])
    # the reference test feeds fp16 activations; these values are exact in bf16 as well
    x = np.array(g["x"], dtype=np.float32)
    assert np.array_equal(pkg.bf16_to_f32(pkg.f32_to_bf16(x)), x)
    blocks = oracle.staf_repack(w, s, z)
    y = oracle.staf_gemv_f32(blocks, 1, 64, x)
    tol = max(g["abs_tol"], g["rel_tol"] * abs(g["expected"]))
    assert abs(float(y[0]) - g["expected"]) < tol
    assert float(y[0]) == pytest.approx(g["expected"], abs=1e-6)  # same fp32 loop, same order
    y_bf16, y64 = oracle.qgemm(pkg.f32_to_bf16(x)[None, :], w, s, z, want_f64=True)
    assert abs(float(pkg.bf16_to_f32(y_bf16)[0, 0]) - g["expected"]) < tol
    assert abs(y64[0, 0] - g["expected"]) < 1e-5


def test_gemv_multi_row_and_staf_end_to_end(pkg, oracle, golden):
    g = golden["gemv_multi_row"]
    w = _pack(pkg, g["q"])
    s, z = _bf(pkg, g["scales"]), _bf(pkg, g["zeros"])
    # scale/zero patterns are exact in bf16 and fp16, so MLX -> STAF narrowing loses nothing here
    assert np.array_equal(pkg.bf16_to_f32(s), np.array(g["scales"], dtype=np.float32))
    x = np.array(g["x"], dtype=np.float32)
    k = 64 * g["blocks"]
    blocks = oracle.staf_repack(w, s, z)
    y = oracle.staf_gemv_f32(blocks, g["rows"], k, x)
    for r in range(g["rows"]):
        tol = max(g["abs_tol"], g["rel_tol"] * abs(g["expected"][r]))
        assert abs(float(y[r]) - g["expected"][r]) < tol
        assert float(y[r]) == pytest.approx(g["expected"][r], abs=2e-6)
    # the MLX-format path and the STAF-block path dequantise to the same weights
    assert np.array_equal(oracle.dequant_mlx(w, s, z), oracle.dequant_staf(blocks, g["rows"], k))


def test_dequant_block_bits(pkg, oracle, golden):
    g = golden["dequant_block"]
    w = _pack(pkg, [g["q"]])
    out = oracle.dequant_bf16(w, _bf(pkg, [[g["scale"]]]), _bf(pkg, [[g["zero"]]]))
    assert out[0].tolist() == g["expected_bf16_bits"]


@pytest.mark.parametrize("case", ["staf_roundtrip_single", "staf_roundtrip_multi"])
def test_staf_repack_is_byte_exact(pkg, oracle, golden, case):
    g = golden[case]
    w = _pack(pkg, g["q"])
    s, z = _bf(pkg, g["scales"]), _bf(pkg, g["zeros"])
    expected = np.array(g["expected_blocks"], dtype=np.uint8).reshape(g["rows"], g["blocks"], 36)
    assert np.array_equal(oracle.staf_repack(w, s, z), expected)
    assert np.array_equal(pkg.formats.repack_mlx_to_staf(w, s, z), expected)  # host-side NumPy converter


@pytest.mark.parametrize("case", ["attention_pattern", "attention_pattern_hd128"])
def test_attention_decode_trace(pkg, oracle, golden, case):
    """Repeated decode over the reference's equivalence-test inputs against an fp64 softmax attention,
    and the K/V cache bytes against the inputs themselves."""
    g = golden[case]
    H, KV, D, T = g["heads"], g["kv_heads"], g["head_dim"], g["seq_len"]
    q = pattern_bf16(T * H * D, *g["q_pattern"]).reshape(T, H * D)
    k = pattern_bf16(T * KV * D, *g["k_pattern"]).reshape(T, KV * D)
    v = pattern_bf16(T * KV * D, *g["v_pattern"]).reshape(T, KV * D)
    expected = np.frombuffer(base64.b64decode(g["expected_f32_b64"]), dtype="<f4").reshape(T, H * D)
    desc = pkg.BuffersDesc(hidden=H * D, slot_dim=H * D, vocab=8, max_seq=g["max_seq"], max_batch=1, kv_layers=1,
                           kv_heads=KV, head_dim=D, conv_layers=0, conv_dim=0, conv_kernel=0)
    m = oracle.model(desc)
    step = pkg.plan._step(pkg.plan.STEP_ATTN_DECODE, layer=0, in_buf=3, in2_buf=4, in3_buf=5, out_buf=2, heads=H,
                          kv_heads=KV, head_dim=D, rope_dim=0, rope_base=0.0, scale=1.0 / np.sqrt(D))
    for t in range(T):
        m.set_position(t)
        m.write_buffer(3, pkg.f32_to_bf16(q[t]))
        m.write_buffer(4, pkg.f32_to_bf16(k[t]))
        m.write_buffer(5, pkg.f32_to_bf16(v[t]))
        m.run_step(step)
        out = pkg.bf16_to_f32(m.read_buffer(2, H * D))[0]
        assert np.max(np.abs(out - expected[t])) < g["tol"] * max(1.0, np.max(np.abs(expected[t])))
    for h in range(KV):
        kc = pkg.bf16_to_f32(m.read_kv(0, 0, 0, h, T))
        vc = pkg.bf16_to_f32(m.read_kv(1, 0, 0, h, T))
        assert np.array_equal(kc, k.reshape(T, KV, D)[:, h])
        assert np.array_equal(vc, v.reshape(T, KV, D)[:, h])


@pytest.mark.parametrize("window", [1, 3, 8, 100])
def test_attention_sliding_window_against_fp64_softmax(pkg, oracle, window):
    """windowLeft (Generator/MetalSourceGenerator+Attention.swift:851-853): position p attends rows
    max(0, p - W + 1) .. p. The reference's tests hold no known answer for it, so the oracle is checked against an
    fp64 softmax over exactly those rows."""
    H, KV, D, T = 4, 2, 64, 12
    rng = np.random.default_rng(window)
    q = pkg.bf16_to_f32(pkg.f32_to_bf16(rng.normal(size=(T, H * D)).astype(np.float32)))
    k = pkg.bf16_to_f32(pkg.f32_to_bf16(rng.normal(size=(T, KV * D)).astype(np.float32)))
    v = pkg.bf16_to_f32(pkg.f32_to_bf16(rng.normal(size=(T, KV * D)).astype(np.float32)))
    desc = pkg.BuffersDesc(hidden=H * D, slot_dim=H * D, vocab=8, max_seq=16, max_batch=1, kv_layers=1,
                           kv_heads=KV, head_dim=D, conv_layers=0, conv_dim=0, conv_kernel=0)
    m = oracle.model(desc)
    step = pkg.plan._step(pkg.plan.STEP_ATTN_DECODE, layer=0, in_buf=3, in2_buf=4, in3_buf=5, out_buf=2, heads=H,
                          kv_heads=KV, head_dim=D, rope_dim=0, rope_base=0.0, scale=1.0 / np.sqrt(D), window_left=window)
    for t in range(T):
        m.set_position(t)
        m.write_buffer(3, pkg.f32_to_bf16(q[t]))
        m.write_buffer(4, pkg.f32_to_bf16(np.pad(k[t], (0, (H - KV) * D))))
        m.write_buffer(5, pkg.f32_to_bf16(np.pad(v[t], (0, (H - KV) * D))))
        m.run_step(step)
        out = pkg.bf16_to_f32(m.read_buffer(2, H * D))[0].reshape(H, D)
        lo = max(0, t - window + 1)
        for h in range(H):
            kh = h * KV // H
            keys = k[lo:t + 1].reshape(-1, KV, D)[:, kh].astype(np.float64)
            vals = v[lo:t + 1].reshape(-1, KV, D)[:, kh].astype(np.float64)
            sc = keys @ q[t].reshape(H, D)[h].astype(np.float64) / np.sqrt(D)
            w = np.exp(sc - sc.max()); w /= w.sum()
            assert np.max(np.abs(out[h] - w @ vals)) < 2e-2


@pytest.mark.parametrize("scheme,bits,group", [(0x10, 8, 32), (0x11, 8, 64), (0x40, 4, 64)])
def test_attention_over_q8_group32_cache_against_fp64(pkg, oracle, scheme, bits, group):
    """8-bit KV rows (36-byte blocks of 32 values, Generator/MetalSourceGenerator+Attention.swift:1923-1956, 2057-2101):
    the rows the oracle appends dequantise to within half a quantisation step of what was written, and attention over
    them equals an fp64 softmax over the DEQUANTISED rows plus the current token's unrounded k and v."""
    H, KV, D, T = 4, 2, 64, 10
    rng = np.random.default_rng(5)
    bf = lambda a: pkg.bf16_to_f32(pkg.f32_to_bf16(np.asarray(a, dtype=np.float32)))
    q, k, v = bf(rng.normal(size=(T, H * D))), bf(rng.normal(size=(T, KV * D))), bf(rng.normal(size=(T, KV * D)))
    desc = pkg.BuffersDesc(hidden=H * D, slot_dim=H * D, vocab=8, max_seq=16, max_batch=1, kv_layers=1, kv_heads=KV, head_dim=D,
                           conv_layers=0, conv_dim=0, conv_kernel=0, kv_scheme=scheme)
    m = oracle.model(desc)
    step = pkg.plan._step(pkg.plan.STEP_ATTN_DECODE, layer=0, in_buf=3, in2_buf=4, in3_buf=5, out_buf=2, heads=H, kv_heads=KV,
                          head_dim=D, rope_dim=0, rope_base=0.0, scale=1.0 / np.sqrt(D))
    for t in range(T):
        m.set_position(t)
        m.write_buffer(3, pkg.f32_to_bf16(q[t]))
        m.write_buffer(4, pkg.f32_to_bf16(np.pad(k[t], (0, (H - KV) * D))))
        m.write_buffer(5, pkg.f32_to_bf16(np.pad(v[t], (0, (H - KV) * D))))
        m.run_step(step)
        out = pkg.bf16_to_f32(m.read_buffer(2, H * D))[0].reshape(H, D)
        for h in range(H):
            kh = h * KV // H
            keys = np.concatenate([pkg.bf16_to_f32(m.read_kv(0, 0, 0, kh, t)).reshape(t, D), k[t].reshape(KV, D)[kh][None]]).astype(np.float64)
            vals = np.concatenate([pkg.bf16_to_f32(m.read_kv(1, 0, 0, kh, t)).reshape(t, D), v[t].reshape(KV, D)[kh][None]]).astype(np.float64)
            sc = keys @ q[t].reshape(H, D)[h].astype(np.float64) / np.sqrt(D)
            w = np.exp(sc - sc.max()); w /= w.sum()
            assert np.max(np.abs(out[h] - w @ vals)) < 2e-2
    # appended rows: within half a step (range / 255 per group of 32) of the inputs, plus the bf16 rounding of the probe
    for h in range(KV):
        got = pkg.bf16_to_f32(m.read_kv(0, 0, 0, h, T)).reshape(T, D)
        want = k.reshape(T, KV, D)[:, h]
        step_size = (want.reshape(T, D // group, group).max(-1) - want.reshape(T, D // group, group).min(-1)) / (255.0 if bits == 8 else 15.0)
        assert np.all(np.abs(got - want).reshape(T, D // group, group).max(-1) <= 0.51 * step_size + 2.0 ** -7 * np.abs(want).max())


def ssm_case(pkg, heads=4, groups=2, dk=16, dv=16, K=4, batch=1, seed=1):
    """Random inputs and weights of one recurrent layer (bf16-exact where the reference reads bf16)."""
    rng = np.random.default_rng(seed)
    conv_dim = 2 * groups * dk + heads * dv
    bf = lambda a: pkg.bf16_to_f32(pkg.f32_to_bf16(np.asarray(a, dtype=np.float32)))
    return dict(heads=heads, groups=groups, dk=dk, dv=dv, K=K, conv_dim=conv_dim, batch=batch,
                conv_w=bf(rng.normal(0.0, 0.5, size=(conv_dim, K))), norm_w=(1.0 + rng.normal(0.0, 0.1, size=dv)).astype(np.float32),
                dt_bias=bf(rng.normal(0.0, 0.5, size=heads)), a_log=rng.normal(0.0, 0.5, size=heads).astype(np.float32),
                rng=rng, bf=bf)


def ssm_reference_f64(c, state, cstate, qkv, z, beta, alpha):
    """fp64 restatement of the gated delta rule step (Generator/MetalSourceGenerator+ConvAndState.swift:392-497) for
    one sequence; updates `state` [H][dk][dv] and `cstate` [K][conv_dim] in place, returns the output [H*dv]."""
    H, G, dk, dv, K = c["heads"], c["groups"], c["dk"], c["dv"], c["K"]
    kgd, hpg = G * dk, H // G
    cstate[:-1] = cstate[1:]
    cstate[-1] = qkv
    s = (cstate * c["conv_w"].T.astype(np.float64)).sum(axis=0)
    act = s / (1.0 + np.exp(-s))
    out = np.zeros(H * dv)
    for h in range(H):
        g = h // hpg
        Q, Kk, V = act[g * dk:(g + 1) * dk], act[kgd + g * dk:kgd + (g + 1) * dk], act[2 * kgd + h * dv:2 * kgd + (h + 1) * dv]
        x = float(alpha[h]) + float(c["dt_bias"][h])
        decay = np.exp(-np.exp(float(c["a_log"][h])) * (max(x, 0.0) + np.log1p(np.exp(-abs(x)))))
        b = 1.0 / (1.0 + np.exp(-float(beta[h])))
        qn = Q / np.sqrt((Q * Q).sum() + 1e-6) / np.sqrt(dk)
        kn = Kk / np.sqrt((Kk * Kk).sum() + 1e-6)
        S = state[h] * decay
        delta = b * (V - kn @ S)
        S = S + np.outer(kn, delta)
        state[h] = S
        o = qn @ S
        o = o / np.sqrt((o * o).mean() + 1e-6) * c["norm_w"]
        zz = z[h * dv:(h + 1) * dv]
        out[h * dv:(h + 1) * dv] = o * zz / (1.0 + np.exp(-zz))
    return out


def ssm_step_and_desc(pkg, c, max_batch=1):
    P = pkg.plan
    width = max(c["conv_dim"], c["heads"] * c["dv"], 256)
    desc = pkg.BuffersDesc(hidden=256, slot_dim=width, vocab=8, max_seq=8, max_batch=max_batch, kv_layers=0, kv_heads=0, head_dim=0,
                           conv_layers=0, conv_dim=0, conv_kernel=0, ssm_layers=1, ssm_heads=c["heads"], ssm_groups=c["groups"],
                           ssm_key_dim=c["dk"], ssm_value_dim=c["dv"], ssm_conv_kernel=c["K"])
    step = P._step(P.STEP_SSM_RECURRENCE, layer=0, in_buf=P.BUF_S1, in2_buf=P.BUF_S2, in3_buf=P.BUF_S3, in4_buf=P.BUF_S4,
                   out_buf=P.BUF_S0, heads=c["heads"], groups=c["groups"], key_dim=c["dk"], value_dim=c["dv"], conv_kernel=c["K"],
                   weight="l0.conv1d.weight", weight2="l0.norm.weight", weight3="l0.dt_bias", weight4="l0.A_log")
    return desc, step, width


def test_ssm_recurrence_against_fp64_gated_delta_rule(pkg, oracle):
    """The reference's tests compare its two SSM kernels with each other and hold no known answer, so the oracle's
    restatement is checked against the textbook form of the recurrence in fp64: S <- decay S + k (x) beta (v - S^T k),
    out = norm(S^T q) * silu(z), over 6 steps with the state carried."""
    c = ssm_case(pkg)
    desc, step, width = ssm_step_and_desc(pkg, c)
    m = oracle.model(desc)
    m.add_dense("l0.conv1d.weight", pkg.f32_to_bf16(c["conv_w"]))
    m.add_dense_f32("l0.norm.weight", c["norm_w"])
    m.add_dense("l0.dt_bias", pkg.f32_to_bf16(c["dt_bias"]))
    m.add_dense_f32("l0.A_log", c["a_log"])
    P = pkg.plan
    state = np.zeros((c["heads"], c["dk"], c["dv"]))
    cstate = np.zeros((c["K"], c["conv_dim"]))
    pad = lambda a: np.pad(a, (0, width - a.size))[None, :]
    for t in range(6):
        qkv, z = c["bf"](c["rng"].normal(size=c["conv_dim"])), c["bf"](c["rng"].normal(size=c["heads"] * c["dv"]))
        beta, alpha = c["bf"](c["rng"].normal(size=c["heads"])), c["bf"](c["rng"].normal(size=c["heads"]))
        for buf, v in ((P.BUF_S1, qkv), (P.BUF_S2, z), (P.BUF_S3, beta), (P.BUF_S4, alpha)):
            m.write_buffer(buf, pkg.f32_to_bf16(pad(v)))
        m.run_step(step)
        got = pkg.bf16_to_f32(m.read_buffer(P.BUF_S0, c["heads"] * c["dv"]))[0]
        ref = ssm_reference_f64(c, state, cstate, qkv.astype(np.float64), z.astype(np.float64), beta, alpha)
        # the kernel rounds the un-normalised output to bf16 before the norm and the result once more
        assert np.max(np.abs(got - ref)) <= 2e-2 * max(1.0, np.max(np.abs(ref))), t
        assert np.max(np.abs(m.read_ssm_state(0, 0) - state)) <= 1e-4 * max(1.0, np.max(np.abs(state)))


def test_conv_decode_trace_matches_sequence_formula_bit_for_bit(pkg, oracle, golden):
    g = golden["conv_pattern"]
    D, K, T = g["dim"], g["kernel"], g["seq_len"]
    x = np.array(g["x"], dtype=np.float32).reshape(T, 3 * D)
    assert np.array_equal(pkg.bf16_to_f32(pkg.f32_to_bf16(x)), x)  # exact in bf16
    desc = pkg.BuffersDesc(hidden=D, slot_dim=3 * D, vocab=8, max_seq=8, max_batch=1, kv_layers=0, kv_heads=0,
                           head_dim=0, conv_layers=1, conv_dim=D, conv_kernel=K)
    m = oracle.model(desc)
    m.add_dense("conv.weight", np.array(g["w_bf16_bits"], dtype=np.uint16))
    step = pkg.plan._step(pkg.plan.STEP_CONV_STATE_UPDATE, layer=0, in_buf=3, out_buf=2, n=D, conv_kernel=K, weight="conv.weight")
    out_bits = []
    for t in range(T):
        m.write_buffer(3, pkg.f32_to_bf16(x[t]))
        m.run_step(step)
        out_bits += m.read_buffer(2, D)[0].tolist()
    assert out_bits == g["expected_out_bf16_bits"]
    assert m.read_conv(0, 0).tolist() == g["expected_state_bf16_bits"]


def test_bf16_rounding_rule(pkg, oracle):
    rng = np.random.default_rng(0)
    x = rng.normal(size=4096).astype(np.float32)
    x[:4] = [1.00390625, 1.01171875, -1.00390625, 3.0e-40]  # ties to even, and a subnormal
    ours = pkg.f32_to_bf16(x)
    for v, b in zip(x[:64], ours[:64]):
        assert oracle.dll.orc_f32_to_bf16(__import__("ctypes").c_float(float(v))) == int(b)
    assert pkg.bf16_to_f32(ours[:2]).tolist() == [1.0, 1.015625]


def test_rope_matches_closed_form(pkg, oracle):
    hd, pos, base = 128, 777, 500000.0
    rng = np.random.default_rng(1)
    v = pkg.bf16_to_f32(pkg.f32_to_bf16(rng.normal(size=hd).astype(np.float32)))
    got = pkg.bf16_to_f32(oracle.rope_bf16(pkg.f32_to_bf16(v), 1, hd, hd, base, pos))
    i = np.arange(hd // 2)
    theta = pos * base ** (-2.0 * i / hd)
    want = np.concatenate([v[: hd // 2] * np.cos(theta) - v[hd // 2:] * np.sin(theta),
                           v[: hd // 2] * np.sin(theta) + v[hd // 2:] * np.cos(theta)])
    assert np.max(np.abs(got - want)) < 2e-2
