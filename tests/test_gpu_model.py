"""End-to-end parity of the CUDA dispatch plan against the oracle interpreting the same plan.

Acceptance: greedy tokens identical over 64 decode steps after a prompt. Logits are also compared, at 4e-2
relative error: every kernel is held to 1e-2 on its own (tests/test_gpu_kernels.py), but through a stack of
layers each differently-ordered fp32 sum flips some bf16 roundings by one ulp and those flips compound, most
in the gated conv layers where three rounded factors are multiplied.
When a token differs the test reports the oracle's top-1/top-2 logit margin at that step: with bf16 logits a
margin of zero or one bf16 ulp is a tie that summation order may legitimately break either way; any larger
margin is a failure.
"""
import numpy as np
import pytest

from swlm_helpers import rel_err

pytestmark = pytest.mark.gpu


def small_llama(pkg, batch=1, max_seq=128):
    return pkg.ModelConfig("llama", hidden=512, intermediate=1536, layers=4, heads=8, kv_heads=2, head_dim=64,
                           vocab=4096, norm_eps=1e-5, rope_theta=500000.0, max_seq=max_seq, max_batch=batch)


def small_lfm2(pkg, batch=1, max_seq=128):
    return pkg.ModelConfig("lfm2", hidden=512, intermediate=1024, layers=5, heads=8, kv_heads=2, head_dim=64,
                           vocab=4096, norm_eps=1e-5, rope_theta=1000000.0, conv_kernel=3, attention_layers=[1, 3],
                           max_seq=max_seq, max_batch=batch)


def build_pair(pkg, oracle, cfg, seed=3, centered=False):
    builder = pkg.DispatchPlanBuilder(cfg)
    weights = pkg.synth_model_weights(builder, seed=seed, centered=centered)
    store = pkg.WeightStore(0)
    gm = pkg.load_model(store, builder, weights)
    om = oracle.model(cfg.buffers_desc())
    om.load(builder, weights)
    oracle.set_threads(0)
    return store, gm, om


def greedy_compare(pkg, gm, om, cfg, prompt_len, steps):
    rng = np.random.default_rng(11)
    prompt = rng.integers(0, cfg.vocab, size=(cfg.max_batch, prompt_len), dtype=np.int32)
    g_tok = gm.prefill(prompt)
    o_tok = om.prefill(prompt)
    mismatches = []
    for step in range(steps + 1):
        logits_g = pkg.bf16_to_f32(gm.logits())
        logits_o = pkg.bf16_to_f32(om.read_buffer(pkg.plan.BUF_LOGITS, cfg.vocab))
        err = rel_err(logits_g, logits_o).max()
        assert err <= 4e-2, f"step {step}: logits rel-err {err}"
        for b in range(cfg.max_batch):
            if g_tok[b] != o_tok[b]:
                top2 = np.sort(logits_o[b])[-2:]
                ulp = 2.0 ** (np.floor(np.log2(max(abs(top2[1]), 1e-30))) - 7)
                mismatches.append((step, b, int(g_tok[b]), int(o_tok[b]), float(top2[1] - top2[0]), float(ulp)))
        if step == steps:
            break
        # feed the oracle's token to both so that one tie does not fork the two traces
        g_tok = gm.decode(o_tok)
        o_tok = om.decode(o_tok)
    assert gm.position == om.position == prompt_len + steps
    for step, b, gt, ot, margin, ulp in mismatches:
        assert margin <= ulp, f"step {step} seq {b}: token {gt} != {ot} with top-1/top-2 margin {margin} (bf16 ulp {ulp})"
    return mismatches


@pytest.mark.parametrize("batch", [1, 4])
def test_llama_shape_greedy_64_steps(pkg, oracle, batch):
    cfg = small_llama(pkg, batch=batch)
    store, gm, om = build_pair(pkg, oracle, cfg)
    mism = greedy_compare(pkg, gm, om, cfg, prompt_len=12, steps=64)
    assert len(mism) <= 2, mism
    gm.close(); store.close()


@pytest.mark.parametrize("batch", [1, 3])
def test_lfm2_shape_greedy_64_steps(pkg, oracle, batch):
    cfg = small_lfm2(pkg, batch=batch)
    store, gm, om = build_pair(pkg, oracle, cfg)
    mism = greedy_compare(pkg, gm, om, cfg, prompt_len=10, steps=64)
    assert len(mism) <= 2, mism
    # conv state and KV cache bytes agree with the oracle's after 74 positions
    for layer in range(cfg.conv_layer_count):
        for b in range(batch):
            g, o = pkg.bf16_to_f32(gm.read_conv(layer, b)), pkg.bf16_to_f32(om.read_conv(layer, b))
            assert rel_err(g, o).max() <= 1e-2
    gm.close(); store.close()


@pytest.mark.parametrize("family", ["llama", "lfm2"])
def test_chunked_prompt_ingestion_matches_oracle_and_token_by_token(pkg, oracle, family):
    """A 100-token prompt goes through the chunked path (tensor-core products, rope + append for the whole chunk,
    causal attention over the cache, the conv recurrence walked inside one kernel): chunks of 64 and 35 tokens,
    the last token through the decode graph. The oracle ingests token by token. Tokens must agree over the
    following decode steps, and the KV cache / conv state of both ingestion modes must agree with the oracle's
    (the chunked products round the dequantised weights to bf16, as the reference's dequantise-then-matmul
    prefill route does)."""
    cfg = (small_llama if family == "llama" else small_lfm2)(pkg, batch=1, max_seq=256)
    store, gm, om = build_pair(pkg, oracle, cfg)
    gm.set_prefill_chunk(64)
    before = gm.launches
    mism = greedy_compare(pkg, gm, om, cfg, prompt_len=100, steps=24)
    assert len(mism) <= 2, mism
    # far fewer launches than 100 decode steps: the prompt really went through the chunked path
    assert gm.launches - before < 40 * gm.launches_per_step
    keys = [(w, layer, h) for w in (0, 1) for layer in range(cfg.kv_layer_count) for h in range(cfg.kv_heads)]
    kv_oracle = {k: pkg.bf16_to_f32(om.read_kv(k[0], k[1], 0, k[2], 100)) for k in keys}
    kv_chunked = {k: pkg.bf16_to_f32(gm.read_kv(k[0], k[1], 0, k[2], 100)) for k in keys}
    conv_oracle = [pkg.bf16_to_f32(om.read_conv(layer, 0)) for layer in range(cfg.conv_layer_count)]
    conv_chunked = [pkg.bf16_to_f32(gm.read_conv(layer, 0)) for layer in range(cfg.conv_layer_count)]
    # the same prompt, one token at a time
    gm.reset_state()
    gm.set_prefill_chunk(0)
    rng = np.random.default_rng(11)
    prompt = rng.integers(0, cfg.vocab, size=(1, 100), dtype=np.int32)
    gm.prefill(prompt)
    kv_single = {k: pkg.bf16_to_f32(gm.read_kv(k[0], k[1], 0, k[2], 100)) for k in keys}
    # Cache rows of the prompt against the oracle's, per (K/V, layer, head). With these synthetic weights (rows
    # with a large common mean) a V row is close to mean(W) * sum(x), a cancellation-prone sum: a few rows (the
    # first token behind a conv layer with empty history, for one) amplify rounding noise a hundredfold in either
    # ingestion mode, and the bf16 rounding of the weights in the chunked products is ten times the noise of a
    # reordered fp32 sum. Hence: typical rows tight, the whole cache in the L2 norm, only a few loose rows.
    for k in keys:
        ref = kv_oracle[k]
        for name, got, l2_tol in (("chunked", kv_chunked[k], 6e-2), ("token by token", kv_single[k], 2e-2)):
            row_err = np.linalg.norm(got - ref, axis=1) / np.maximum(np.linalg.norm(ref, axis=1), 1e-6)
            what = f"{name} ingestion, cache {k}: worst row {int(row_err.argmax())} rel L2 {row_err.max():.4f}"
            assert np.median(row_err) <= 1e-2, what
            assert int((row_err > 5e-2).sum()) <= 4, what
            assert np.linalg.norm(got - ref) <= l2_tol * np.linalg.norm(ref), what
    for got, ref in zip(conv_chunked, conv_oracle):
        assert np.linalg.norm(got - ref) <= 3e-2 * np.linalg.norm(ref)
    gm.close(); store.close()


@pytest.mark.parametrize("family", ["llama", "lfm2"])
def test_chunked_and_token_by_token_ingestion_fill_the_same_cache(pkg, oracle, family):
    """The reference's sequence-equivalence property (Tests/MetalCompilerTests/Core/AttentionSequenceEquivalenceTests
    .swift:21-43, Conv1dSequenceEquivalenceTests.swift:21-30: a prompt ingested as a sequence leaves the caches a
    token-by-token ingestion leaves), for this library's two ingestion paths. They cannot be equal bit for bit here:
    the two kinds of product add their fp32 terms in different orders, which flips the bf16 rounding of an element
    here and there (one bf16 ulp is 0.4-0.8 % of the element, and the flips compound through the layers), and a
    chunk reads its newest K/V row back from the cache (rounded) where a decode step uses it unrounded. So the
    property is asserted per cache row, for EVERY row: relative L2 distance at most 4e-2 (median at most 2e-2)
    between any two of chunked ingestion, token-by-token ingestion and the oracle, on zero-mean weights (with the
    benchmark distribution's common mean every V row is a small difference of large sums and amplifies any rounding
    a hundredfold; that case is the test above). The conv recurrence is walked in order inside one kernel and its
    state must agree likewise."""
    cfg = (small_llama if family == "llama" else small_lfm2)(pkg, batch=1, max_seq=256)
    store, gm, om = build_pair(pkg, oracle, cfg, centered=True)
    prompt = np.random.default_rng(5).integers(0, cfg.vocab, size=(1, 150), dtype=np.int32)
    keys = [(w, layer, h) for w in (0, 1) for layer in range(cfg.kv_layer_count) for h in range(cfg.kv_heads)]
    caches = {}
    for mode, chunk in (("chunked", 64), ("single", 0)):
        gm.reset_state()
        gm.set_prefill_chunk(chunk)
        before = gm.launches
        first = gm.prefill(prompt)
        if chunk:
            assert gm.launches - before < 60 * gm.launches_per_step   # really the chunked path
        caches[mode] = ({k: pkg.bf16_to_f32(gm.read_kv(k[0], k[1], 0, k[2], 150)) for k in keys},
                        [pkg.bf16_to_f32(gm.read_conv(layer, 0)) for layer in range(cfg.conv_layer_count)], first)
    o_first = om.prefill(prompt)
    kv_oracle = {k: pkg.bf16_to_f32(om.read_kv(k[0], k[1], 0, k[2], 150)) for k in keys}
    worst = 0.0
    for k in keys:
        a, b, ref = caches["chunked"][0][k], caches["single"][0][k], kv_oracle[k]
        for name, got, want in (("chunked vs token by token", a, b), ("chunked vs oracle", a, ref), ("token by token vs oracle", b, ref)):
            row_err = np.linalg.norm(got - want, axis=1) / np.maximum(np.linalg.norm(want, axis=1), 1e-6)
            worst = max(worst, float(row_err.max()))
            assert row_err.max() <= 4e-2, f"{name}, cache {k}: row {int(row_err.argmax())} rel L2 {row_err.max():.4f}"
            assert np.median(row_err) <= 2e-2, f"{name}, cache {k}: median {np.median(row_err):.4f}"
    for a, b in zip(caches["chunked"][1], caches["single"][1]):
        assert np.linalg.norm(a - b) <= 3e-2 * np.linalg.norm(b)
    assert caches["chunked"][2].tolist() == caches["single"][2].tolist() == o_first.tolist()
    print(f"worst cache-row deviation between any two ingestion paths: {worst:.5f}")
    gm.close(); store.close()


def test_chunked_prompt_ingestion_head_dim_128_over_several_key_tiles(pkg, oracle):
    """Head dimension 128, one KV head for four query heads, a 200-token prompt in chunks of 128 and 71: the tiled
    causal attention walks up to four 64-row key tiles, the second chunk starts at a position that is not zero."""
    cfg = pkg.ModelConfig("llama", hidden=512, intermediate=1536, layers=2, heads=4, kv_heads=1, head_dim=128,
                          vocab=4096, norm_eps=1e-5, rope_theta=500000.0, max_seq=256, max_batch=1)
    store, gm, om = build_pair(pkg, oracle, cfg)
    gm.set_prefill_chunk(128)
    before = gm.launches
    mism = greedy_compare(pkg, gm, om, cfg, prompt_len=200, steps=16)
    assert len(mism) <= 2, mism
    assert gm.launches - before < 60 * gm.launches_per_step
    for which in (0, 1):
        for layer in range(cfg.kv_layer_count):
            ref = pkg.bf16_to_f32(om.read_kv(which, layer, 0, 0, 200))
            got = pkg.bf16_to_f32(gm.read_kv(which, layer, 0, 0, 200))
            row_err = np.linalg.norm(got - ref, axis=1) / np.maximum(np.linalg.norm(ref, axis=1), 1e-6)
            what = f"cache {which} layer {layer}: worst row {int(row_err.argmax())} rel L2 {row_err.max():.4f}"
            assert np.median(row_err) <= 1e-2, what
            assert int((row_err > 5e-2).sum()) <= 4, what
            assert np.linalg.norm(got - ref) <= 6e-2 * np.linalg.norm(ref), what
    gm.close(); store.close()


def test_objects_may_be_destroyed_in_any_order(pkg, oracle):
    """Wrappers with garbage collection release context, plan and state in no particular order; a context
    destroyed first must stay valid until its plan and state are gone, and leave no CUDA error behind."""
    cfg = small_llama(pkg)
    store, gm, om = build_pair(pkg, oracle, cfg)
    first = gm.prefill(np.arange(1, 6, dtype=np.int32)[None, :])
    store.close()                      # context first: deferred
    tok = gm.decode(first)             # the state still works
    assert tok.shape == (1,)
    gm.close()                         # the last user takes the plan and the context with it
    store2, gm2, _ = build_pair(pkg, oracle, cfg)   # uploads run the stale-error check
    assert gm2.prefill(np.arange(1, 6, dtype=np.int32)[None, :]).tolist() == first.tolist()
    gm2.close(); store2.close()


def test_plan_fuses_launches(pkg, oracle):
    cfg = small_llama(pkg)
    store, gm, om = build_pair(pkg, oracle, cfg)
    text = gm.describe()
    # per layer: norm + fused qkv, attention, o, norm + fused gate/up + swiglu, down; then norm + lm_head, argmax x2
    assert text.count("qgemv+swiglu") == cfg.layers
    assert text.count("rmsnorm+") == 2 * cfg.layers + 1
    assert sum("self_attn.q_proj" in l and "self_attn.v_proj" in l for l in text.splitlines()) == cfg.layers
    assert gm.launches_per_step == 1 + cfg.layers * 5 + 1 + 2
    before = gm.launches
    gm.decode([1])
    assert gm.launches - before == gm.launches_per_step
    gm.close(); store.close()


def test_decode_n_equals_repeated_decode_and_snapshot_restore(pkg, oracle):
    cfg = small_llama(pkg)
    store, gm, om = build_pair(pkg, oracle, cfg)
    prompt = np.arange(1, 9, dtype=np.int32)[None, :]
    first = gm.prefill(prompt)
    snap = gm.prompt_snapshot()
    a = gm.decode_n(first, 20)[:, 0]
    assert gm.position == 28
    gm.restore(snap)
    assert gm.position == 8
    tok, b = first, []
    for _ in range(20):
        tok = gm.decode(tok)
        b.append(int(tok[0]))
    assert a.tolist() == b
    # a second state restored from scratch reproduces the same trace (prefill -> decode uses the KV from prefill)
    gm.reset_state()
    assert gm.position == 0
    assert gm.prefill(prompt).tolist() == first.tolist()
    assert gm.decode_n(first, 20)[:, 0].tolist() == b
    gm.free_snapshot(snap)
    gm.close(); store.close()


def test_zeroed_kv_changes_logits(pkg, oracle):
    # Tests/MetalCompilerTests/Core/DecodeTests.swift:13-137 — decode after prefill must depend on the cache
    cfg = small_llama(pkg)
    store, gm, om = build_pair(pkg, oracle, cfg)
    prompt = np.arange(5, 25, dtype=np.int32)[None, :]
    first = gm.prefill(prompt)
    snap = gm.prompt_snapshot()
    gm.decode(first)
    ref = gm.logits().copy()
    gm.restore(snap)
    zero = np.zeros((20, cfg.head_dim), dtype=np.uint16)
    for layer in range(cfg.kv_layer_count):
        for h in range(cfg.kv_heads):
            gm.write_kv(0, layer, 0, h, zero)
            gm.write_kv(1, layer, 0, h, zero)
    gm.decode(first)
    assert not np.array_equal(gm.logits(), ref)
    gm.free_snapshot(snap)
    gm.close(); store.close()


def test_errors_surface_as_status(pkg, oracle):
    cfg = small_llama(pkg, max_seq=16)
    store, gm, om = build_pair(pkg, oracle, cfg)
    with pytest.raises(pkg.SwlmError):
        gm.prefill(np.zeros((1, 17), dtype=np.int32))  # longer than the KV cache
    bad = pkg.DispatchPlanBuilder(cfg).decode_steps()
    bad[3].weight = b"model.layers.0.self_attn.missing"
    with pytest.raises(pkg.SwlmError) as e:
        pkg.InferenceModel(store, bad, cfg.buffers_desc())
    assert e.value.status == -3
    gm.close(); store.close()


@pytest.mark.parametrize("batch", [1, 3])
def test_gemma_style_variants_geglu_and_norm_weight_bias(pkg, oracle, batch):
    """The same recipe with the GELU-gated MLP (GEGLU) and weightBias = 1 on every RMSNorm
    (Generator/MetalSourceGenerator+NormAndElementwise.swift:160-208): fused epilogue and fused norm prologue at
    batch 1, the batched kernels at batch 3, and the unfused steps inside a prompt chunk."""
    cfg = small_llama(pkg, batch=batch, max_seq=160)
    cfg.activation = "gelu_tanh"
    cfg.norm_weight_bias = 1.0
    store, gm, om = build_pair(pkg, oracle, cfg)
    assert "geglu" in gm.describe() and "swiglu" not in gm.describe()
    mism = greedy_compare(pkg, gm, om, cfg, prompt_len=8, steps=32)
    assert len(mism) <= 2, mism
    if batch == 1:
        gm.reset_state(); om.reset()
        gm.set_prefill_chunk(64)
        mism = greedy_compare(pkg, gm, om, cfg, prompt_len=90, steps=8)
        assert len(mism) <= 1, mism
    gm.close(); store.close()


def test_model_loaded_from_a_staf_file(pkg, oracle, tmp_path):
    """A synthetic model written as an MLX-shaped safetensors bundle, converted to a STAF file and loaded from that file:
    the weights enter as interleaved fp16-scale blocks (the reference's execution format), so the oracle takes its
    scales and zeros through fp16 as well; tokens and logits must agree as for any other model."""
    import os

    cfg = small_llama(pkg, batch=1)
    builder = pkg.DispatchPlanBuilder(cfg)
    weights = pkg.synth_model_weights(builder, seed=9)
    src = os.path.join(tmp_path, "model.safetensors")
    pkg.staf.write_safetensors(src, pkg.bundle_tensors(builder, weights))
    out = os.path.join(tmp_path, "model.staf")
    assert pkg.staf.convert_safetensors([src], out) and pkg.staf.is_valid(out, [src], pkg.staf.default_cache_metadata(1))
    store = pkg.WeightStore(0)
    gm = pkg.load_model_from_staf(store, builder, pkg.staf.read_staf(out))
    # the oracle narrows scales and zeros through fp16 exactly as the STAF blocks carry them
    om = oracle.model(cfg.buffers_desc())
    om.load(builder, weights, staf_fp16=True)
    oracle.set_threads(0)
    mism = greedy_compare(pkg, gm, om, cfg, prompt_len=9, steps=32)
    assert len(mism) <= 2, mism
    gm.close(); store.close()


def test_lfm2_tied_q4_embedding_table(pkg, oracle):
    """A tied output head (Sources/Models/LlamaFamilyNaming.swift:22-27): one Q4 group-64 tensor is both the embedding
    table (embedding_lookup_q4, Generator/MetalSourceGenerator+Embedding.swift:79-154) and the lm_head weight. Token by
    token and through a prompt chunk."""
    cfg = small_lfm2(pkg, batch=2, max_seq=160)
    cfg.tie_embeddings = True
    store, gm, om = build_pair(pkg, oracle, cfg)
    assert "lm_head" not in gm.describe() and "model.embed_tokens.weight" in gm.describe()
    mism = greedy_compare(pkg, gm, om, cfg, prompt_len=7, steps=24)
    assert len(mism) <= 2, mism
    gm.close(); store.close()
    cfg1 = small_lfm2(pkg, batch=1, max_seq=160)
    cfg1.tie_embeddings = True
    store, gm, om = build_pair(pkg, oracle, cfg1)
    gm.set_prefill_chunk(64)
    mism = greedy_compare(pkg, gm, om, cfg1, prompt_len=90, steps=8)
    assert len(mism) <= 1, mism
    gm.close(); store.close()


def test_full_size_lfm2_like_shape_against_oracle(pkg, oracle):
    """The hybrid benchmark shape (16 layers: 10 gated short-conv + 6 attention with QK norm, hidden 2048, FFN 8192,
    vocab 65536, tied Q4 head): a short prompt and 16 greedy steps against the oracle, logits parity at every step."""
    cfg = pkg.lfm2_like_config(max_seq=48)
    store, gm, om = build_pair(pkg, oracle, cfg)
    mism = greedy_compare(pkg, gm, om, cfg, prompt_len=4, steps=16)
    assert len(mism) <= 1, mism
    gm.close(); store.close()


def test_full_size_llama3_8b_shape_against_oracle(pkg, oracle):
    """The benchmark's model shape (32 layers, hidden 4096, FFN 14336, vocab 128256): a short prompt and 64 greedy
    steps against the oracle on all host cores (the oracle's token is fed to both sides), with logits parity at the
    full vocabulary width at every step."""
    cfg = pkg.llama3_8b_config(max_seq=80)
    store, gm, om = build_pair(pkg, oracle, cfg)
    assert store.resident_bytes > 4_221_370_368
    mism = greedy_compare(pkg, gm, om, cfg, prompt_len=3, steps=64)
    assert len(mism) <= 2, mism
    gm.close(); store.close()
