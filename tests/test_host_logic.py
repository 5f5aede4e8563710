"""CPU-only checks: format helpers, sizing contracts, plan builder shape, and that the C-ABI library loads
and exports every symbol include/swlm.h declares (no compute calls without a GPU)."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_pack_unpack_roundtrip(pkg):
    rng = np.random.default_rng(0)
    q = rng.integers(0, 16, size=(5, 192), dtype=np.uint8)
    w = pkg.pack_mlx_q4(q)
    assert w.shape == (5, 24) and w.dtype == np.uint32
    assert np.array_equal(pkg.formats.unpack_mlx_q4(w, 192), q)
    # element j of a row is nibble j%8 of word j/8, i.e. byte j/2, low nibble for even j
    raw = w.view(np.uint8).reshape(5, 96)
    assert np.array_equal(raw & 0xF, q[:, 0::2]) and np.array_equal(raw >> 4, q[:, 1::2])


def test_staf_block_geometry(pkg):
    fmt = pkg.AffineQ4Group64Format
    # Tests/MetalCompilerTests/Core/SupportedQuantizationsContractTests.swift:95-113 (block geometry)
    assert (fmt.bits, fmt.group_size, fmt.weights_per_block, fmt.bytes_per_block) == (4, 64, 64, 36)
    assert fmt.bytes_per_block == 4 + fmt.weights_per_block * fmt.bits // 8
    assert fmt.bytes_per_weight() == 0.5625


def test_kv_cache_sizing_contract(pkg):
    # Tests/MetalCompilerTests/Core/KVCacheSizingContractTests.swift:32-53, 129-185
    spec = pkg.KVCacheSpecification(layer_count=32, kv_head_count=8, head_dimension=128, maximum_sequence_length=4224)
    assert spec.bytes_per_head_slot() == 256
    assert spec.bytes_per_token_slot() == 8 * 256
    assert spec.bytes_per_layer() % spec.bytes_per_head_slot() == 0
    assert spec.total_bytes() == 553_648_128
    small = pkg.KVCacheSpecification(layer_count=6, kv_head_count=8, head_dimension=64, maximum_sequence_length=16)
    assert small.bytes_per_head_slot() == 256  # 128 bytes of data aligned up to the 256-byte dense slot
    assert small.sequence_major_offset(1, 2, 3) == 1 * 8 * 16 * 256 + 2 * 16 * 256 + 3 * 256


def test_kv_cache_sizing_of_block_and_rotated_schemes(pkg):
    # Tests/MetalCompilerTests/Core/KVCacheSizingContractTests.swift:32-80, 100-125 (rotated schemes size like their base);
    # Tests/MetalCompilerTests/Models/RotorQuant/RotorQuantCorrectnessTests.swift:52-67, 163-202
    def spec(scheme, hd=128, layers=16, seq=4096):
        return pkg.KVCacheSpecification(layer_count=layers, kv_head_count=8, head_dimension=hd, maximum_sequence_length=seq, scheme=scheme)
    assert spec(0x00).bytes_per_head_slot() == 256 and spec(0x01, hd=192).bytes_per_head_slot() == 512 and spec(0x02).bytes_per_head_slot() == 512
    assert spec(0x10).bytes_per_head_slot() == 192     # 4 blocks x 36 = 144 -> 64-byte slots
    assert spec(0x11).bytes_per_head_slot() == 192     # 2 x 68 = 136
    assert spec(0x40).bytes_per_head_slot() == 128     # 2 x 36 = 72
    assert spec(0x42).bytes_per_head_slot() == 128     # 1 x 68
    assert spec(0x70).bytes_per_head_slot() == spec(0x10).bytes_per_head_slot() and spec(0x71).bytes_per_head_slot() == spec(0x40).bytes_per_head_slot()
    assert spec(0x70).uses_rotor_quant and spec(0x71).uses_rotor_quant and not spec(0x10).uses_rotor_quant and not spec(0x01).uses_rotor_quant
    assert [spec(0x70, hd=h).num_rotor_groups() for h in (3, 4, 6, 64, 128, 1)] == [1, 2, 2, 22, 43, 1]
    r = spec(0x70)
    assert r.rotor_parameters_bytes_per_layer() == 8 * 43 * 4 * 2 and r.total_rotor_parameters_size() == 8 * 43 * 4 * 2 * 16
    assert r.qjl_matrix_size(16) == 128 * 16 * 2
    assert r.qjl_residual_bytes_per_layer(16) == 4096 * 8 * 16 * 2 and r.total_qjl_residual_size(16) == 4096 * 8 * 16 * 2 * 16
    assert r.qjl_matrix_size(0) == 0 and r.qjl_residual_bytes_per_layer(0) == 0 and r.total_qjl_residual_size(0) == 0
    # the C header's helpers agree on the unpadded rows this build stores (144 / 72 bytes for head_dim 128)
    desc = pkg.ModelConfig(family="llama", hidden=256, intermediate=512, layers=2, heads=4, kv_heads=2, head_dim=128, vocab=512,
                           max_seq=64, kv_scheme=0x71, kv_qjl_dim=16).buffers_desc()
    assert desc.kv_scheme == 0x71 and desc.kv_qjl_dim == 16


def test_llama_plan_shape(pkg):
    cfg = pkg.llama3_8b_config()
    b = pkg.DispatchPlanBuilder(cfg)
    steps = b.decode_steps()
    kinds = [s.kind for s in steps]
    P = pkg.plan
    # embed + 32 x (norm, q, k, v, attn, o, norm, gate, up, swiglu, down) + final norm + lm_head + argmax
    assert len(steps) == 1 + 32 * 11 + 3
    assert kinds[0] == P.STEP_EMBED and kinds[1] == P.STEP_COPY_RMSNORM
    assert kinds.count(P.STEP_QGEMV) == 32 * 7 + 1
    assert kinds.count(P.STEP_RESADD_COPY_RMSNORM) == 63 and kinds[-3:] == [P.STEP_RESADD_RMSNORM, P.STEP_QGEMV, P.STEP_ARGMAX]
    assert cfg.slot_dim == 16384
    assert cfg.q4_weight_elems() == 7_504_658_432
    assert int(cfg.q4_weight_elems() * 0.5625) == 4_221_370_368
    # the step count does not depend on the token count (Tests/MetalCompilerTests/Core/PrefillTests.swift:49-71)
    assert len(pkg.DispatchPlanBuilder(pkg.llama3_8b_config(max_seq=128)).decode_steps()) == len(steps)
    names = {t[0] for t in b.tensors()}
    for s in steps:
        if s.weight:
            assert s.weight.decode() in names


def test_lfm2_plan_shape(pkg):
    cfg = pkg.lfm2_like_config()
    b = pkg.DispatchPlanBuilder(cfg)
    steps = b.decode_steps()
    P = pkg.plan
    kinds = [s.kind for s in steps]
    assert cfg.kv_layer_count == 6 and cfg.conv_layer_count == 10
    assert kinds.count(P.STEP_CONV_STATE_UPDATE) == 10 and kinds.count(P.STEP_ATTN_DECODE) == 6
    assert kinds.count(P.STEP_QK_NORM) == 6
    conv_layers = [s.layer for s in steps if s.kind == P.STEP_CONV_STATE_UPDATE]
    assert conv_layers == list(range(10))
    assert cfg.q4_weight_elems() == 16 * 50_331_648 + 10 * 16_777_216 + 6 * 10_485_760 + 134_217_728


def test_deltanet_plan_shape_windows_and_cache_scheme(pkg):
    """The hybrid recurrent recipe: per recurrent layer four projections of one input, the recurrence step with its
    four buffers and four tensors, the out projection; every name the steps use is in the tensor inventory with the
    right kind; sliding windows and the cache scheme travel through the plan and the buffer description."""
    import dataclasses
    P = pkg.plan
    cfg = pkg.ModelConfig("deltanet", hidden=256, intermediate=512, layers=6, heads=4, kv_heads=2, head_dim=64, vocab=1024,
                          attention_layers=[2, 5], max_seq=64, ssm_heads=8, ssm_groups=4, ssm_key_dim=32, ssm_value_dim=64,
                          ssm_conv_kernel=4, sliding_window=16, sliding_window_layers=[5], kv_scheme=0x11)
    b = pkg.DispatchPlanBuilder(cfg)
    steps = b.decode_steps()
    kinds = [s.kind for s in steps]
    assert cfg.ssm_layer_count == 4 and cfg.kv_layer_count == 2 and cfg.conv_layer_count == 0
    assert cfg.ssm_conv_dim == 2 * 4 * 32 + 8 * 64 and cfg.slot_dim >= cfg.ssm_conv_dim
    assert kinds.count(P.STEP_SSM_RECURRENCE) == 4 and kinds.count(P.STEP_ATTN_DECODE) == 2
    assert kinds.count(P.STEP_QGEMV) == 4 * 5 + 2 * 4 + 6 * 3 + 1
    rec = [s for s in steps if s.kind == P.STEP_SSM_RECURRENCE]
    assert [s.layer for s in rec] == [0, 1, 2, 3]
    r0 = rec[0]
    assert (r0.in_buf, r0.in2_buf, r0.in3_buf, r0.in4_buf, r0.out_buf) == (P.BUF_S1, P.BUF_S2, P.BUF_S3, P.BUF_S4, P.BUF_S0)
    assert (r0.heads, r0.groups, r0.key_dim, r0.value_dim, r0.conv_kernel) == (8, 4, 32, 64, 4)
    assert r0.weight.decode().endswith("linear_attn.conv1d.weight") and r0.weight4.decode().endswith("linear_attn.A_log")
    kinds_by_name = {t[0]: t[1] for t in b.tensors()}
    assert kinds_by_name[r0.weight2.decode()] == "f32" and kinds_by_name[r0.weight4.decode()] == "f32"
    assert kinds_by_name[r0.weight.decode()] == "conv" and kinds_by_name[r0.weight3.decode()] == "dense"
    for s in steps:
        for w in (s.weight, s.weight2, s.weight3, s.weight4):
            if w:
                assert w.decode() in kinds_by_name
    att = [s for s in steps if s.kind == P.STEP_ATTN_DECODE]
    assert [s.window_left for s in att] == [0, 16]                 # only model layer 5 is windowed
    d = cfg.buffers_desc()
    assert (d.ssm_layers, d.ssm_heads, d.ssm_groups, d.ssm_key_dim, d.ssm_value_dim, d.ssm_conv_kernel, d.kv_scheme) == (4, 8, 4, 32, 64, 4, 0x11)
    plain = dataclasses.replace(cfg, family="llama", attention_layers=[]).buffers_desc()
    assert plain.ssm_layers == 0 and plain.ssm_heads == 0
    w = pkg.synth_model_weights(b, seed=1)
    assert w[r0.weight2.decode()].dtype == np.float32 and w[r0.weight3.decode()].dtype == np.uint16
    assert abs(float(w[r0.weight4.decode()].min())) <= 1.0


def test_synth_distributions(pkg):
    w, s, b = pkg.synth_q4(64, 4096, seed=0)
    q = pkg.formats.unpack_mlx_q4(w, 4096)
    assert q.min() == 0 and q.max() == 15 and abs(q.mean() - 7.5) < 0.05
    sf, bf = pkg.bf16_to_f32(s), pkg.bf16_to_f32(b)
    assert 0.00498 <= sf.min() and sf.max() <= 0.0201
    assert abs(bf.std() - 0.01) < 0.001
    w2, _, _ = pkg.synth_q4(64, 4096, seed=0)
    assert np.array_equal(w, w2)


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "swlm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(swlm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    syms = _declared_symbols()
    assert len(syms) >= 35
    lib = pkg.load_library()  # raises if the .so is missing: there is no fallback
    for s in syms:
        assert hasattr(lib.dll, s), f"{s} declared in include/swlm.h but not exported"
        assert s in pkg.lib.SIGNATURES, f"{s} has no ctypes signature"
    assert lib.swlm_version().startswith(b"swlm-cuda")


def test_no_device_means_error_not_fallback(pkg):
    lib = pkg.load_library()
    if lib.swlm_device_count() > 0:
        pytest.skip("a CUDA device is present")
    h = ctypes.c_void_p()
    rc = lib.swlm_ctx_create(0, 0, 1, ctypes.byref(h))
    assert rc != 0 and not h.value
    assert b"no CUDA device" in lib.swlm_last_error()
    with pytest.raises(pkg.SwlmError):
        pkg.WeightStore(0)


def test_bad_arguments_are_rejected(pkg):
    lib = pkg.load_library()
    h = ctypes.c_void_p()
    assert lib.swlm_ctx_create(0, 3, 2, ctypes.byref(h)) == -1  # rank outside the group
    assert lib.swlm_position(None) == -1
    assert lib.swlm_plan_launch_count(None) == 0


def test_kv_cache_schemes_the_library_accepts(pkg):
    """KVCacheKernelSupportContractTests 'isSupportedForKVCache matches the pinned supported set'
    (Tests/MetalCompilerTests/Core/KVCacheKernelSupportContractTests.swift:20-50): the reference's attention kernels read
    and write fp16 / bf16 / fp32, q4 g64 / g128 / g128zero, q8 g32 / g64 / g128 and the two rotated schemes, and nothing
    else. This library offers that set without the dense fp16 and fp32 caches (its activations are bf16), 0 standing
    for "unset" = bf16; the sizable-but-unsupported schemes of the reference are refused here as well."""
    lib = pkg.load_library()
    reference_supported = {0x00, 0x01, 0x02, 0x40, 0x41, 0x42, 0x10, 0x11, 0x12, 0x71, 0x70}
    here = {s for s in range(0x100) if lib.swlm_kv_scheme_supported(s)}
    assert here == (reference_supported - {0x02}) and lib.swlm_kv_scheme_supported(0x00)    # (0 accepted as "unset", not as fp16)
    for scheme in here - {0x00, 0x01}:
        spec = pkg.KVCacheSpecification(layer_count=1, kv_head_count=1, head_dimension=128, maximum_sequence_length=1, scheme=scheme)
        assert spec.bytes_per_head_slot() % 64 == 0 and spec.bytes_per_head_slot() < 256     # every accepted block scheme is sizable


def test_tensor_parallel_head_split_is_checked(pkg):
    """Heads and KV heads must divide by the number of ranks, and every rank must keep whole GQA groups; anything else
    would silently compute with truncated head counts, so it is refused (host-only entry point; swlm_plan_build applies
    the same check to every attention and QK-norm step)."""
    lib = pkg.load_library()
    ok, unsupported = 0, -4
    assert lib.swlm_tp_check_heads(32, 8, 1) == ok
    assert lib.swlm_tp_check_heads(32, 8, 2) == ok
    assert lib.swlm_tp_check_heads(32, 8, 8) == ok       # one KV head per rank
    assert lib.swlm_tp_check_heads(8, 4, 8) == unsupported   # half a KV head per rank
    assert lib.swlm_tp_check_heads(12, 4, 8) == unsupported  # query heads do not divide
    assert lib.swlm_tp_check_heads(12, 6, 4) == unsupported
    assert lib.swlm_tp_check_heads(24, 8, 4) == ok
    assert b"GQA" in lib.swlm_last_error() or True
    assert lib.swlm_tp_check_heads(0, 8, 2) == -1


# ---- model directories (config.json + shards) ------------------------------------------------------------------------

LLAMA_CONFIG = {"model_type": "llama", "hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 2, "num_attention_heads": 4,
                "num_key_value_heads": 2, "vocab_size": 512, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
                "quantization": {"group_size": 64, "bits": 4}}


def test_config_json_decoding_follows_the_reference_rules(pkg):
    """HFConfigDecoder (Sources/SwiftLM/HFConfigDecoder.swift:6-170): quantization hint (also under text_config), defaults
    of heads / KV heads / head_dim / epsilon / RoPE base, LFM2's feed-forward adjustment and layer pattern, text_config
    merged over the top level; ModelGraphResolver's model types; refusal of what the recipes cannot express."""
    B = pkg.bundle
    assert B.quantization_hint(LLAMA_CONFIG) == (4, 64)
    assert B.quantization_hint({"text_config": {"quantization": {"bits": 4, "group_size": 128}}}) == (4, 128)
    assert B.quantization_hint({"quantization": {"bits": 4}}) is None and B.quantization_hint({}) is None
    c = B.decode_config(LLAMA_CONFIG)
    assert (c.family, c.hidden, c.intermediate, c.layers, c.heads, c.kv_heads, c.head_dim, c.vocab) == ("llama", 256, 512, 2, 4, 2, 64, 512)
    assert c.norm_eps == 1e-5 and c.rope_theta == 10000.0 and c.tie_embeddings is False and c.sliding_window == 0
    d = B.decode_config({"model_type": "mistral", "hidden_size": 128, "num_hidden_layers": 1, "vocab_size": 64, "sliding_window": 32})
    assert (d.heads, d.kv_heads, d.head_dim, d.intermediate, d.norm_eps, d.rope_theta, d.sliding_window) == (32, 32, 4, 512, 1e-6, 500000.0, 32)
    lfm2 = {"model_type": "lfm2", "hidden_size": 2048, "num_hidden_layers": 16, "vocab_size": 65536, "num_attention_heads": 32,
            "num_key_value_heads": 8, "block_ff_dim": 12288, "block_auto_adjust_ff_dim": True, "block_ffn_dim_multiplier": 1.0,
            "block_multiple_of": 256, "norm_eps": 1e-5, "rope_theta": 1000000.0, "conv_L_cache": 3, "tie_embedding": True,
            "full_attn_idxs": [2, 5, 8, 10, 12, 14]}
    l = B.decode_config(lfm2)
    assert (l.family, l.intermediate, l.head_dim, l.conv_kernel, l.tie_embeddings) == ("lfm2", 8192, 64, 3, True)
    assert list(l.attention_layers) == [2, 5, 8, 10, 12, 14] and l.kv_layer_count == 6 and l.conv_layer_count == 10
    types = ["conv", "conv", "full_attention", "conv"]
    assert list(B.decode_config(dict(lfm2, num_hidden_layers=4, layer_types=types, full_attn_idxs=None)).attention_layers) == [2]
    assert B.decode_config(dict(LLAMA_CONFIG, model_type="qwen3", qk_norm=True)).qk_norm is True and c.qk_norm is False
    merged = B.decode_config({"model_type": "llama", "vocab_size": 8, "text_config": {"hidden_size": 64, "num_hidden_layers": 3, "num_attention_heads": 2}})
    assert (merged.hidden, merged.layers, merged.vocab, merged.head_dim) == (64, 3, 8, 32)
    for bad, word in ((dict(LLAMA_CONFIG, num_local_experts=8), "experts"), (dict(LLAMA_CONFIG, attention_bias=True), "biases"),
                      (dict(LLAMA_CONFIG, model_type="gemma3_text"), "Unsupported"),
                      (dict(LLAMA_CONFIG, partial_rotary_factor=0.25), "rotary"), ({"model_type": "llama"}, "Missing hidden_size")):
        with pytest.raises(B.BundleError, match=word):
            B.decode_config(bad)
    with pytest.raises(B.BundleError, match="model_type"):
        B.decode_config({"hidden_size": 8})


def test_default_cache_policy_is_model_aware(pkg):
    """RotorQuantCorrectnessTests 'ModelBundleLoader resolves default policy to RotorQuant only for plain transformer
    attention graphs' (:99-161): the untouched default becomes the rotated 4-bit group-64 cache for K and V when the model
    has attention and no short-conv or recurrent layer; an explicit policy stands."""
    B = pkg.bundle
    llama, lfm2 = B.decode_config(LLAMA_CONFIG), pkg.lfm2_like_config()
    assert B.resolve_kv_policy(llama) == (0x71, 0)
    assert B.resolve_kv_policy(lfm2) == (0x01, 0)
    assert B.resolve_kv_policy(llama, requested_scheme=0x10) == (0x10, 0) and B.resolve_kv_policy(llama, 0x70, 16) == (0x70, 16)
    assert B.resolve_kv_policy(llama, maximum_sequence_length=8192) == (0x01, 0)     # not the default policy any more


def test_model_directory_is_prepared_without_a_gpu(pkg, tmp_path):
    """config.json + one MLX-quantized shard -> decoded recipe, resolved cache policy, model.staf beside the shards with
    the bundle's validity metadata; a second call reuses the file, a changed config.json rewrites it."""
    import json
    import os
    B, staf = pkg.bundle, pkg.staf
    d = str(tmp_path)
    config = dict(LLAMA_CONFIG, tie_word_embeddings=False)
    open(os.path.join(d, "config.json"), "w").write(json.dumps(config))
    cfg = B.decode_config(config)
    builder = pkg.DispatchPlanBuilder(cfg)
    weights = pkg.synth_model_weights(builder, seed=3)
    staf.write_safetensors(os.path.join(d, "model.safetensors"), pkg.bundle_tensors(builder, weights))
    got_cfg, got_builder, f = B.prepare_bundle(d, max_batch=2)
    assert (got_cfg.kv_scheme, got_cfg.kv_qjl_dim, got_cfg.max_batch, got_cfg.max_seq) == (0x71, 0, 2, 4096 + 128)
    assert got_cfg.buffers_desc().kv_scheme == 0x71
    out = os.path.join(d, "model.staf")
    assert f.metadata[staf.KEY_MODEL_FAMILY] == "llama" and f.metadata[staf.KEY_MODEL_HIDDEN] == 256
    for name, kind, _shape, _shard in got_builder.tensors():
        assert pkg.model.staf_tensor_name(name, kind) in f.names()
    stamp = os.stat(out).st_mtime_ns
    B.prepare_bundle(d, max_batch=2)
    assert os.stat(out).st_mtime_ns == stamp                                  # valid cache: kept
    open(os.path.join(d, "config.json"), "w").write(json.dumps(dict(config, rope_theta=20000.0)))
    cfg2, _, f2 = B.prepare_bundle(d, kv_scheme=0x10)
    assert cfg2.rope_theta == 20000.0 and cfg2.kv_scheme == 0x10 and f2.metadata[staf.KEY_MODEL_ROPE_THETA] == 20000.0
    assert f2.metadata[staf.KEY_SRC_CONFIG_HASH] != f.metadata[staf.KEY_SRC_CONFIG_HASH]
    with pytest.raises(B.BundleError, match="4-bit"):
        open(os.path.join(d, "config.json"), "w").write(json.dumps(dict(config, quantization={"bits": 8, "group_size": 64})))
        B.prepare_bundle(d)
    # a bundle whose embedding table is quantized too (what MLX's converter writes): the gather reads the Q4 rows, the
    # head stays its own tensor
    open(os.path.join(d, "config.json"), "w").write(json.dumps(config))
    qcfg = B.decode_config(config)
    qcfg.quantized_embedding = True
    qb = pkg.DispatchPlanBuilder(qcfg)
    kinds = {name: kind for name, kind, _s, _k in qb.tensors()}
    assert kinds["model.embed_tokens.weight"] == "q4" and kinds["lm_head"] == "q4"
    staf.write_safetensors(os.path.join(d, "model.safetensors"), pkg.bundle_tensors(qb, pkg.synth_model_weights(qb, seed=4)))
    cfg3, b3, f3 = B.prepare_bundle(d)
    assert cfg3.quantized_embedding and f3["model.embed_tokens.weight"].scheme == staf.SCHEME_Q4_G64 and "lm_head.weight" in f3.names()


def test_transformer_recipe_with_qk_norm(pkg, oracle):
    """Attention(qkNorm: .rmsNorm) of the plain transformer recipe (Sources/Models/Transformer.swift:49-64): the plan
    gains the two per-head norm weights per layer and a QK-norm step between the projections and attention; the oracle
    runs it, and the norm changes the result."""
    P = pkg.plan
    base = dict(hidden=256, intermediate=512, layers=2, heads=4, kv_heads=2, head_dim=64, vocab=512, max_seq=32)
    plain, normed = pkg.ModelConfig("llama", **base), pkg.ModelConfig("llama", qk_norm=True, **base)
    b0, b1 = pkg.DispatchPlanBuilder(plain), pkg.DispatchPlanBuilder(normed)
    names = [n for n, _k, _s, _sh in b1.tensors()]
    assert "model.layers.1.self_attn.q_layernorm.weight" in names and "model.layers.0.self_attn.k_layernorm.weight" in names
    assert len(b1.tensors()) == len(b0.tensors()) + 2 * base["layers"]
    kinds0, kinds1 = [s.kind for s in b0.decode_steps()], [s.kind for s in b1.decode_steps()]
    assert kinds0.count(P.STEP_QK_NORM) == 0 and kinds1.count(P.STEP_QK_NORM) == base["layers"]
    i = kinds1.index(P.STEP_QK_NORM)
    assert kinds1[i - 1] == P.STEP_QGEMV and kinds1[i + 1] == P.STEP_ATTN_DECODE
    weights = pkg.synth_model_weights(b1, seed=2)
    out = []
    for builder in (b0, b1):
        m = oracle.model(builder.config.buffers_desc())
        m.load(builder, weights)
        tok = m.prefill(np.array([[5, 6, 7, 8]], dtype=np.int32))
        out.append(pkg.bf16_to_f32(m.read_buffer(P.BUF_LOGITS, base["vocab"]))[0].copy())
        assert 0 <= int(tok[0]) < base["vocab"]
    assert np.max(np.abs(out[0] - out[1])) > 1e-3
