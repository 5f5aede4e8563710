"""On a B200: the reference's multi-block known answers through both upload formats, a model directory (config.json +
MLX-quantized shard) loaded the way the reference's bundle loader takes it, and the plain transformer recipe with QK norm."""
import numpy as np
import pytest

from test_gpu_model import greedy_compare

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def store(pkg):
    s = pkg.WeightStore(0)
    yield s
    s.close()


def _bf(pkg, a):
    return pkg.f32_to_bf16(np.asarray(a, dtype=np.float32))


@pytest.mark.parametrize("case", ["gemv_multi_block_g64", "gemv_multi_block_g128"])
def test_qgemv_multi_block_known_answers(pkg, store, golden, case):
    """UnifiedGEMVMultiBlockTests (Q4G64, Q4G128): one row over four blocks with their own scale and zero, against the
    reference test's fp32 expectation and tolerance; as MLX words and as STAF blocks."""
    g = golden[case]
    group, k = g["group"], g["group"] * g["blocks"]
    w = pkg.pack_mlx_q4(np.array([g["q"]], dtype=np.uint8))
    s, z = _bf(pkg, [g["scales"]]), _bf(pkg, [g["zeros"]])
    store.add_q4_mlx(f"kat.{case}", w, s, z)
    store.add_q4_staf(f"kat.{case}.staf", pkg.formats.repack_mlx_to_staf(w, s, z, group=group), 1, k, group=group)
    for name in (f"kat.{case}", f"kat.{case}.staf"):
        y = pkg.bf16_to_f32(store.qgemm(name, _bf(pkg, [g["x"]]), 1))
        assert abs(float(y[0, 0]) - g["expected"]) < max(g["abs_tol"], g["rel_tol"] * abs(g["expected"]))


@pytest.mark.parametrize("default_policy", [False, True])
def test_model_directory_loads_and_decodes(pkg, oracle, tmp_path, default_policy):
    """ModelBundleLoader's route for the plain transformer recipe: config.json + an MLX-quantized shard in a directory ->
    decoded recipe, model.staf with the bundle's metadata, upload, plan. With an explicit sequence length the cache is dense
    bf16; with the loader's untouched default policy it is the rotated 4-bit group-64 cache, as the reference resolves it
    (Sources/SwiftLM/ModelBundleLoader.swift:352-370). Tokens and logits against the oracle under the same policy."""
    import json
    import os

    d = str(tmp_path)
    config = {"model_type": "llama", "hidden_size": 512, "intermediate_size": 1536, "num_hidden_layers": 4, "num_attention_heads": 8,
              "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 4096, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
              "tie_word_embeddings": False, "quantization": {"group_size": 64, "bits": 4}}
    open(os.path.join(d, "config.json"), "w").write(json.dumps(config))
    source_cfg = pkg.bundle.decode_config(config)
    source_cfg.quantized_embedding = default_policy     # MLX's converter quantizes embed_tokens too: the Q4 row gather
    builder = pkg.DispatchPlanBuilder(source_cfg)
    weights = pkg.synth_model_weights(builder, seed=9)
    pkg.staf.write_safetensors(os.path.join(d, "model.safetensors"), pkg.bundle_tensors(builder, weights))
    store = pkg.WeightStore(0)
    gm = pkg.load_bundle(d, store) if default_policy else pkg.load_bundle(d, store, max_seq=128)
    cfg, _, _ = pkg.prepare_bundle(d) if default_policy else pkg.prepare_bundle(d, max_seq=128)
    assert (cfg.kv_scheme, cfg.max_seq, cfg.quantized_embedding) == ((0x71, 4096 + 128, True) if default_policy else (0x01, 128, False))
    assert os.path.exists(os.path.join(d, "model.staf"))
    om = oracle.model(cfg.buffers_desc())
    om.load(pkg.DispatchPlanBuilder(cfg), weights, staf_fp16=True)     # STAF blocks carry fp16 scales and zeros
    oracle.set_threads(0)
    mism = greedy_compare(pkg, gm, om, cfg, prompt_len=9, steps=24)
    assert len(mism) <= 2, mism
    gm.close(); store.close()


@pytest.mark.parametrize("batch", [1, 3])
def test_transformer_recipe_with_qk_norm_against_oracle(pkg, oracle, batch):
    """The plain transformer recipe with per-head q / k RMS norm before RoPE (Sources/Models/Transformer.swift:49-64):
    a short prompt and greedy steps against the oracle, one sequence and three."""
    from test_gpu_model import build_pair

    cfg = pkg.ModelConfig("llama", hidden=512, intermediate=1536, layers=4, heads=8, kv_heads=2, head_dim=64, vocab=4096,
                          norm_eps=1e-5, rope_theta=500000.0, max_seq=128, max_batch=batch, qk_norm=True)
    store, gm, om = build_pair(pkg, oracle, cfg)
    assert "qk" in gm.describe().lower()
    mism = greedy_compare(pkg, gm, om, cfg, prompt_len=7, steps=24)
    assert len(mism) <= 2, mism
    gm.close(); store.close()
