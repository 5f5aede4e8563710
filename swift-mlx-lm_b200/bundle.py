"""A model directory (config.json + MLX-quantized safetensors shards) into a running model: the host side of the
reference's ModelBundleLoader for the recipes this package builds (Sources/SwiftLM/ModelBundleLoader.swift,
HFConfigDecoder.swift, ModelGraphResolver.swift).

    cfg, builder, staf_file = prepare_bundle(directory)          # host only: decode config, convert / reuse model.staf
    model = load_bundle(directory, WeightStore(0))               # + upload and plan build

Tokenizers, chat templates, vision towers and the recipes outside the hot path (mixture-of-experts, Gemma, Cohere,
the real Qwen3.5 attention with its output gate) stay with the reference; configurations that need them are refused
with the reason.
"""
from __future__ import annotations

import glob
import json
import os
from typing import Dict, Optional, Tuple

from . import staf as _staf
from .plan import DispatchPlanBuilder, ModelConfig

# model_type values ModelGraphResolver.resolveModelGraph sends to the plain Transformer recipe (:9-13), without the
# mixture-of-experts ones
TRANSFORMER_MODEL_TYPES = ("llama", "qwen2", "qwen3", "mistral", "phi", "phi3", "starcoder2", "gpt_neox", "internlm2",
                           "deepseek", "yi", "baichuan", "chatglm")
LFM2_MODEL_TYPES = ("lfm2",)

# KVCachePolicy of InferencePolicy.default (Sources/MetalCompiler/InferencePolicy.swift:55-100)
DEFAULT_MAXIMUM_SEQUENCE_LENGTH = 4096
KV_AUTOMATIC = "automatic"


class BundleError(ValueError):
    pass


def quantization_hint(config: Dict) -> Optional[Tuple[int, int]]:
    """(bits, group_size) of config.json's `quantization` object, also looked for under `text_config`
    (HFConfigDecoder.quantizationHint, HFConfigDecoder.swift:6-20); None when absent or incomplete."""
    text = config.get("text_config")
    for candidate in (config.get("quantization"), text.get("quantization") if isinstance(text, dict) else None):
        if isinstance(candidate, dict):
            bits, group = candidate.get("bits"), candidate.get("group_size")
            if isinstance(bits, int) and isinstance(group, int):
                return bits, group
            return None
    return None


def model_type(config: Dict) -> str:
    mt = config.get("model_type")
    if not isinstance(mt, str):
        raise BundleError("Missing model_type in config.json")
    return mt


def _first(config: Dict, keys, default=None):
    for key in keys:
        if config.get(key) is not None:
            return config[key]
    return default


def decode_config(config: Dict, max_seq: int = DEFAULT_MAXIMUM_SEQUENCE_LENGTH + 128, max_batch: int = 1) -> ModelConfig:
    """config.json into a ModelConfig by HFConfigDecoder.decode's key rules (HFConfigDecoder.swift:30-170): `text_config`
    merged over the top level when it carries `hidden_size`; intermediate size from `intermediate_size` / `block_ff_dim`
    with LFM2's two-thirds / multiplier / multiple-of adjustment; heads, KV heads and head_dim with the reference's
    defaults; norm epsilon and RoPE base from the same key chains; tied head from `tie_word_embeddings` /
    `tie_embedding`; LFM2's layer pattern from `layer_types` or `full_attn_idxs`. Anything the Llama / LFM2 recipes of
    this package cannot express is refused."""
    raw = config
    text = raw.get("text_config")
    if isinstance(text, dict) and text.get("hidden_size") is not None:
        config = dict(raw)
        config.update(text)
    mt = model_type(config).lower()
    for key in ("hidden_size", "num_hidden_layers", "vocab_size"):
        if not isinstance(config.get(key), int):
            raise BundleError(f"Missing {key}")
    hidden, layers, vocab = config["hidden_size"], config["num_hidden_layers"], config["vocab_size"]
    intermediate = _first(config, ("intermediate_size", "block_ff_dim"), hidden * 4)
    if _first(config, ("block_auto_adjust_ff_dim", "block_use_swiglu"), False):
        adjusted = intermediate * 2 // 3
        if isinstance(config.get("block_ffn_dim_multiplier"), (int, float)):
            adjusted = int(float(config["block_ffn_dim_multiplier"]) * float(adjusted))
        multiple = config.get("block_multiple_of") or 256
        intermediate = multiple * ((adjusted + multiple - 1) // multiple)
    heads = config.get("num_attention_heads") or 32
    kv_heads = config.get("num_key_value_heads") or heads
    head_dim = config.get("head_dim") or hidden // heads
    eps = float(_first(config, ("rms_norm_eps", "layer_norm_eps", "norm_eps", "block_norm_eps"), 1e-6))
    rope = config.get("rope_parameters") if isinstance(config.get("rope_parameters"), dict) else {}
    theta = float(_first(config, ("rope_local_base_freq", "rope_theta"), rope.get("rope_theta", 500000.0)))
    tied = bool(_first(config, ("tie_word_embeddings", "tie_embedding"), False))

    def refuse(what):
        raise BundleError(f"model_type {mt}: {what} is outside the recipes of this package")

    if _first(config, ("num_local_experts", "num_experts")):
        refuse("a mixture of experts")
    if config.get("attention_bias") or config.get("mlp_bias"):
        refuse("projection biases")
    partial = _first(config, ("partial_rotary_factor",), rope.get("partial_rotary_factor"))
    if partial is not None and float(partial) != 1.0:
        refuse("a partial rotary factor")
    if config.get("rope_dim") not in (None, head_dim):
        refuse("a RoPE dimension below head_dim")
    common = dict(hidden=hidden, intermediate=intermediate, layers=layers, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                  vocab=vocab, norm_eps=eps, rope_theta=theta, tie_embeddings=tied, max_seq=max_seq, max_batch=max_batch)
    if mt in LFM2_MODEL_TYPES:
        types = config.get("layer_types")
        if isinstance(types, list):
            attention = [i for i, t in enumerate(types) if t == "full_attention"]
        elif isinstance(config.get("full_attn_idxs"), list):
            attention = [int(i) for i in config["full_attn_idxs"]]
        else:
            raise BundleError("lfm2: neither layer_types nor full_attn_idxs says which layers are attention layers")
        kernel = _first(config, ("conv_L_cache", "conv_kernel_size"), 3)
        return ModelConfig("lfm2", conv_kernel=int(kernel), attention_layers=attention, **common)
    if mt in TRANSFORMER_MODEL_TYPES:
        window = config.get("sliding_window")
        return ModelConfig("llama", sliding_window=int(window) if isinstance(window, int) and window > 0 else 0,
                           qk_norm=bool(config.get("qk_norm", False)), **common)
    raise BundleError(f"Unsupported model_type: {mt}")


def resolve_kv_policy(cfg: ModelConfig, requested_scheme=KV_AUTOMATIC, qjl_dimension: int = 0,
                      maximum_sequence_length: int = DEFAULT_MAXIMUM_SEQUENCE_LENGTH) -> Tuple[int, int]:
    """(kv_scheme, kv_qjl_dim) by ModelBundleLoader.resolveInferencePolicy (ModelBundleLoader.swift:352-370, 445-447): a
    caller's explicit scheme stands; the untouched default policy (automatic scheme, 4096 tokens) becomes the rotated
    4-bit group-64 cache for K and V when the model has attention layers and no layer with sequence state (short conv or
    recurrent), and stays dense otherwise."""
    if requested_scheme != KV_AUTOMATIC:
        return int(requested_scheme), int(qjl_dimension)
    plain_attention = cfg.kv_layer_count > 0 and cfg.conv_layer_count == 0 and cfg.ssm_layer_count == 0
    if maximum_sequence_length == DEFAULT_MAXIMUM_SEQUENCE_LENGTH and qjl_dimension == 0 and plain_attention:
        return 0x71, 0
    return 0x01, 0


def prepare_bundle(directory: str, max_seq: Optional[int] = None, max_batch: int = 1, kv_scheme=KV_AUTOMATIC, qjl_dimension: int = 0):
    """Everything that needs no GPU: read config.json, decode it, resolve the cache policy, convert the shards to
    `model.staf` beside them unless a cache that is valid for this bundle is already there (STAFCacheLoader with the
    bundle's metadata), and open it. Returns (ModelConfig, DispatchPlanBuilder, STAFFile)."""
    config_path = os.path.join(directory, "config.json")
    if not os.path.exists(config_path):
        raise BundleError(f"{directory}: no config.json")
    config_data = open(config_path, "rb").read()
    config = json.loads(config_data.decode())
    if not isinstance(config, dict):
        raise BundleError("config.json is not a JSON object")
    hint = quantization_hint(config)
    if hint is None or hint[0] != 4 or hint[1] not in (64, 128):
        raise BundleError(f"quantization {hint}: this package runs 4-bit bundles with groups of 64 or 128")
    policy_seq = DEFAULT_MAXIMUM_SEQUENCE_LENGTH if max_seq is None else max_seq
    cfg = decode_config(config, max_seq=policy_seq + 128 if max_seq is None else max_seq, max_batch=max_batch)
    cfg.kv_scheme, cfg.kv_qjl_dim = resolve_kv_policy(cfg, kv_scheme, qjl_dimension, policy_seq)
    shards = sorted(glob.glob(os.path.join(directory, "*.safetensors")))
    if not shards:
        raise BundleError(f"{directory}: no safetensors shard")
    # MLX-quantized bundles carry the embedding table as a quantized triple as well
    cfg.quantized_embedding = any(name.endswith("embed_tokens.scales") for p in shards for name in _staf.safetensors_names(p))
    expected = _staf.bundle_metadata(directory, model_type(config), cfg, config_data, shards)
    out = os.path.join(directory, "model.staf")
    _staf.convert_safetensors(shards, out, extra_metadata=expected, group_size=hint[1])
    return cfg, DispatchPlanBuilder(cfg), _staf.read_staf(out)


def load_bundle(directory: str, store, **kw):
    """prepare_bundle, then upload what the plan needs from the STAF file and build the plan (needs a GPU)."""
    from .model import load_model_from_staf

    _cfg, builder, staf_file = prepare_bundle(directory, **kw)
    return load_model_from_staf(store, builder, staf_file)
