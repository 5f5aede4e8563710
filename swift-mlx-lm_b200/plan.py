"""Dispatch-plan builder: model recipe -> flat `swlm_step` list.

Mirrors what the reference's compiler emits for the two recipes of the hot path:
`Transformer` (Sources/Models/Transformer.swift:9-100) and `LFM2` (Sources/Models/LFM2/LFM2.swift:60-158),
lowered by `AttentionAttributes.fragment` (Sources/MetalCompiler/Compilable/AttentionFragment.swift:8-153),
`MLPFragment.swift:7-14`, `ShortConvFragment.swift:5-9`, with the copy / residual-add / norm fusion of
`MetalEntryCollector` (Compiler/MetalEntryCollector.swift:143-218, :238-249) and the scratch-slot routing of
`DecodeRoutingPlanner` (Compiler/MetalDispatchStepBuilder.swift:587-737). Tensor names follow
`LlamaFamilyNaming.swift:36-96` and `LFM2FamilyNaming.swift:22-96`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Sequence

from .lib import BuffersDesc, Step

# logical buffers (include/swlm_plan.h)
BUF_HIDDEN, BUF_RESIDUAL, BUF_S0, BUF_S1, BUF_S2, BUF_S3, BUF_S4, BUF_LOGITS = range(8)

STEP_EMBED = 1
STEP_COPY_RMSNORM = 2
STEP_RESADD_COPY_RMSNORM = 3
STEP_RESADD_RMSNORM = 4
STEP_QGEMV = 5
STEP_QK_NORM = 6
STEP_ATTN_DECODE = 7
STEP_SWIGLU = 8
STEP_CONV_STATE_UPDATE = 9
STEP_ARGMAX = 10
STEP_GEGLU = 11
STEP_SSM_RECURRENCE = 12

SHARD_REPLICATE, SHARD_COLUMN, SHARD_ROW, SHARD_COLUMN3 = 0, 1, 2, 3


@dataclass
class ModelConfig:
    family: str  # "llama" | "lfm2" | "deltanet" (recurrent layers of the Qwen3.5 kind between Llama-style attention layers)
    hidden: int
    intermediate: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    vocab: int
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    conv_kernel: int = 3
    attention_layers: Sequence[int] = field(default_factory=list)  # lfm2: indices that are attention layers
    max_seq: int = 4224
    max_batch: int = 1
    # The output head reuses the embedding table (Sources/Models/LlamaFamilyNaming.swift:22-27): one Q4 group-64
    # tensor serves the row gather (embedding_lookup_q4) and the lm_head product.
    tie_embeddings: bool = False
    # An untied model whose embedding table is a Q4 tensor of its own (MLX-quantized bundles quantize embed_tokens as
    # well as lm_head): the row gather reads the packed rows (embedding_lookup_q4), the head stays a separate tensor.
    quantized_embedding: bool = False
    # Per-head RMS norm of q and k before RoPE in the plain transformer recipe (Attention(qkNorm: .rmsNorm),
    # Sources/Models/Transformer.swift:49-64; tensors `self_attn.q_layernorm.weight` / `k_layernorm.weight`,
    # LlamaFamilyNaming.swift:50-54). The LFM2 recipe always has it.
    qk_norm: bool = False
    # Gemma-style variants of the same recipe (Generator/MetalSourceGenerator+NormAndElementwise.swift:176-208):
    # the gated MLP's activation ("silu" = SwiGLU, "gelu_tanh" = GEGLU) and the constant added to every RMSNorm
    # weight (weightBias, 1.0 for checkpoints that store weight - 1).
    activation: str = "silu"
    norm_weight_bias: float = 0.0
    # Sliding-window attention (windowLeft, Generator/MetalSourceGenerator+Attention.swift:851-853): a token attends
    # itself and the sliding_window - 1 positions before it; 0 = full attention. `sliding_window_layers` names the
    # layers that use it (None: every attention layer), the others attend everything.
    sliding_window: int = 0
    sliding_window_layers: Sequence[int] = None
    # "deltanet": the layers not listed in attention_layers are gated-delta-rule recurrent layers
    # (Sources/LMArchitecture/Declaration/Components/DeltaNet.swift, Primitives/SSMRecurrenceFragment.swift) with
    # `ssm_heads` value heads of `ssm_value_dim`, `ssm_groups` key groups of `ssm_key_dim`, a causal conv of
    # `ssm_conv_kernel` taps over the q|k|v channels; tensor names follow Models/Qwen35/Qwen35FamilyNaming.swift:73-87.
    # KV cache elements: 0 = bf16; 0x10 / 0x11 / 0x12 = 8-bit groups of 32 / 64 / 128; 0x40 / 0x41 / 0x42 = 4-bit groups of 64 / 128 / 128
    # (KVCacheSpecification's affine block schemes); 0x70 / 0x71 = the rotated forms of 0x10 / 0x40 (rows turned by
    # Cl(3,0) rotors before quantisation), with kv_qjl_dim > 0 (at most 64) plus the projected K residuals that correct
    # the scores (RotorQuant + QJL, Buffer/MetalGraphAllocator.swift:177-216)
    kv_scheme: int = 0
    kv_qjl_dim: int = 0
    ssm_heads: int = 0
    ssm_groups: int = 0
    ssm_key_dim: int = 0
    ssm_value_dim: int = 0
    ssm_conv_kernel: int = 4

    def is_attention_layer(self, i: int) -> bool:
        return self.family == "llama" or i in self.attention_layers

    @property
    def kv_layer_count(self) -> int:
        return sum(1 for i in range(self.layers) if self.is_attention_layer(i))

    @property
    def conv_layer_count(self) -> int:
        return self.layers - self.kv_layer_count if self.family == "lfm2" else 0

    @property
    def ssm_layer_count(self) -> int:
        return self.layers - self.kv_layer_count if self.family == "deltanet" else 0

    @property
    def ssm_conv_dim(self) -> int:
        return 2 * self.ssm_groups * self.ssm_key_dim + self.ssm_heads * self.ssm_value_dim

    @property
    def slot_dim(self) -> int:
        # slotDimension = max(hidden, max(intermediate, 4*hidden), widest projection)
        # (Sources/MetalCompiler/Buffer/MetalBufferAllocator.swift:13-18)
        widest = max(self.heads * self.head_dim, 3 * self.hidden if self.family == "lfm2" else 0,
                     self.ssm_conv_dim if self.family == "deltanet" else 0)
        return max(self.hidden, self.intermediate, 4 * self.hidden, widest)

    def buffers_desc(self) -> BuffersDesc:
        return BuffersDesc(
            hidden=self.hidden, slot_dim=self.slot_dim, vocab=self.vocab, max_seq=self.max_seq,
            max_batch=self.max_batch, kv_layers=self.kv_layer_count, kv_heads=self.kv_heads,
            head_dim=self.head_dim, conv_layers=self.conv_layer_count,
            conv_dim=self.hidden if self.conv_layer_count else 0,
            conv_kernel=self.conv_kernel if self.conv_layer_count else 0,
            ssm_layers=self.ssm_layer_count, ssm_heads=self.ssm_heads if self.ssm_layer_count else 0,
            ssm_groups=self.ssm_groups if self.ssm_layer_count else 0, ssm_key_dim=self.ssm_key_dim if self.ssm_layer_count else 0,
            ssm_value_dim=self.ssm_value_dim if self.ssm_layer_count else 0,
            ssm_conv_kernel=self.ssm_conv_kernel if self.ssm_layer_count else 0,
            kv_scheme=self.kv_scheme, kv_qjl_dim=self.kv_qjl_dim,
        )

    # Algorithmic weight bytes one decode step streams: 0.5625 bytes per quantized weight.
    def q4_weight_elems(self) -> int:
        h, f = self.hidden, self.intermediate
        total = 0
        for i in range(self.layers):
            total += 3 * h * f
            if self.is_attention_layer(i):
                total += 2 * h * self.heads * self.head_dim + 2 * h * self.kv_heads * self.head_dim
            elif self.family == "deltanet":
                total += h * (self.ssm_conv_dim + 2 * self.ssm_heads * self.ssm_value_dim + 2 * self.ssm_heads)
            else:
                total += 3 * h * h + h * h
        return total + h * self.vocab


def llama3_8b_config(max_seq: int = 4224, max_batch: int = 1) -> ModelConfig:
    return ModelConfig("llama", 4096, 14336, 32, 32, 8, 128, 128256, 1e-5, 500000.0, max_seq=max_seq, max_batch=max_batch)


def lfm2_like_config(max_seq: int = 2304, max_batch: int = 1, tie_embeddings: bool = True) -> ModelConfig:
    # 16 layers, 10 gated short-conv (kernel 3) + 6 attention; the attention layer indices are this
    # build's choice (every third layer starting at 2), the layer pattern not being part of the reference tree.
    # LFM2 ties its output head to the embedding table; the choice here is the MLX-bundle convention, one Q4
    # group-64 table of 65536 x 2048 (75.5 MB per token for the head, not the 268 MB of a bf16 table).
    return ModelConfig("lfm2", 2048, 8192, 16, 32, 8, 64, 65536, 1e-5, 1000000.0, 3,
                       attention_layers=[2, 5, 8, 10, 12, 14], max_seq=max_seq, max_batch=max_batch,
                       tie_embeddings=tie_embeddings)


def _step(kind: int, **kw) -> Step:
    s = Step()
    s.kind = kind
    s.layer = -1
    s.in_buf = s.in2_buf = s.in3_buf = s.in4_buf = s.out_buf = -1
    for key, value in kw.items():
        if key in ("weight", "weight2", "weight3", "weight4"):
            value = value.encode()
        setattr(s, key, value)
    return s


class DispatchPlanBuilder:
    """Emit the decode step list for a model recipe; also lists the tensors the plan needs."""

    def __init__(self, config: ModelConfig):
        self.config = config

    # -- tensor inventory: (name, kind, shape, shard_kind) ----------------------------------------
    def tensors(self):
        c = self.config
        h, f, qd, kvd = c.hidden, c.intermediate, c.heads * c.head_dim, c.kv_heads * c.head_dim
        out = [("model.embed_tokens.weight", "q4" if c.tie_embeddings or c.quantized_embedding else "dense", (c.vocab, h), SHARD_REPLICATE)]
        for i in range(c.layers):
            p = f"model.layers.{i}."
            if c.family in ("llama", "deltanet"):
                out.append((p + "input_layernorm.weight", "norm", (h,), SHARD_REPLICATE))
                if c.is_attention_layer(i):
                    out += [
                        (p + "self_attn.q_proj", "q4", (qd, h), SHARD_COLUMN),
                        (p + "self_attn.k_proj", "q4", (kvd, h), SHARD_COLUMN),
                        (p + "self_attn.v_proj", "q4", (kvd, h), SHARD_COLUMN),
                        (p + "self_attn.o_proj", "q4", (h, qd), SHARD_ROW),
                    ]
                    if c.qk_norm:
                        out += [(p + "self_attn.q_layernorm.weight", "norm", (c.head_dim,), SHARD_REPLICATE),
                                (p + "self_attn.k_layernorm.weight", "norm", (c.head_dim,), SHARD_REPLICATE)]
                else:
                    vd = c.ssm_heads * c.ssm_value_dim
                    out += [
                        (p + "linear_attn.in_proj_qkv", "q4", (c.ssm_conv_dim, h), SHARD_REPLICATE),
                        (p + "linear_attn.in_proj_z", "q4", (vd, h), SHARD_REPLICATE),
                        (p + "linear_attn.in_proj_b", "q4", (c.ssm_heads, h), SHARD_REPLICATE),
                        (p + "linear_attn.in_proj_a", "q4", (c.ssm_heads, h), SHARD_REPLICATE),
                        (p + "linear_attn.conv1d.weight", "conv", (c.ssm_conv_dim, c.ssm_conv_kernel), SHARD_REPLICATE),
                        (p + "linear_attn.norm.weight", "f32", (c.ssm_value_dim,), SHARD_REPLICATE),
                        (p + "linear_attn.dt_bias", "dense", (c.ssm_heads,), SHARD_REPLICATE),
                        (p + "linear_attn.A_log", "f32", (c.ssm_heads,), SHARD_REPLICATE),
                        (p + "linear_attn.out_proj", "q4", (h, vd), SHARD_REPLICATE),
                    ]
                out += [
                    (p + "post_attention_layernorm.weight", "norm", (h,), SHARD_REPLICATE),
                    (p + "mlp.gate_proj", "q4", (f, h), SHARD_COLUMN),
                    (p + "mlp.up_proj", "q4", (f, h), SHARD_COLUMN),
                    (p + "mlp.down_proj", "q4", (h, f), SHARD_ROW),
                ]
            else:
                out.append((p + "operator_norm.weight", "norm", (h,), SHARD_REPLICATE))
                if c.is_attention_layer(i):
                    out += [
                        (p + "self_attn.q_proj", "q4", (qd, h), SHARD_COLUMN),
                        (p + "self_attn.k_proj", "q4", (kvd, h), SHARD_COLUMN),
                        (p + "self_attn.v_proj", "q4", (kvd, h), SHARD_COLUMN),
                        (p + "self_attn.q_layernorm.weight", "norm", (c.head_dim,), SHARD_REPLICATE),
                        (p + "self_attn.k_layernorm.weight", "norm", (c.head_dim,), SHARD_REPLICATE),
                        (p + "self_attn.out_proj", "q4", (h, qd), SHARD_ROW),
                    ]
                else:
                    out += [
                        (p + "conv.in_proj", "q4", (3 * h, h), SHARD_COLUMN3),
                        (p + "conv.conv.weight", "conv", (h, c.conv_kernel), SHARD_COLUMN),
                        (p + "conv.out_proj", "q4", (h, h), SHARD_ROW),
                    ]
                out += [
                    (p + "ffn_norm.weight", "norm", (h,), SHARD_REPLICATE),
                    (p + "feed_forward.w1", "q4", (f, h), SHARD_COLUMN),
                    (p + "feed_forward.w3", "q4", (f, h), SHARD_COLUMN),
                    (p + "feed_forward.w2", "q4", (h, f), SHARD_ROW),
                ]
        final_norm = "model.norm.weight" if c.family != "lfm2" else "model.embedding_norm.weight"
        out.append((final_norm, "norm", (h,), SHARD_REPLICATE))
        if not c.tie_embeddings:
            out.append(("lm_head", "q4", (c.vocab, h), SHARD_COLUMN))
        return out

    # -- decode steps ---------------------------------------------------------------------------
    def decode_steps(self) -> List[Step]:
        c = self.config
        h, f, qd, kvd = c.hidden, c.intermediate, c.heads * c.head_dim, c.kv_heads * c.head_dim
        eps = c.norm_eps
        steps = [_step(STEP_EMBED, out_buf=BUF_HIDDEN, n=h, weight="model.embed_tokens.weight")]
        kv_layer = conv_layer = ssm_layer = 0
        first = True

        def norm(name: str):
            nonlocal first
            kind = STEP_COPY_RMSNORM if first else STEP_RESADD_COPY_RMSNORM
            first = False
            steps.append(_step(kind, in_buf=BUF_HIDDEN, out_buf=BUF_S0, n=h, eps=eps, weight_bias=c.norm_weight_bias, weight=name))

        def gemv(name: str, src: int, dst: int, n: int, k: int):
            steps.append(_step(STEP_QGEMV, in_buf=src, out_buf=dst, n=n, k=k, weight=name))

        for i in range(c.layers):
            p = f"model.layers.{i}."
            attn = c.is_attention_layer(i)
            norm(p + ("input_layernorm.weight" if c.family != "lfm2" else "operator_norm.weight"))
            if attn:
                gemv(p + "self_attn.q_proj", BUF_S0, BUF_S1, qd, h)
                gemv(p + "self_attn.k_proj", BUF_S0, BUF_S2, kvd, h)
                gemv(p + "self_attn.v_proj", BUF_S0, BUF_S3, kvd, h)
                if c.family == "lfm2" or c.qk_norm:
                    steps.append(_step(STEP_QK_NORM, in_buf=BUF_S1, in2_buf=BUF_S2, heads=c.heads, kv_heads=c.kv_heads,
                                       head_dim=c.head_dim, eps=eps, weight_bias=0.0,
                                       weight=p + "self_attn.q_layernorm.weight", weight2=p + "self_attn.k_layernorm.weight"))
                steps.append(_step(STEP_ATTN_DECODE, layer=kv_layer, in_buf=BUF_S1, in2_buf=BUF_S2, in3_buf=BUF_S3,
                                   out_buf=BUF_S0, heads=c.heads, kv_heads=c.kv_heads, head_dim=c.head_dim,
                                   rope_dim=c.head_dim, rope_base=c.rope_theta, scale=1.0 / math.sqrt(c.head_dim),
                                   window_left=c.sliding_window if c.sliding_window > 0 and (
                                       c.sliding_window_layers is None or i in c.sliding_window_layers) else 0))
                kv_layer += 1
                gemv(p + ("self_attn.o_proj" if c.family != "lfm2" else "self_attn.out_proj"), BUF_S0, BUF_HIDDEN, h, qd)
            elif c.family == "deltanet":
                lp, vd = p + "linear_attn.", c.ssm_heads * c.ssm_value_dim
                gemv(lp + "in_proj_qkv", BUF_S0, BUF_S1, c.ssm_conv_dim, h)
                gemv(lp + "in_proj_z", BUF_S0, BUF_S2, vd, h)
                gemv(lp + "in_proj_b", BUF_S0, BUF_S3, c.ssm_heads, h)
                gemv(lp + "in_proj_a", BUF_S0, BUF_S4, c.ssm_heads, h)
                steps.append(_step(STEP_SSM_RECURRENCE, layer=ssm_layer, in_buf=BUF_S1, in2_buf=BUF_S2, in3_buf=BUF_S3, in4_buf=BUF_S4,
                                   out_buf=BUF_S0, heads=c.ssm_heads, groups=c.ssm_groups, key_dim=c.ssm_key_dim,
                                   value_dim=c.ssm_value_dim, conv_kernel=c.ssm_conv_kernel, weight=lp + "conv1d.weight",
                                   weight2=lp + "norm.weight", weight3=lp + "dt_bias", weight4=lp + "A_log"))
                ssm_layer += 1
                gemv(lp + "out_proj", BUF_S0, BUF_HIDDEN, h, vd)
            else:
                gemv(p + "conv.in_proj", BUF_S0, BUF_S1, 3 * h, h)
                steps.append(_step(STEP_CONV_STATE_UPDATE, layer=conv_layer, in_buf=BUF_S1, out_buf=BUF_S0, n=h,
                                   conv_kernel=c.conv_kernel, weight=p + "conv.conv.weight"))
                conv_layer += 1
                gemv(p + "conv.out_proj", BUF_S0, BUF_HIDDEN, h, h)
            norm(p + ("post_attention_layernorm.weight" if c.family != "lfm2" else "ffn_norm.weight"))
            gate, up, down = (("mlp.gate_proj", "mlp.up_proj", "mlp.down_proj") if c.family != "lfm2"
                              else ("feed_forward.w1", "feed_forward.w3", "feed_forward.w2"))
            gemv(p + gate, BUF_S0, BUF_S1, f, h)
            gemv(p + up, BUF_S0, BUF_S2, f, h)
            steps.append(_step(STEP_GEGLU if c.activation == "gelu_tanh" else STEP_SWIGLU, in_buf=BUF_S1, in2_buf=BUF_S2, out_buf=BUF_S0, n=f))
            gemv(p + down, BUF_S0, BUF_HIDDEN, h, f)
        final_norm = "model.norm.weight" if c.family != "lfm2" else "model.embedding_norm.weight"
        steps.append(_step(STEP_RESADD_RMSNORM, in_buf=BUF_HIDDEN, out_buf=BUF_S0, n=h, eps=eps, weight_bias=c.norm_weight_bias, weight=final_norm))
        gemv("model.embed_tokens.weight" if c.tie_embeddings else "lm_head", BUF_S0, BUF_LOGITS, c.vocab, h)
        steps.append(_step(STEP_ARGMAX, in_buf=BUF_LOGITS, n=c.vocab))
        return steps
