/*
 * swlm_plan.h — the execution record shared by the host and the CUDA backend.
 *
 * A plan is a flat array of `swlm_step` records, one per reference dispatch.
 * It replaces the reference's `MetalDispatchStep` / `MetalDispatchPlan`
 * (Sources/MetalCompiler/Execution/MetalDecodePlan.swift:6-193): where the
 * reference stores {pipeline, grid, buffer bindings, constants}, a step here
 * stores {operation kind, logical buffer slots, tensor names, dimensions}.
 * The backend is free to fuse adjacent steps into one launch as long as every
 * value that the reference stores to a decode buffer is rounded to bf16 at the
 * same point.
 *
 * Logical buffers follow the reference's decode buffer set
 * (Sources/MetalCompiler/Buffer/MetalBufferAllocator.swift:4-132): `hidden`,
 * `residual`, five scratch slots of `slot_dim` elements, `logits`, all bf16,
 * one row per sequence of the batch.
 */
#ifndef SWLM_PLAN_H
#define SWLM_PLAN_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SWLM_NAME_MAX 96

/* Logical buffer ids used by swlm_step.in_buf / in2_buf / out_buf. */
enum {
    SWLM_BUF_NONE = -1,
    SWLM_BUF_HIDDEN = 0,
    SWLM_BUF_RESIDUAL = 1,
    SWLM_BUF_SCRATCH0 = 2, /* block output: attention / conv / swiglu result, norm output */
    SWLM_BUF_SCRATCH1 = 3, /* q, gate, packed B|C|x */
    SWLM_BUF_SCRATCH2 = 4, /* k, up */
    SWLM_BUF_SCRATCH3 = 5, /* v */
    SWLM_BUF_SCRATCH4 = 6,
    SWLM_BUF_LOGITS = 7,
    SWLM_BUF_COUNT = 8
};

/* Step kinds. The comment names the reference kernel each one stands for. */
enum {
    /* embedding_lookup_bf16 — Generator/MetalSourceGenerator+Embedding.swift:3-48.
       hidden[b] = table[token_in[b]]; weight = table [vocab, n] bf16. */
    SWLM_STEP_EMBED = 1,
    /* fused_copy_rms_norm — Primitives/Reduction.swift:74-115 + CopyFragment.
       residual = in; out = bf16(in * rsqrt(mean(in^2)+eps) * (w + weight_bias)). */
    SWLM_STEP_COPY_RMSNORM = 2,
    /* fused_residual_add_copy_rms_norm — Compiler/MetalEntryCollector.swift:143-218.
       h = float(in) + float(residual); residual = bf16(h);
       out = bf16(h * rsqrt(mean(h^2)+eps) * (w + weight_bias)). */
    SWLM_STEP_RESADD_COPY_RMSNORM = 3,
    /* fused_residual_add_rms_norm (final norm): as above without the residual store. */
    SWLM_STEP_RESADD_RMSNORM = 4,
    /* gemv_q4_g64 — Generator/MetalSourceGenerator+Quantized.swift:496-575.
       out[n] = bf16(sum_k (scale*q + zero) * in[k]), fp32 accumulation. */
    SWLM_STEP_QGEMV = 5,
    /* batched_qk_rms_norm_2 — Generator/MetalSourceGenerator+Batched.swift:681-760.
       per-head RMSNorm of q (in_buf, `heads`) with `weight` and of k (in2_buf,
       `kv_heads`) with `weight2`, in place. */
    SWLM_STEP_QK_NORM = 6,
    /* rope_flash_attn_decode — Generator/MetalSourceGenerator+Attention.swift:551-930.
       q = in_buf, k = in2_buf, v = in3_buf, result = out_buf. Inline rotate-half
       RoPE on q and the new k, append k,v at `position`, attend over [0, position]. */
    SWLM_STEP_ATTN_DECODE = 7,
    /* swiglu — Primitives/ElementwiseFragment.swift:49-54.
       out = bf16(g/(1+exp(-g)) * up), g = in_buf, up = in2_buf. */
    SWLM_STEP_SWIGLU = 8,
    /* conv_state_update_bf16 — Generator/MetalSourceGenerator+ConvAndState.swift:27-70.
       in_buf holds B|C|x (3*n); state [conv_kernel][n] bf16; weight [n][conv_kernel] bf16. */
    SWLM_STEP_CONV_STATE_UPDATE = 9,
    /* argmax — Generator/MetalSourceGenerator+Sampling.swift:62-107; lowest index
       wins among equal maxima. token_out[b] = argmax(in_buf[b][0..n)). */
    SWLM_STEP_ARGMAX = 10,
    /* geglu — the gated activation with GELU (tanh approximation) instead of SiLU
       (Generator/MetalSourceGenerator+NormAndElementwise.swift:176-208, GatedActivation.geluTanh):
       out = bf16(0.5 g (1 + tanh(0.7978845608 (g + 0.044715 g^3))) * up), g = in_buf, up = in2_buf. */
    SWLM_STEP_GEGLU = 11,
    /* ssm_recurrence (gated delta rule of the DeltaNet / Qwen3.5 linear-attention layers) —
       Generator/MetalSourceGenerator+ConvAndState.swift:282-500, Primitives/SSMRecurrenceFragment.swift.
       in_buf = projected q|k|v (2*groups*key_dim + heads*value_dim values), in2_buf = z (heads*value_dim),
       in3_buf = beta (heads), in4_buf = alpha (heads), out_buf = heads*value_dim values.
       Per channel: causal conv over conv_kernel taps (state [conv_kernel][conv_dim], weight dtype) + SiLU; per head:
       decay = exp(-exp(A_log) * softplus(alpha + dt_bias)), beta = sigmoid(beta), q and k L2-normalised (q also scaled
       by key_dim^-1/2), S = decay * S + k (x) beta (v - S^T k), out = S^T q (state S [key_dim][value_dim] fp32); then
       RMS norm over value_dim with `weight2` and the gate z * sigmoid(z).
       weight = conv taps [conv_dim][conv_kernel] bf16, weight2 = norm weight [value_dim] fp32, weight3 = dt_bias
       [heads] bf16, weight4 = A_log [heads] fp32 (the two fp32 tensors: swlm_weights_add_dense_f32). */
    SWLM_STEP_SSM_RECURRENCE = 12
};

typedef struct swlm_step {
    int32_t kind;
    int32_t layer;       /* index of the KV-cache / conv-state slab this step owns, else -1 */
    int32_t in_buf;
    int32_t in2_buf;
    int32_t in3_buf;
    int32_t out_buf;
    int32_t n;           /* output width (rows of the weight) / vector dimension */
    int32_t k;           /* input width (columns of the weight) */
    int32_t heads;
    int32_t kv_heads;
    int32_t head_dim;
    int32_t rope_dim;    /* 0 = no RoPE */
    int32_t conv_kernel;
    float   eps;
    float   weight_bias;
    float   scale;       /* attention scale */
    float   rope_base;
    char    weight[SWLM_NAME_MAX];
    char    weight2[SWLM_NAME_MAX];
    /* attention: sliding window. 0 = attend everything; W > 0 = the current token and the W - 1 before it
       (windowLeft, Generator/MetalSourceGenerator+Attention.swift:851-853; decode and prompt chunks alike). */
    int32_t window_left;
    /* SWLM_STEP_SSM_RECURRENCE only */
    int32_t in4_buf;
    int32_t groups;      /* key groups; heads / groups value heads share one q and k */
    int32_t key_dim;
    int32_t value_dim;
    char    weight3[SWLM_NAME_MAX];
    char    weight4[SWLM_NAME_MAX];
} swlm_step;

/* Sizes of the runtime buffer set; mirrors the inputs of
   MetalBufferAllocator.makeDecodeBufferAllocation (Buffer/MetalBufferAllocator.swift:4-132)
   and KVCacheSpecification (Buffer/MetalGraphAllocator.swift:15-223). */
typedef struct swlm_buffers_desc {
    int32_t hidden;       /* hidden size */
    int32_t slot_dim;     /* elements per scratch slot */
    int32_t vocab;
    int32_t max_seq;      /* KV slots per sequence (maximumSequenceLength) */
    int32_t max_batch;    /* sequences decoded together; the reference is 1 */
    int32_t kv_layers;    /* number of attention layers (KV slabs) */
    int32_t kv_heads;
    int32_t head_dim;
    int32_t conv_layers;  /* number of short-conv layers (state slabs) */
    int32_t conv_dim;
    int32_t conv_kernel;
    /* recurrent layers (SWLM_STEP_SSM_RECURRENCE): per layer and sequence a conv state [ssm_conv_kernel][conv_dim]
       (conv_dim = 2*ssm_groups*ssm_key_dim + ssm_heads*ssm_value_dim) and an fp32 state [ssm_heads][ssm_key_dim][ssm_value_dim].
       All zero when the plan has no such layer. */
    int32_t ssm_layers;
    int32_t ssm_heads;
    int32_t ssm_groups;
    int32_t ssm_key_dim;
    int32_t ssm_value_dim;
    int32_t ssm_conv_kernel;
    /* KV cache element scheme (KVCacheSpecification, Buffer/MetalGraphAllocator.swift): 0 or SWLM_KV_BF16 = dense bf16;
       the quantized schemes keep groups of 32 / 64 / 128 values along the head dimension as blocks fp16 scale | fp16 zero
       | payload (8-bit: one byte per value; 4-bit: two values per byte, the even one in the low nibble), value = scale *
       q + zero (kv_quant_bits / _group_size / _bytes_per_block, read_kv_element, write_kv_quantized_q8 / _q4:
       Generator/MetalSourceGenerator+Attention.swift:1894-1956, 2057-2155). K and V use the same scheme; a group may not
       be wider than head_dim. */
    int32_t kv_scheme;
    /* The two rotated schemes (is_rotor_scheme / rotor_base_scheme, :1791-1800) store rows in the block layout of their
       base scheme after every group of three consecutive values of a K or V row was turned by a unit rotor of Cl(3,0)
       (rotor_sandwich, :1807-1813; one rotor per attention layer, KV head and group, ceil(head_dim / 3) groups, the
       last one padded with zeros); q is turned the same way and the attention output turned back
       (rotor_sandwich_inverse, :1815-1821). kv_qjl_dim > 0 (at most 64; rotated schemes only) adds the correction of
       the K quantisation error: per cached row kv_qjl_dim fp16 values Phi . (k_rotated - dequantised row) with the fixed
       +-1/sqrt(kv_qjl_dim) matrix Phi [head_dim][kv_qjl_dim], and every score over a cached row gains
       (Phi . q_rotated) . (that row's values) (qjl_compute_residual, qjl_project_query, qjl_score_correction,
       :1983-2048). */
    int32_t kv_qjl_dim;
} swlm_buffers_desc;

enum {
    SWLM_KV_BF16 = 0x01,
    SWLM_KV_Q8G32 = 0x10, SWLM_KV_Q8G64 = 0x11, SWLM_KV_Q8G128 = 0x12,   /* 36 / 68 / 132 bytes per block */
    SWLM_KV_Q4G64 = 0x40, SWLM_KV_Q4G128 = 0x41, SWLM_KV_Q4G128Z = 0x42, /* 36 / 68 / 68 bytes per block (0x42, the
                                                                            reference's q4Group128ScaleF16Zero, reads and
                                                                            writes cache rows exactly as 0x41 does) */
    SWLM_KV_ROTOR_Q8G32 = 0x70, SWLM_KV_ROTOR_Q4G64 = 0x71               /* rotated rows in the layout of 0x10 / 0x40 */
};
static inline int swlm_kv_is_rotor(int scheme) { return scheme == 0x70 || scheme == 0x71; }
static inline int swlm_kv_base_scheme(int scheme) { return scheme == 0x70 ? 0x10 : scheme == 0x71 ? 0x40 : scheme; }
/* rotors per KV head: groups of three values along the head dimension (KVCacheSpecification.numRotorGroups) */
static inline int swlm_kv_rotor_groups(int head_dim) { return (head_dim + 2) / 3; }
/* bits per value (0: dense), values per group, bytes per block and bytes per row of head_dim values */
static inline int swlm_kv_bits(int scheme) {
    scheme = swlm_kv_base_scheme(scheme);
    return scheme >= 0x10 && scheme <= 0x12 ? 8 : (scheme >= 0x40 && scheme <= 0x42) ? 4 : 0;
}
static inline int swlm_kv_group(int scheme) {
    scheme = swlm_kv_base_scheme(scheme);
    return scheme == 0x10 ? 32 : (scheme == 0x11 || scheme == 0x40) ? 64 : (scheme == 0x12 || scheme == 0x41 || scheme == 0x42) ? 128 : 0;
}
static inline int swlm_kv_block_bytes(int scheme) { return swlm_kv_bits(scheme) ? 4 + swlm_kv_group(scheme) * swlm_kv_bits(scheme) / 8 : 0; }
static inline int swlm_kv_row_bytes(int scheme, int head_dim) {
    return swlm_kv_bits(scheme) ? head_dim / swlm_kv_group(scheme) * swlm_kv_block_bytes(scheme) : head_dim * 2;
}

#ifdef __cplusplus
}
#endif
#endif /* SWLM_PLAN_H */
