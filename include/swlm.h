/*
 * swlm.h — C ABI of libswlm_cuda.so, a CUDA (sm_100a) dispatch-plan backend for
 * swift-lm's 4-bit decode/prefill hot path.
 *
 * The reference has no FFI of its own: its seams are Swift types. Each entry
 * point below names the Swift interface it stands in for (paths relative to the
 * reference project root).
 *
 * Conventions: every function returns 0 (SWLM_OK) or a negative status and never
 * throws or aborts; the message for the last failure is read with
 * swlm_last_error(). Weights belong to a `swlm_ctx` and are immutable and shared;
 * runtime buffers belong to a `swlm_state`, one per generation context, and a
 * state must not be used from two threads at once (the reference gives every
 * LanguageModelContext its own clone of the runtime buffers —
 * Sources/MetalCompiler/Execution/MetalCompiledModelRuntimeIsolation.swift:28-110).
 * There is no CPU fallback: without a CUDA device every call that needs one fails.
 */
#ifndef SWLM_H
#define SWLM_H

#include <stddef.h>
#include <stdint.h>

#include "swlm_plan.h"

#ifdef __cplusplus
extern "C" {
#endif

#define SWLM_OK 0
#define SWLM_ERR_INVALID (-1)     /* bad argument / shape */
#define SWLM_ERR_CUDA (-2)        /* a CUDA runtime call failed */
#define SWLM_ERR_NOT_FOUND (-3)   /* tensor name not in the weight store */
#define SWLM_ERR_UNSUPPORTED (-4) /* step kind / format outside the hot path */
#define SWLM_ERR_TIMEOUT (-5)     /* a bounded device-side wait expired */
#define SWLM_ERR_STATE (-6)       /* call not valid in the current state */

/* How a tensor is cut when ctx was created with tp_size > 1 (Megatron style). */
#define SWLM_SHARD_REPLICATE 0
#define SWLM_SHARD_COLUMN 1 /* split output rows N; result stays sharded */
#define SWLM_SHARD_ROW 2    /* split input columns K on 64-element group boundaries; result needs an all-reduce */
#define SWLM_SHARD_COLUMN3 3 /* N = three equal thirds (B|C|x of LFM2 in_proj), each split on its own: a rank holds
                               rows [row0, row0 + rows) of every third, one third after the other */

typedef struct swlm_ctx swlm_ctx;
typedef struct swlm_plan swlm_plan;
typedef struct swlm_state swlm_state;
typedef struct swlm_snap swlm_snap;

const char* swlm_version(void);
int swlm_device_count(void);
/* Message of the most recent failure on this thread. */
const char* swlm_last_error(void);

/* ---- context + weight store ------------------------------------------------
 * Replaces STAFLoader.load(at:device:) -> STAFWeightStore
 * (Sources/MetalCompiler/STAF/STAFLoader.swift:19-198, :213-299): a name ->
 * device tensor map. Quantized tensors are re-tiled once, at upload, into the
 * layout the GEMV kernels stream. */
int swlm_ctx_create(int device_id, int tp_rank, int tp_size, swlm_ctx** out);
/* Plans keep their context alive and states their plan: destroying an object that still has users is deferred
 * until the last of them is destroyed, so wrappers may release context, plan and state in any order. */
void swlm_ctx_destroy(swlm_ctx* ctx);

/* MLX affine source format: weight u32[n][k/8] (8 nibbles per word, LSB first
 * along K), scales/biases bf16 [n][k/64]
 * (Sources/MetalCompiler/STAF/STAFPayloadConverter.swift:209-282). */
int swlm_weights_add_q4g64_mlx(swlm_ctx* ctx, const char* name, int n, int k, const uint32_t* weight,
                               const uint16_t* scales_bf16, const uint16_t* biases_bf16, int shard_kind);
/* STAF execution blocks, 36 bytes per 64 weights: fp16 scale | fp16 zero | 32 payload bytes
 * (Sources/MetalCompiler/STAF/QuantizationFormat.swift:463-528). */
int swlm_weights_add_q4g64_staf(swlm_ctx* ctx, const char* name, int n, int k, const void* blocks36,
                                int shard_kind);
/* The same two formats with one scale / bias pair per 128 weights (AffineQ4Group128Format,
 * Sources/MetalCompiler/STAF/QuantizationFormat.swift:539-604): MLX scales/biases are [n][k/128], STAF blocks are
 * 68 bytes (fp16 scale | fp16 zero | 64 payload bytes). On the device the tensor takes the group-64 streaming layout
 * with every pair written for both halves of its group, so all kernels serve it unchanged and results are those of
 * w = scale * q + zero with the group-128 parameters; 0.5625 bytes per weight are streamed instead of 0.53125. */
int swlm_weights_add_q4g128_mlx(swlm_ctx* ctx, const char* name, int n, int k, const uint32_t* weight,
                                const uint16_t* scales_bf16, const uint16_t* biases_bf16, int shard_kind);
int swlm_weights_add_q4g128_staf(swlm_ctx* ctx, const char* name, int n, int k, const void* blocks68,
                                 int shard_kind);
/* Dense bf16 tensor (norm weights, embedding table, conv weights). `count` elements;
 * rows/cols describe a 2-D view when shard_kind != replicate (cols = count / rows). */
int swlm_weights_add_dense_bf16(swlm_ctx* ctx, const char* name, int64_t rows, int64_t cols,
                                const uint16_t* data, int shard_kind);
/* Dense fp32 tensor, replicated: the recurrent layers' norm weight and A_log, which the reference keeps in fp32
 * whatever the bundle's dtype (STAF/STAFConversionPlanner.swift:117-127). */
int swlm_weights_add_dense_f32(swlm_ctx* ctx, const char* name, int64_t count, const float* data);
/* Total bytes of weights resident on the device for this context. */
int64_t swlm_weights_bytes(const swlm_ctx* ctx);

/* ---- plan --------------------------------------------------------------------
 * Replaces MetalInferenceCompiler.compile(...) -> MetalCompiledModel.decodePlan
 * (Sources/MetalCompiler/Compiler/MetalInferenceCompiler.swift:520-615) and
 * MetalDispatchStepBuilder.buildDecodePlan (Compiler/MetalDispatchStepBuilder.swift:4-105):
 * resolves tensor names, fuses adjacent steps into launches and sizes the buffer set. */
int swlm_plan_build(swlm_ctx* ctx, const swlm_step* steps, int n_steps, const swlm_buffers_desc* desc,
                    swlm_plan** out);
void swlm_plan_destroy(swlm_plan* plan);
/* Number of kernel launches one decode step issues after fusion. */
int swlm_plan_launch_count(const swlm_plan* plan);
/* Human-readable launch list, the counterpart of the reference's decode diagnostics
 * (Execution/MetalDecodePlan.swift:122-133). Returns bytes needed, copies at most cap. */
int swlm_plan_describe(const swlm_plan* plan, char* dst, int cap);

/* ---- runtime state -------------------------------------------------------------
 * Replaces MetalInferenceModel(plan:device:) and its buffer set
 * (Sources/MetalCompiler/Execution/MetalInferenceModel.swift; MetalDecodePlan.swift MetalBufferSet). */
int swlm_state_create(swlm_plan* plan, swlm_state** out);
void swlm_state_destroy(swlm_state* state);
/* Launch on this CUDA stream (a cudaStream_t) instead of the state's own. */
int swlm_state_set_stream(swlm_state* state, void* cuda_stream);
/* Prompt ingestion (swlm_prefill) runs the prompt in chunks of up to `tokens` tokens with one activation row per
 * token and the products on the tensor cores, as the reference's sequence prefill does
 * (Execution/MetalPrefillExecutor.swift); the last prompt token always takes the decode path. 0 = one token at a
 * time through the decode graph. Default 2048. Chunking applies to single-sequence states (under tensor parallelism
 * in chunks of at most 1024 tokens, whose partial rows are summed across the ranks) and, on one GPU, to the sequences
 * of a batch one after the other; other cases ingest token by token through the decode graph. */
int swlm_state_set_prefill_chunk(swlm_state* state, int tokens);
/* resetState() — MetalInferenceModel.swift:1911. */
int swlm_state_reset(swlm_state* state);
/* promptSnapshot / restore — Execution/MetalPromptStateStore.swift:5-137. */
int swlm_state_snapshot(swlm_state* state, swlm_snap** out);
int swlm_state_restore(swlm_state* state, const swlm_snap* snap);
void swlm_snap_destroy(swlm_snap* snap);
/* `position` — MetalInferenceModel.swift:9. */
int swlm_position(const swlm_state* state);

/* prefill(tokens:) -> first generated token — MetalInferenceModel.swift:464-526.
 * tokens is [max_batch][n] int32 on the host; first_token receives max_batch values.
 * Returns a negative status on failure and sets first_token[*] = -1 (the reference
 * signals a failed submission with token -1, Execution/MetalDecodeExecutor.swift:33-42). */
int swlm_prefill(swlm_state* state, const int32_t* tokens, int n, int32_t* first_token);
/* decode(tokenID:) -> next token — MetalInferenceModel.swift:311-322,
 * Execution/MetalDecodeExecutor.swift:7-43. One host round trip per token, as in the reference. */
int swlm_decode(swlm_state* state, const int32_t* token_in, int32_t* token_out);
/* n greedy steps without host round trips: token_out of step i feeds step i+1 on the
 * device. tokens_out is [n][max_batch]. No counterpart in the reference, which
 * synchronises every token (Execution/MetalSubmissionContext.swift:56-124). */
int swlm_decode_n(swlm_state* state, const int32_t* token_in, int n, int32_t* tokens_out);
/* Same loop, enqueue only: tokens stay in a device ring, read later with swlm_read_tokens. */
int swlm_decode_n_async(swlm_state* state, const int32_t* token_in_or_null, int n);
int swlm_read_tokens(swlm_state* state, int n, int32_t* tokens_out);
int swlm_sync(swlm_state* state);
/* decodePlan.buffers.logits for host-side sampling
 * (Sources/SwiftLM/LanguageModelContext.swift:2197-2209): bf16 [max_batch][vocab]. */
int swlm_read_logits(swlm_state* state, uint16_t* dst, size_t count);
/* Copy a logical buffer (SWLM_BUF_*) to the host: [max_batch][count_per_row] bf16.
 * Counterpart of the reference's binding probes (MetalInferenceModel.swift:59-62). */
int swlm_read_buffer(swlm_state* state, int buf, uint16_t* dst, int count_per_row);
int swlm_write_buffer(swlm_state* state, int buf, const uint16_t* src, int count_per_row);
/* K (which=0) or V (which=1) rows [count][head_dim] bf16 of one KV slab / sequence / head. */
int swlm_read_kv(swlm_state* state, int which, int layer, int b, int head, int count, uint16_t* dst);
int swlm_write_kv(swlm_state* state, int which, int layer, int b, int head, int count, const uint16_t* src);
/* Rotated KV schemes (SWLM_KV_ROTOR_*). The probes above speak the model's basis: swlm_write_kv turns the rows before
 * it quantises them (K rows also get their projected residuals when kv_qjl_dim > 0), swlm_read_kv turns the
 * dequantised rows back. The rotors are [kv_layers][kv_heads][swlm_kv_rotor_groups(head_dim)][4] fp16 values
 * (s, b12, b13, b23), filled at state creation by the reference's deterministic rule (MetalKVCache.
 * initializeRandomUnitRotors, Buffer/MetalGraphAllocator.swift:349-390; the reference keeps them in a CPU-writable
 * buffer); swlm_state_set_rotors replaces all of them and must be called before the first row is cached.
 * swlm_read_qjl copies the projected K residuals [count][kv_qjl_dim] fp16 of one KV slab / sequence / head
 * (qjlResidualK, :268-272). */
int swlm_state_get_rotors(swlm_state* state, uint16_t* dst, size_t count);
/* 1 when swlm_plan_build accepts `scheme` as swlm_buffers_desc.kv_scheme (0 = unset = bf16), else 0: the counterpart of
 * QuantizationSchemeIdentifier.isSupportedForKVCache (the reference's set also holds dense fp16 0x00 and fp32 0x02
 * caches, which this library, whose activations are bf16, does not offer; note that 0 means "unset" here, not fp16).
 * Needs no device. */
int swlm_kv_scheme_supported(int scheme);
int swlm_state_set_rotors(swlm_state* state, const uint16_t* src, size_t count);
int swlm_read_qjl(swlm_state* state, int layer, int b, int head, int count, uint16_t* dst);
int swlm_read_conv(swlm_state* state, int layer, int b, uint16_t* dst);
/* fp32 recurrent state [ssm_heads][ssm_key_dim][ssm_value_dim] of one recurrent layer / sequence. */
int swlm_read_ssm_state(swlm_state* state, int layer, int b, float* dst);
/* Sets the position of every sequence. */
int swlm_set_position(swlm_state* state, int position);

/* ---- several sequences per step, each at its own position ------------------------
 * The reference decodes one sequence (its decode plan has one position, MetalInferenceModel.swift:9); a state with
 * max_batch > 1 holds max_batch independent sequences (own KV rows, conv state and position) that advance together,
 * one token each per decode step: 2..16 of them share one pass over the weights in the GEMV kernels, 17..64 take
 * the tensor-core product with one row per sequence (single GPU). Every slot decodes on every step; a slot
 * nobody uses is parked by swlm_state_reset_seq before it reaches max_seq. */
int swlm_set_positions(swlm_state* state, const int32_t* positions);      /* [max_batch] */
int swlm_get_positions(const swlm_state* state, int32_t* positions);      /* [max_batch] */
/* Appends n prompt tokens to sequence `seq` alone, starting at that sequence's position (chunks on the tensor
 * cores, the output head on the last token's row) and returns its next token, which is also left in the device-side
 * input slot of that sequence; the other sequences are not touched. Single-GPU plans whose steps can run row-wise. */
int swlm_prefill_seq(swlm_state* state, int seq, const int32_t* tokens, int n, int32_t* first_token);
/* Position 0 and a cleared short-conv state for one sequence. */
int swlm_state_reset_seq(swlm_state* state, int seq);
/* Execute one plan step on the current buffers (kernel-level parity tests). */
int swlm_run_step(swlm_state* state, const swlm_step* step, const int32_t* token_in, int32_t* token_out);
/* Kernel launches issued by this state since creation. */
int64_t swlm_launches(const swlm_state* state);
/* Enqueue, `repeats` times, only the launches that one step kind compiled to (SWLM_STEP_QGEMV,
 * SWLM_STEP_ATTN_DECODE or SWLM_STEP_RESADD_COPY_RMSNORM), in plan order, without advancing the position.
 * The per-kernel timing hook of the benchmark; counterpart of decodeSyncTimed
 * (Sources/MetalCompiler/Execution/MetalDecodeExecutor.swift). */
int swlm_profile_kind(swlm_state* state, int step_kind, int repeats);

/* ---- tensor parallel: one process per GPU, tp_size of them ----------------------------------------------
 * No counterpart in the reference (single device). Each rank creates its context with (tp_rank, tp_size),
 * uploads the full tensors with a shard kind (the library keeps its slice), builds the same plan and state,
 * then: swlm_tp_export -> exchange the 64-byte handles between the processes (any transport; the harness
 * uses torch.distributed) -> swlm_tp_attach with all handles in rank order -> a barrier -> decode as usual.
 * Row-parallel products push their partial sums into every rank's exchange buffer over NVLink and the next
 * product adds them up in its prologue; the vocabulary-sharded argmax is exchanged the same way. Every device
 * wait is bounded: if a rank does not arrive, the call that was producing tokens (swlm_decode, swlm_read_tokens /
 * swlm_decode_n, swlm_prefill, swlm_sync) returns SWLM_ERR_TIMEOUT with token -1 instead of hanging, and so does
 * swlm_tp_status. After a timeout the ranks' exchange counters no longer agree: destroy the state and create a new
 * one on every rank before decoding again. */
#define SWLM_TP_HANDLE_BYTES 64
int swlm_tp_export(swlm_state* state, void* handle_out);
int swlm_tp_attach(swlm_state* state, const void* handles);
int swlm_tp_status(swlm_state* state);
/* Rank-local slice {row0, rows, col0, cols} of an n x k tensor under a SWLM_SHARD_* kind (host only). */
int swlm_shard_range(int shard_kind, int n, int k, int tp_rank, int tp_size, int* out4);
/* Can `heads` query heads over `kv_heads` KV heads be cut into tp_size equal shards (host only)? Both counts must be
 * multiples of tp_size and every rank must keep whole GQA groups; otherwise SWLM_ERR_UNSUPPORTED. swlm_plan_build
 * applies the same check to every attention and QK-norm step. */
int swlm_tp_check_heads(int heads, int kv_heads, int tp_size);

/* ---- op-level entry points (host buffers; copies are part of the call) ----------
 * Y[m][n] = bf16(X[m][k] . W^T): gemv_q4_g64 for m = 1
 * (Generator/MetalSourceGenerator+Quantized.swift:496-575), gemm_q4_g64 for m > 1 (:88-156). */
int swlm_op_qgemm(swlm_ctx* ctx, const char* weight, int m, const uint16_t* x_bf16, uint16_t* y_bf16);
/* Device-pointer form: x [m][k] and y [m][n] bf16 already resident; enqueued on
 * `cuda_stream` (NULL = the context's stream) without synchronising. */
int swlm_op_qgemm_dev(swlm_ctx* ctx, const char* weight, int m, const void* x_dev, void* y_dev,
                      void* cuda_stream);
/* generateUnifiedDequantToBFloat (Generator/MetalSourceGenerator+Quantized.swift:361-416):
 * the stored tensor unpacked to bf16 [n][k] on the host, from the device layout. */
int swlm_op_dequant_bf16(swlm_ctx* ctx, const char* weight, uint16_t* out_bf16);
/* Flash-decode over caller-provided device tensors: q [b][heads][hd] (RoPE already applied),
 * k,v [b][kv_heads][ctx_stride][hd] bf16, attends over [0, ctx_len); out [b][heads][hd] bf16.
 * scratch_dev needs swlm_op_flash_decode_scratch_bytes(). */
size_t swlm_op_flash_decode_scratch_bytes(int b, int heads, int kv_heads, int hd, int ctx_len);
int swlm_op_flash_decode_dev(swlm_ctx* ctx, int b, int heads, int kv_heads, int hd, int ctx_len,
                             int ctx_stride, float scale, const void* q_dev, const void* k_dev,
                             const void* v_dev, void* out_dev, void* scratch_dev, void* cuda_stream);

/* Flash-decode that allocates nothing. No counterpart in the reference.
 * For callers that are not allowed to allocate device memory while running: a serving process that
 * reserved its whole budget at start-up and forbids later cudaMalloc (it synchronises the device and may
 * fail under pressure), or an embedder whose runtime owns the allocator. Same arguments and result as
 * swlm_op_flash_decode_dev, but the split kernel's partials and arrival counters live in an 8 MiB array
 * built into the library (held by every GPU that loads it, until the process exits) instead of in scratch
 * the caller or the library allocates; the call issues no cudaMalloc/cudaFree.
 * Limits and rules: a request whose scratch need exceeds swlm_op_flash_decode_noalloc_capacity() bytes
 * (roughly batch x heads x splits x (head_dim + 2) x 4) is rejected with SWLM_ERR_INVALID. The first call on
 * a device resolves the array's device address; make that first call before any stream capture. All calls
 * share the array: it keeps the last call's contents (the counters are cleared on the call's stream before
 * each launch), and two calls that overlap on the GPU race on it — keep them ordered. */
size_t swlm_op_flash_decode_noalloc_capacity(void);
int swlm_op_flash_decode_noalloc_dev(swlm_ctx* ctx, int b, int heads, int kv_heads, int hd, int ctx_len,
                                     int ctx_stride, float scale, const void* q_dev, const void* k_dev,
                                     const void* v_dev, void* out_dev, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* SWLM_H */
