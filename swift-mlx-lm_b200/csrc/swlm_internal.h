// Internal declarations shared by the translation units of libswlm_cuda.so.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/swlm.h"
#include "tp_device.cuh"

namespace swlm {

// ---- errors ------------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);  // records the message, returns SWLM_ERR_CUDA
#define SWLM_CUDA(call)                                          \
    do {                                                         \
        cudaError_t e__ = (call);                                \
        if (e__ != cudaSuccess) return ::swlm::cuda_fail(e__, #call); \
    } while (0)

// ---- launches ------------------------------------------------------------------
// Every kernel of the decode step is launched with programmatic stream serialization (programmatic
// dependent launch): a kernel may start while its predecessor drains, does what does not depend on it
// (the GEMV kernels start streaming weights), and executes `griddepcontrol.wait` before it touches
// anything the predecessor wrote. SWLM_NO_PDL=1 in the environment turns the attribute off.
bool pdl_enabled();
template <typename... P, typename... A>
inline cudaError_t launch_k(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, A... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}
#ifdef __CUDACC__
// Wait until the preceding kernel in the stream has completed and its writes are visible.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Allow the next kernel in the stream to begin launching.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// ---- device tensors -----------------------------------------------------------
//
// Q4 group-64 tensor in the streaming layout of the GEMV/GEMM kernels.
//   tiles : uint4[row_tiles][kt_pad][32]   one 512-byte tile = 16 rows x 64 columns,
//           lane (g = lane>>2, t = lane&3) owns 16 bytes = 4 words; word j, nibble e holds
//           W[16*rt + g + 8*(e&1)][64*kt + 16*t + 4*j + (e>>2) + 2*((e>>1)&1)]:
//           the A-fragment order of mma.m16n8k16 for k-step j, with the group's columns assigned to
//           k-steps so that lane t's B fragments are the 16 consecutive activations 16t..16t+15.
//   sb    : uint4[row_tiles][kt_pad/4][16]  per row, four consecutive groups' (scale, zero)
//           pairs, each pair two 16-bit floats (bf16, or fp16 when the source was STAF).
// kt_pad = K/64 rounded up to a multiple of 4; padding tiles hold q = 0, scale = zero = 0.
struct Q4Tiled {
    int n = 0, k = 0;           // logical (per-rank) shape
    int row_tiles = 0;          // ceil(n / 16)
    int kt_pad = 0;             // k-tiles including padding
    bool sb_f16 = false;        // scale/zero stored as fp16 instead of bf16
    bool interleaved = false;   // rows 0-7 of each tile from source A, rows 8-15 from source B
    uint4* tiles = nullptr;
    uint4* sb = nullptr;
    size_t bytes() const { return (size_t)row_tiles * kt_pad * 512 + (size_t)row_tiles * (kt_pad / 4) * 256; }
};

// Raw source copy kept on the device so that fused tensors can be assembled at plan time.
struct Q4Raw {
    int n = 0, k = 0;
    bool sb_f16 = false;
    int shard_kind = 0;
    uint32_t* w = nullptr;      // [n][k/8]
    uint16_t* scales = nullptr; // [n][k/64]
    uint16_t* biases = nullptr;
};

struct DenseTensor {
    int64_t rows = 0, cols = 0;
    int shard_kind = 0;
    __nv_bfloat16* data = nullptr;
};

struct DenseF32 {
    int64_t count = 0;
    float* data = nullptr;
};

// ---- kernels: launch wrappers (each returns a status; no synchronisation) -------

struct RepackSrc {
    const uint32_t* w;
    const uint16_t* scales;
    const uint16_t* biases;
    int n;
};
// Build a tiled tensor from up to three raw sources that share K.
// mode 0: rows concatenated; mode 1: two sources interleaved 8 rows each per tile.
int launch_repack(const RepackSrc* src, int n_src, int mode, int k, const Q4Tiled& dst, cudaStream_t s);
int launch_untile_bf16(const Q4Tiled& t, __nv_bfloat16* out, cudaStream_t s);

enum { QGEMV_EPI_STORE = 0, QGEMV_EPI_SWIGLU = 1 };   // SWIGLU: the gated-activation epilogue (SiLU or GELU, see gated_act)
enum { GATED_ACT_SILU = 0, GATED_ACT_GELU_TANH = 1 };
#ifdef __CUDACC__
// activation(gate) * up of the gated MLP (Generator/MetalSourceGenerator+NormAndElementwise.swift:176-208):
// SiLU for SwiGLU, the tanh approximation of GELU for GEGLU.
__device__ __forceinline__ float gated_activation(float g, float up, int act) {
    const float a = act == GATED_ACT_GELU_TANH ? 0.5f * g * (1.0f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)))
                                               : g * (1.0f / (1.0f + expf(-g)));
    return a * up;
}
#endif

// Weights of a later launch that this launch asks the memory system to bring from HBM into L2 while it runs
// (its own data comes from L2 or is small, so HBM would otherwise idle). Two arrays, sizes multiples of 256.
struct PrefetchTarget {
    const void* p[2] = {nullptr, nullptr};
    unsigned long long bytes[2] = {0, 0};
    // heads > 0: the two arrays are the K and V caches of one layer and sequence; what is requested is the first
    // position[0] rows (row_bytes each) of every head, heads being head_stride bytes apart. The position is only a
    // hint here: a stale value requests a row too few.
    int heads = 0, row_bytes = 0;
    unsigned long long head_stride = 0;
    const int* position = nullptr;
};
#ifdef __CUDACC__
// CTA `part` of `nparts` requests its share, 16 KB per instruction, one instruction per thread and round.
__device__ __forceinline__ void prefetch_target_slice(const PrefetchTarget& t, int part, int nparts, int tid, int nthreads) {
    if (t.heads > 0) {
        // KV rows: 256-byte granules, numbered head-major over both caches
        const unsigned long long per_head = ((unsigned long long)t.position[0] * (unsigned)t.row_bytes) >> 8;
        if (per_head == 0) return;
        const unsigned long long gran = per_head * (unsigned)t.heads * 2ull;
        const unsigned long long g0 = gran * (unsigned long long)part / (unsigned long long)nparts;
        const unsigned long long g1 = gran * (unsigned long long)(part + 1) / (unsigned long long)nparts;
        for (unsigned long long g = g0 + 16ull * tid; g < g1; g += 16ull * nthreads) {  // 4 KB per instruction
            const unsigned long long hd = g / per_head, off = g - hd * per_head;        // head index over both caches
            const unsigned long long run = per_head - off < 16ull ? per_head - off : 16ull;
            const unsigned n = (unsigned)((g1 - g < run ? g1 - g : run) << 8);
            const unsigned char* base = static_cast<const unsigned char*>(t.p[hd >= (unsigned)t.heads ? 1 : 0]) +
                                        (hd % (unsigned)t.heads) * t.head_stride + (off << 8);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base), "r"(n) : "memory");
        }
        return;
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {
        if (!t.p[a]) continue;
        const unsigned long long gran = t.bytes[a] >> 8;
        const unsigned long long g0 = gran * (unsigned long long)part / (unsigned long long)nparts;
        const unsigned long long g1 = gran * (unsigned long long)(part + 1) / (unsigned long long)nparts;
        for (unsigned long long g = g0 + 64ull * tid; g < g1; g += 64ull * nthreads) {
            const unsigned n = (unsigned)((g1 - g < 64ull ? g1 - g : 64ull) << 8);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(static_cast<const unsigned char*>(t.p[a]) + (g << 8)), "r"(n) : "memory");
        }
    }
}
#endif

// Residual add / copy / RMSNorm fused in front of a product (mode = the step kind it replaces, 0 = none).
// x of the launch is then the un-normalised input; res_in and res_out must be different buffers.
struct XNorm {
    int mode = 0;
    const __nv_bfloat16* res_in = nullptr;
    __nv_bfloat16* res_out = nullptr;
    int res_stride = 0;
    const __nv_bfloat16* weight = nullptr;
    float eps = 0.f, weight_bias = 0.f;
};

struct QGemvLaunch {
    const Q4Tiled* w = nullptr;
    XNorm norm;
    int push = 0, in_tp = 0;   // tensor parallel: push partial rows to every rank / consume pushed partials
    TpParams tp{};
    const __nv_bfloat16* x = nullptr;  // [m][x_stride]
    int x_stride = 0;
    // result rows [0, seg_end[0]) go to y[0], [seg_end[0], seg_end[1]) to y[1], ... each [m][y_stride[i]]
    __nv_bfloat16* y[3] = {nullptr, nullptr, nullptr};
    int y_stride[3] = {0, 0, 0};
    int seg_end[3] = {0, 0, 0};
    int m = 1;
    int epilogue = QGEMV_EPI_STORE;
    int gated_act = GATED_ACT_SILU;   // activation of the gated epilogue
    float* partial = nullptr;     // split-K scratch, see qgemv_scratch_floats()
    unsigned* counters = nullptr; // one per CTA row group, zero between launches
    PrefetchTarget prefetch;      // batch-1 kernel only
};
size_t qgemv_scratch_floats(const Q4Tiled& w, int m);
int qgemv_counter_count(const Q4Tiled& w);
int launch_qgemv(const QGemvLaunch& a, cudaStream_t s);
// SWLM_TRACE=1: slot for the phase timestamps of one launch (nullptr when tracing is off or the slots are used up)
unsigned long long* qgemv_trace_slot(int ctas, int row_tiles, int kt4, int epi, int norm);
int qgemv_init();  // sets shared-memory attributes once per process
void qgemv_trace_report();  // SWLM_TRACE=1: phase timeline of the batch-1 launches, to stderr

// rmsnorm family: mode = SWLM_STEP_COPY_RMSNORM / RESADD_COPY_RMSNORM / RESADD_RMSNORM
int launch_rmsnorm(int mode, int m, int dim, const __nv_bfloat16* in, int in_stride, __nv_bfloat16* residual,
                   int res_stride, const __nv_bfloat16* weight, float eps, float weight_bias,
                   __nv_bfloat16* out, int out_stride, cudaStream_t s);
int launch_qk_norm(int m, int heads, int kv_heads, int head_dim, __nv_bfloat16* q, int q_stride,
                   __nv_bfloat16* k, int k_stride, const __nv_bfloat16* wq, const __nv_bfloat16* wk,
                   float eps, float weight_bias, cudaStream_t s);
int launch_embed(int m, int dim, const int32_t* tokens, int vocab, const __nv_bfloat16* table,
                 __nv_bfloat16* out, int out_stride, cudaStream_t s);
// the same gather from a Q4 group-64 table (packed source copy): out = bf16(q * scale + zero)
int launch_embed_q4(int m, int dim, const int32_t* tokens, const Q4Raw& table, __nv_bfloat16* out, int out_stride, cudaStream_t s);
int launch_swiglu(int m, int n, const __nv_bfloat16* gate, int g_stride, const __nv_bfloat16* up, int u_stride,
                  __nv_bfloat16* out, int o_stride, int act, cudaStream_t s);
int launch_conv_step(int m, int dim, int kernel, __nv_bfloat16* state, size_t state_seq_stride,
                     const __nv_bfloat16* in, int in_stride, const __nv_bfloat16* weight,
                     __nv_bfloat16* out, int out_stride, cudaStream_t s);
// conv_state_update over `tokens` consecutive tokens of one sequence (state of that sequence), bit-identical to
// `tokens` single steps.
// One step of the gated delta rule for m sequences (see SWLM_STEP_SSM_RECURRENCE): conv shift + SiLU over the q|k|v
// channels, per-head state update and read-out, RMS norm and z gate. conv_state [m][kernel][conv_dim] bf16 (row pitch
// conv_seq_stride elements per sequence), state [m][heads][key_dim][value_dim] fp32.
struct SsmLaunch {
    int m = 1, heads = 0, groups = 1, key_dim = 0, value_dim = 0, kernel = 0;
    // > 1 (with m == 1): the rows are consecutive prompt tokens of one sequence, walked in order inside the kernel
    // (ssm_recurrence_seq, Generator/MetalSourceGenerator+ConvAndState.swift:502-): the same code as the single step,
    // so a chunk leaves the state repeated decode steps would
    int tokens = 1;
    const __nv_bfloat16* qkv = nullptr; int qkv_stride = 0;
    const __nv_bfloat16* z = nullptr; int z_stride = 0;
    const __nv_bfloat16* beta = nullptr; int beta_stride = 0;
    const __nv_bfloat16* alpha = nullptr; int alpha_stride = 0;
    const __nv_bfloat16* conv_weight = nullptr;   // [conv_dim][kernel]
    const float* norm_weight = nullptr;           // [value_dim]
    const __nv_bfloat16* dt_bias = nullptr;       // [heads]
    const float* a_log = nullptr;                 // [heads]
    __nv_bfloat16* conv_state = nullptr; size_t conv_seq_stride = 0;
    float* state = nullptr; size_t state_seq_stride = 0;
    __nv_bfloat16* out = nullptr; int out_stride = 0;
};
int launch_ssm_recurrence(const SsmLaunch& a, cudaStream_t s);
int launch_conv_prefill(int tokens, int dim, int kernel, __nv_bfloat16* state, const __nv_bfloat16* in, int in_stride,
                        const __nv_bfloat16* weight, __nv_bfloat16* out, int out_stride, cudaStream_t s);
// argmax over [m][n] bf16, lowest index wins. Writes token_out[m], token_in_next[m] (may be null) and
// ring[(step_counter % ring_cap) * m + b] (ring may be null); when advance != 0 the last thread also
// increments the device-side position and step counter. Two launches.
int launch_argmax(int m, int n, const __nv_bfloat16* logits, int stride, int32_t* token_out,
                  int32_t* token_in_next, int32_t* ring, int32_t* step_counter, int ring_cap,
                  int32_t* position, int advance, float* scratch_val, int32_t* scratch_idx, const TpParams& tp,
                  int32_t* am_epoch, int shard_offset, cudaStream_t s);
size_t argmax_scratch_elems(int m);

// Sequences decoded together: 1..16 ride in the GEMV kernels (one weight pass for all of them), 17..kMaxSequences
// take the tensor-core product, one row per sequence.
constexpr int kMaxSequences = 64;
constexpr int kQGemvMaxRows = 16;

struct AttnLaunch {
    int m = 1;            // sequences
    int heads = 0, kv_heads = 0, head_dim = 0;
    int rope_dim = 0;
    const float* inv_freq = nullptr;  // [rope_dim/2] device
    float scale = 1.f;
    const __nv_bfloat16* q = nullptr; int q_stride = 0;   // [m][heads*hd]
    const __nv_bfloat16* k = nullptr; int k_stride = 0;   // new token's k [m][kv_heads*hd]
    const __nv_bfloat16* v = nullptr; int v_stride = 0;
    __nv_bfloat16* kcache = nullptr;  // [m][kv_heads][max_seq][hd]
    __nv_bfloat16* vcache = nullptr;
    int max_seq = 0;
    const int32_t* position = nullptr;  // device array [m]: index of each sequence's new token
    __nv_bfloat16* out = nullptr; int out_stride = 0;
    float* scratch = nullptr;   // attn_scratch_floats()
    unsigned* counters = nullptr;  // m * kv_heads arrival counters, zero between launches
    int splits = 1;             // KV splits per (sequence, kv head)
    // >= 0: prompt ingestion. The m rows are consecutive tokens of sequence 0 starting at this position; their
    // k/v rows are appended first, then token b attends cache rows 0..pos_base+b. `position` is not read.
    int pos_base = -1;
    int window = 0;       // sliding window: the current token and the window - 1 before it; 0 = everything
    int kv_scheme = 0;    // one of the quantized SWLM_KV_* schemes: the cache rows are blocks of 8- or 4-bit values (decode steps only)
    // rotated schemes: this layer's rotors [kv_heads][ceil(head_dim / 3)][4], the projection matrix [head_dim][qjl_dim]
    // and this layer's projected K residuals [m][kv_heads][max_seq][qjl_dim] (qjl_dim 0: no correction)
    const __half* rotors = nullptr;
    const __half* qjl_matrix = nullptr;
    __half* qjl_res = nullptr;
    int qjl_dim = 0;
    PrefetchTarget prefetch;
};
int attn_pick_splits(int m, int kv_heads, int max_ctx);
size_t attn_scratch_floats(int m, int heads, int head_dim, int splits);
// decode: q rows are unrotated; RoPE, KV append and the current token's unrounded term are handled inside.
int launch_attn_decode(const AttnLaunch& a, cudaStream_t s);
// generic flash-decode over an existing cache (q already rotated), ctx_len fixed on the host.
int launch_flash_decode_plain(int m, int heads, int kv_heads, int hd, int ctx_len, int ctx_stride, float scale,
                              const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                              __nv_bfloat16* out, float* scratch, unsigned* counters, int splits, cudaStream_t s);
int attn_init();
size_t flash_decode_static_capacity();
int launch_flash_decode_static(int device, int m, int heads, int kv_heads, int hd, int ctx_len, int ctx_stride, float scale,
                               const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, __nv_bfloat16* out,
                               cudaStream_t s);

// Tensor-core (tcgen05) form of the quantised product for m >= kQGemmTcMinRows, fed from the packed source copy.
constexpr int kQGemmTcMinRows = 17;   // 17..63 token rows ride in a 64-token tile whose other rows are zero
int qgemm_tc_init();
size_t qgemm_tc_scratch_bytes(int m, int k);   // fp16 copy of the activations + one float per token row
// kernels one call of launch_qgemm_tc issues: the fp16 copy of the rows (unless reused), the product, and the sum over
// K ranges when a short launch is split
int qgemm_tc_launch_count(const Q4Raw& w, int m, bool reuse_x);
// Where the rows of a product over concatenated weights go: rows [end[q-1], end[q]) to y[q] (up to three outputs,
// e.g. q | k | v); null = all rows to `y`.
struct TcSegments {
    int count = 1;
    int end[3] = {0, 0, 0};
    __nv_bfloat16* y[3] = {nullptr, nullptr, nullptr};
    int stride[3] = {0, 0, 0};
};
int launch_qgemm_tc(const Q4Raw& w, int m, const __nv_bfloat16* x, int x_stride, __nv_bfloat16* y, int y_stride,
                    void* scratch, int* status, cudaStream_t s, bool reuse_x = false, const TcSegments* segments = nullptr);

// Tensor-parallel sum of `rows` bf16 partial rows (prompt chunks): every rank copies its partials into every rank's
// exchange buffer and raises a flag carrying `epoch` (the host counts exchanges); then each rank waits (bounded) for
// all flags and adds the partials in rank order into `x` (in place). Two launches.
int launch_tp_rows_allreduce(const TpParams& tp, __nv_bfloat16* x, int x_stride, int rows, int hidden, int epoch,
                             unsigned* done_counter, cudaStream_t s);
int launch_fill_u32(uint32_t* p, size_t n, uint32_t v, cudaStream_t s);
int launch_advance(int m, int32_t* position, int32_t* step_counter, cudaStream_t s);

}  // namespace swlm
