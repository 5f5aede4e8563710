// Flash-decode GQA attention over a bf16 KV cache for sm_100a.
//
// Replaces `rope_flash_attn_decode` (Generator/MetalSourceGenerator+Attention.swift:551-930): the
// reference runs one 32-thread group per query head that walks the context sequentially and re-reads
// the K/V rows of a GQA group once per query head. Here
//   * the KV range is split across CTAs (flash-decode); the last CTA of a (sequence, KV head) to finish
//     merges the partial (max, sum, output) triples, so the whole step is one launch;
//   * one CTA serves all query heads of a KV head, so K/V are read once per group;
//   * QK^T and PV run on the tensor cores (mma.m16n8k16, bf16 in, fp32 accumulate) with the head
//     dimension permuted so that every lane fetches K and V with 128-bit loads and no shared memory:
//     the contraction over d is order-independent, and for PV two tokens' values of one dimension are
//     paired into a B-fragment register with one PRMT;
//   * q is rotated (RoPE) in fp32 and fed to the tensor core as a bf16 hi + lo pair, so it keeps
//     ~16 bits of mantissa (the reference keeps the rotated q in fp32);
//   * the current token is not read back from the cache: the merging CTA adds its term in fp32 from
//     the unrounded rotated k and v, exactly as the reference does (:866-868, :905-907), while the
//     bf16-rounded copy is appended to the cache for later steps (:761-805).
//   * blocks of 64 tokens are dealt to the splits round-robin, so a split's first block does not depend on the
//     context length: in a decode step it is requested before the device-resident position has arrived, and
//     the split's later blocks are asked into L2 as soon as it has; q, k and v of the new token are requested
//     before any of that, and each RoPE pair is rotated once in shared memory.
// Prompt chunks use a tiled causal kernel further down (attn_prefill_kernel).
#include <atomic>
#include <cstdlib>
#include <cmath>

#include "swlm_internal.h"

namespace swlm {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kSplitWarps = 4;
constexpr int kSplitThreads = kSplitWarps * 32;
constexpr int kMaxGroup = 8;  // query heads per KV head served by one CTA

struct AttnParams {
    int heads, kv_heads, rope_dim, max_seq, splits;
    float scale_log2;  // attention scale * log2(e)
    const float* inv_freq;
    const __nv_bfloat16* q; int q_stride;
    const __nv_bfloat16* k; int k_stride;
    const __nv_bfloat16* v; int v_stride;
    __nv_bfloat16* kcache;
    __nv_bfloat16* vcache;
    size_t cache_seq_stride;   // elements between sequences
    size_t cache_head_stride;  // elements between KV heads
    const int32_t* position;   // decode: device array, one entry per sequence; plain: nullptr
    int ctx_len;               // plain: number of cached tokens
    int pos_base;              // prompt ingestion: position of the chunk's first token
    int chunk_tokens;          // prompt ingestion: tokens in the chunk
    int window;                // sliding window (0 = none): a token attends itself and the window - 1 rows before it
    int kv_bits, kv_group;     // quantized cache: bits per value (8 or 4) and values per block (32, 64 or 128)
    int q_first;               // 1: the first K/V rows are requested only after q, k, v have arrived
    __nv_bfloat16* out; int out_stride;
    float* part_o;   // [m][heads][splits][HD]
    float* part_ml;  // [m][heads][splits][2]
    unsigned* counters;  // [m][kv_heads], zero between launches
    PrefetchTarget prefetch;  // weights of a later product, requested into L2 while this kernel runs
    unsigned long long* trace;  // SWLM_TRACE=1: [cta][4] = entry, predecessor complete, loop done, partials published
    // rotated cache schemes: this layer's rotors [kv_heads][ceil(HD / 3)][4] fp16, the projection matrix
    // [HD][qjl_dim] fp16 and this layer's projected K residuals [m][kv_heads][max_seq][qjl_dim] fp16 (qjl_dim 0: none)
    const __half* rotors;
    const __half* qjl_matrix;
    __half* qjl_res;
    int qjl_dim;
};

__device__ __forceinline__ unsigned long long attn_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ uint4 ldg128(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// rotate-half RoPE of element d of a vector held in shared memory
// (Generator/MetalSourceGenerator+Attention.swift:596-617): pairs (i, i + ropeDim/2).
__device__ __forceinline__ float rope_elem(const float* v, int d, int rope_dim, const float* cs, const float* sn) {
    const int pairs = rope_dim >> 1;
    if (d < pairs) return v[d] * cs[d] - v[d + pairs] * sn[d];
    if (d < rope_dim) return v[d - pairs] * sn[d - pairs] + v[d] * cs[d - pairs];
    return v[d];
}

// MODE 0: plain flash-decode over an existing cache (q already rotated, context length from the host).
// MODE 1: decode step: sequence b at the device-resident position; rotates q and the new k, appends k/v to the
//         cache and adds the new token's own term from the unrounded values.
// MODE 2: prompt ingestion: "sequence" b is prompt token b of ONE sequence at position pos_base + b; all of the
//         chunk's k/v rows are already in the cache (rope_append_kernel), token b attends rows 0..pos_base+b.
template <int HD, int MODE>
__global__ void __launch_bounds__(kSplitThreads) attn_split_kernel(const AttnParams p) {
    constexpr bool DECODE = MODE == 1;
    constexpr bool PREFILL = MODE == 2;
    const int cta_linear = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    if (p.trace && threadIdx.x == 0) p.trace[cta_linear * 4] = attn_timer_ns();
    pdl_launch_dependents();
    if (DECODE)
        prefetch_target_slice(p.prefetch, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x,
                              gridDim.x * gridDim.y * gridDim.z, threadIdx.x, kSplitThreads);
    constexpr int NCH = HD / 32;  // 16-byte K chunks per lane per token
    constexpr int VH = HD / 64;   // 64-dimension halves of V
    constexpr int VPR = HD / 8;   // 16-byte vectors per head row
    constexpr int PITCH = HD + 2; // row pitch of q in shared memory: the 8-byte fragment reads below hit 16 different bank pairs
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int G = p.heads / p.kv_heads;
    const bool rotate = (DECODE || PREFILL) && p.rope_dim > 0;
    // rotation: this thread owns the pairs (i, i + rope_dim/2) of rows tid / (HD/2), + kSplitThreads / (HD/2), ...;
    // its frequency is a constant of the model and is fetched before the predecessor has finished
    const int pairs = p.rope_dim >> 1;
    const int rot_i = tid & (HD / 2 - 1);
    float inv_f = 0.f;
    if (rotate && rot_i < pairs) inv_f = __ldg(p.inv_freq + rot_i);
    pdl_wait();
    if (p.trace && threadIdx.x == 0) p.trace[cta_linear * 4 + 1] = attn_timer_ns();

    __shared__ __align__(16) float qk[kMaxGroup + 1][PITCH];  // rows 0..G-1: q of the group, row G: the new k
    __shared__ float vraw[HD];                                // new v
    __shared__ float self_score[kMaxGroup];                   // q . k of the new token, log2 domain
    __shared__ float osm[kSplitWarps][kMaxGroup][HD + 4];
    __shared__ float msm[kSplitWarps][kMaxGroup], lsm[kSplitWarps][kMaxGroup];

    // ---- q and the new k and v are requested first: they do not depend on the position --------------------
    uint4 qv = make_uint4(0, 0, 0, 0), kv = qv, vv = qv;
    const bool has_q = tid < G * VPR;
    const bool has_k = DECODE && tid >= 64 && tid < 64 + VPR;
    const bool has_v = DECODE && tid >= 96 && tid < 96 + VPR;
    if (has_q) qv = *reinterpret_cast<const uint4*>(p.q + (size_t)b * p.q_stride + (size_t)kvh * G * HD + (size_t)tid * 8);
    if (has_k) kv = *reinterpret_cast<const uint4*>(p.k + (size_t)b * p.k_stride + (size_t)kvh * HD + (size_t)(tid - 64) * 8);
    if (has_v) vv = *reinterpret_cast<const uint4*>(p.v + (size_t)b * p.v_stride + (size_t)kvh * HD + (size_t)(tid - 96) * 8);

    // cached tokens to attend (in a decode step the new token is not among them)
    const int n_ctx = DECODE ? p.position[b] : PREFILL ? p.pos_base + b + 1 : p.ctx_len;
    const int rope_pos = PREFILL ? p.pos_base + b : n_ctx;

    const __nv_bfloat16* kbase = p.kcache + (PREFILL ? 0 : (size_t)b * p.cache_seq_stride) + (size_t)kvh * p.cache_head_stride;
    const __nv_bfloat16* vbase = p.vcache + (PREFILL ? 0 : (size_t)b * p.cache_seq_stride) + (size_t)kvh * p.cache_head_stride;

    // ---- tokens of this split: blocks of 64 tokens, block j belongs to split j % splits. A split's first block
    // does not depend on the context length, so in a decode step it is requested before the position has arrived
    // (rows are clamped to the cache's last row there; what lies beyond the context is masked below).
    constexpr int kBlock = kSplitWarps * 16;
    const int t_begin = split * kBlock;
    const int t_end = n_ctx;
    const int t_stride = p.splits * kBlock;

    // K and V of 16 tokens per warp live in registers; the first batch is requested before the rest of the
    // prologue so that its trip to HBM overlaps it
    uint4 kreg[2][NCH];
    uint4 va[VH], vb[VH], vc[VH], vd[VH];
    auto load_k = [&](int tok0, int last) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const __nv_bfloat16* rowp = kbase + (size_t)min(tok0 + 8 * nt + g, last) * HD;
#pragma unroll
            for (int i = 0; i < NCH; ++i) kreg[nt][i] = ldg128(rowp + (4 * i + t) * 8);
        }
    };
    auto load_v = [&](int tok0, int last) {
        const __nv_bfloat16* ra = vbase + (size_t)min(tok0 + 2 * t, last) * HD + 8 * g;
        const __nv_bfloat16* rb = vbase + (size_t)min(tok0 + 2 * t + 1, last) * HD + 8 * g;
        const __nv_bfloat16* rc = vbase + (size_t)min(tok0 + 2 * t + 8, last) * HD + 8 * g;
        const __nv_bfloat16* rd = vbase + (size_t)min(tok0 + 2 * t + 9, last) * HD + 8 * g;
#pragma unroll
        for (int hh = 0; hh < VH; ++hh) {
            va[hh] = ldg128(ra + 64 * hh); vb[hh] = ldg128(rb + 64 * hh);
            vc[hh] = ldg128(rc + 64 * hh); vd[hh] = ldg128(rd + 64 * hh);
        }
    };
    int tok0 = t_begin + warp * 16;
    if (p.q_first) { /* requested below, once q, k and v are in shared memory */ }
    else if (DECODE) { load_k(tok0, p.max_seq - 1); load_v(tok0, p.max_seq - 1); }
    else if (tok0 < t_end) { load_k(tok0, t_end - 1); load_v(tok0, t_end - 1); }
    // sliding window (Generator/MetalSourceGenerator+Attention.swift:851-853): cached rows below t_lo are left out.
    // A split whose first blocks lie wholly below the window starts at its first block that reaches into it.
    const int t_lo = p.window > 0 ? max(0, n_ctx + (DECODE ? 1 : 0) - p.window) : 0;
    if (t_lo / kBlock > split) {
        const int skip = (t_lo / kBlock - split + p.splits - 1) / p.splits;
        tok0 = (split + skip * p.splits) * kBlock + warp * 16;
        if (!p.q_first && tok0 < t_end) { load_k(tok0, t_end - 1); load_v(tok0, t_end - 1); }
    }
    // the split's later blocks are asked into L2 (two ahead; the loop keeps that distance): the register loads
    // of the loop then find them there
    constexpr int kAhead = 2;
    auto prefetch_block = [&](int blk_tok) {
        if (blk_tok >= t_end) return;
        const unsigned bytes = (unsigned)(min(kBlock, t_end - blk_tok) * HD * 2);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(kbase + (size_t)blk_tok * HD), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(vbase + (size_t)blk_tok * HD), "r"(bytes) : "memory");
    };
    if (tid < kAhead) prefetch_block(t_begin + (tid + 1) * t_stride);

    // ---- prologue: q, k, v to shared memory as floats; then every pair is rotated once, in place ----------
    float rot_s = 0.f, rot_c = 1.f;
    if (rotate && rot_i < pairs) sincosf((float)rope_pos * inv_f, &rot_s, &rot_c);
    {
        auto spill8 = [](float* dst, const uint4& w) {  // dst is 8-byte aligned
            const unsigned u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *reinterpret_cast<float2*>(dst + 2 * j) = make_float2(__uint_as_float(u[j] << 16), __uint_as_float(u[j] & 0xffff0000u));
        };
        if (has_q) spill8(&qk[tid / VPR][(tid % VPR) * 8], qv);
        if (has_k) spill8(&qk[G][(tid - 64) * 8], kv);
        if (has_v) {
            const unsigned u[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) { vraw[(tid - 96) * 8 + 2 * j] = __uint_as_float(u[j] << 16); vraw[(tid - 96) * 8 + 2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u); }
            if (split == 0 && n_ctx < p.max_seq)  // the new v row goes to the cache as it is
                *reinterpret_cast<uint4*>(p.vcache + (size_t)b * p.cache_seq_stride + (size_t)kvh * p.cache_head_stride + (size_t)n_ctx * HD + (size_t)(tid - 96) * 8) = vv;
        }
    }
    __syncthreads();
    // 8 MB of K/V requests from all CTAs at once delay the 4 KB of q, k, v that the whole prologue waits for (the
    // memory system serves requests in arrival order): in this mode the rows are requested behind them
    if (p.q_first && tok0 < t_end) { load_k(tok0, t_end - 1); load_v(tok0, t_end - 1); }
    const int n_ctas = gridDim.x * gridDim.y * gridDim.z;
    const bool stamp0 = p.trace && cta_linear == 0 && threadIdx.x == 0;  // finer stamps of the first CTA only
    if (stamp0) p.trace[n_ctas * 4 + 1] = attn_timer_ns();
    if (rotate) {
        // rotate-half RoPE (Generator/MetalSourceGenerator+Attention.swift:596-617): pairs (i, i + rope_dim/2)
        if (rot_i < pairs)
            for (int r = tid / (HD / 2); r < G + (DECODE ? 1 : 0); r += kSplitThreads / (HD / 2)) {
                const float lo = qk[r][rot_i], hi = qk[r][rot_i + pairs];
                qk[r][rot_i] = lo * rot_c - hi * rot_s;
                qk[r][rot_i + pairs] = lo * rot_s + hi * rot_c;
            }
        __syncthreads();
    }
    if (stamp0) p.trace[(n_ctas + 1) * 4 + 1] = attn_timer_ns();
    if (DECODE) {
        if (split == 0 && n_ctx < p.max_seq) {  // the rotated new k row, rounded, for later steps
            __nv_bfloat16* kw = p.kcache + (size_t)b * p.cache_seq_stride + (size_t)kvh * p.cache_head_stride + (size_t)n_ctx * HD;
            for (int d = tid; d < HD; d += kSplitThreads) kw[d] = __float2bfloat16_rn(qk[G][d]);
        }
        // score of the new token against itself, in fp32 from the unrounded rotated q and k
        // (Generator/MetalSourceGenerator+Attention.swift:866-868)
        for (int r = warp; r < G; r += kSplitWarps) {
            float prod = 0.f;
#pragma unroll
            for (int i = 0; i < HD / 32; ++i) prod = fmaf(qk[r][lane + 32 * i], qk[G][lane + 32 * i], prod);
            for (int o = 16; o > 0; o >>= 1) prod += __shfl_xor_sync(0xffffffffu, prod, o);
            if (lane == 0) self_score[r] = prod * p.scale_log2;
        }
    }

    if (stamp0) p.trace[(n_ctas + 1) * 4 + 2] = attn_timer_ns();
    // A fragments of the rotated q: lane (g, t) holds q[g][32*i + 8*t + 0..7]; hi + lo bf16 split
    unsigned qhi[NCH][4], qlo[NCH][4];
#pragma unroll
    for (int i = 0; i < NCH; ++i)
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            float2 ac = make_float2(0.f, 0.f);
            if (g < G) ac = *reinterpret_cast<const float2*>(&qk[g][32 * i + 8 * t + 2 * w]);
            const float ah = __bfloat162float(__float2bfloat16_rn(ac.x)), ch = __bfloat162float(__float2bfloat16_rn(ac.y));
            qhi[i][w] = pack_bf16(ah, ch);
            qlo[i][w] = pack_bf16(ac.x - ah, ac.y - ch);
        }

    if (stamp0) p.trace[n_ctas * 4 + 2] = attn_timer_ns();
    float m_run = -INFINITY, l_run = 0.f;
    float oacc[VH][8][4];
#pragma unroll
    for (int hh = 0; hh < VH; ++hh)
#pragma unroll
        for (int u = 0; u < 8; ++u) oacc[hh][u][0] = oacc[hh][u][1] = oacc[hh][u][2] = oacc[hh][u][3] = 0.f;

    if (DECODE && tok0 < t_end && tok0 + 16 > t_end) {
        // first batch, requested before the context length was known: rows beyond the context may hold anything;
        // their probabilities are zero, their values must be finite
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int hh = 0; hh < VH; ++hh) {
            if (tok0 + 2 * t >= t_end) va[hh] = z;
            if (tok0 + 2 * t + 1 >= t_end) vb[hh] = z;
            if (tok0 + 2 * t + 8 >= t_end) vc[hh] = z;
            if (tok0 + 2 * t + 9 >= t_end) vd[hh] = z;
        }
    }
    for (; tok0 < t_end; tok0 += t_stride) {
        const int nxt = tok0 + t_stride;
        if (tid == 0) prefetch_block(tok0 + (kAhead + 1) * t_stride);
        // S = q . K^T for 16 tokens
        float sacc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
            for (int i = 0; i < NCH; ++i) {
                const uint4 kk = kreg[nt][i];
                // rows g carry the high parts of q, rows g + 8 the low parts: one instruction forms both
                // products, and their sum is taken in-lane below
                mma_bf16(sacc[nt], qhi[i][0], qlo[i][0], qhi[i][1], qlo[i][1], kk.x, kk.y);
                mma_bf16(sacc[nt], qhi[i][2], qlo[i][2], qhi[i][3], qlo[i][3], kk.z, kk.w);
            }
        }
        if (nxt < t_end) load_k(nxt, t_end - 1);  // the K registers are free again
        // online softmax in the log2 domain; row g lives in the four lanes t = 0..3
        float sv[2][2];
        float rmax = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = tok0 + 8 * nt + 2 * t + e;
                sv[nt][e] = tok < t_end && tok >= t_lo ? (sacc[nt][e] + sacc[nt][2 + e]) * p.scale_log2 : -INFINITY;
                rmax = fmaxf(rmax, sv[nt][e]);
            }
        rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 1));
        rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
        const float m_new = fmaxf(m_run, rmax);
        const float m_ref = m_new == -INFINITY ? 0.f : m_new;  // 16 rows wholly below a sliding window: all weights 0
        const float corr = exp2f(m_run - m_ref);
        float pv[2][2];
        float psum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) { pv[nt][e] = exp2f(sv[nt][e] - m_ref); psum += pv[nt][e]; }
        l_run = l_run * corr + psum;
        m_run = m_new;
        if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
            for (int hh = 0; hh < VH; ++hh)
#pragma unroll
                for (int u = 0; u < 8; ++u) { oacc[hh][u][0] *= corr; oacc[hh][u][1] *= corr; oacc[hh][u][2] *= corr; oacc[hh][u][3] *= corr; }
        }
        // O += P . V ; dimension 64*hh + 8*col + u sits in n-tile (hh, u), column col. P is fed as a bf16
        // hi + lo pair: a single bf16 P (8 mantissa bits) costs ~2 bf16 ulps of the output at short contexts.
        float ph[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) ph[nt][e] = __bfloat162float(__float2bfloat16_rn(pv[nt][e]));
        const unsigned pa0 = pack_bf16(ph[0][0], ph[0][1]);
        const unsigned pa2 = pack_bf16(ph[1][0], ph[1][1]);
        const unsigned pl0 = pack_bf16(pv[0][0] - ph[0][0], pv[0][1] - ph[0][1]);
        const unsigned pl2 = pack_bf16(pv[1][0] - ph[1][0], pv[1][1] - ph[1][1]);
#pragma unroll
        for (int hh = 0; hh < VH; ++hh) {
            const unsigned aw[4] = {va[hh].x, va[hh].y, va[hh].z, va[hh].w};
            const unsigned bw[4] = {vb[hh].x, vb[hh].y, vb[hh].z, vb[hh].w};
            const unsigned cw[4] = {vc[hh].x, vc[hh].y, vc[hh].z, vc[hh].w};
            const unsigned dw[4] = {vd[hh].x, vd[hh].y, vd[hh].z, vd[hh].w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const unsigned b0e = __byte_perm(aw[w], bw[w], 0x5410), b1e = __byte_perm(cw[w], dw[w], 0x5410);
                const unsigned b0o = __byte_perm(aw[w], bw[w], 0x7632), b1o = __byte_perm(cw[w], dw[w], 0x7632);
                // rows g: high part of P, rows g + 8: low part; added when the accumulators are read out
                mma_bf16(oacc[hh][2 * w], pa0, pl0, pa2, pl2, b0e, b1e);
                mma_bf16(oacc[hh][2 * w + 1], pa0, pl0, pa2, pl2, b0o, b1o);
            }
        }
        if (nxt < t_end) load_v(nxt, t_end - 1);
        if (stamp0 && tok0 == t_begin) p.trace[n_ctas * 4 + 3] = attn_timer_ns();
    }

    if (p.trace && threadIdx.x == 0) p.trace[cta_linear * 4 + 2] = attn_timer_ns();
    // ---- merge the warps of this CTA ---------------------------------------------------------------
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (g < G) {
#pragma unroll
        for (int hh = 0; hh < VH; ++hh)
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                osm[warp][g][64 * hh + 8 * (2 * t) + u] = oacc[hh][u][0] + oacc[hh][u][2];
                osm[warp][g][64 * hh + 8 * (2 * t + 1) + u] = oacc[hh][u][1] + oacc[hh][u][3];
            }
        if (t == 0) { msm[warp][g] = m_run; lsm[warp][g] = l_run; }
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += kSplitThreads) {
        const int r = idx / HD, d = idx - r * HD;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < kSplitWarps; ++w) mx = fmaxf(mx, msm[w][r]);
        float o = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < kSplitWarps; ++w) {
            const float wgt = msm[w][r] == -INFINITY ? 0.f : exp2f(msm[w][r] - mx);
            o = fmaf(wgt, osm[w][r][d], o);
            l = fmaf(wgt, lsm[w][r], l);
        }
        const size_t slot = ((size_t)b * p.heads + (size_t)kvh * G + r) * p.splits + split;
        __stcg(p.part_o + slot * HD + d, o);
        if (d == 0) { __stcg(p.part_ml + slot * 2, mx); __stcg(p.part_ml + slot * 2 + 1, l); }
    }

    // ---- the last CTA of this (sequence, KV head) to arrive merges the splits and writes the output ----
    __shared__ int is_last;
    __syncthreads();
    if (tid == 0) {
        // release: cumulative over the partials every thread of this CTA wrote before the barrier; acquire: the
        // last arriver sees the partials of all the others
        unsigned* ctr = p.counters + (size_t)b * p.kv_heads + kvh;
        unsigned prev;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(ctr) : "memory");
        is_last = prev == (unsigned)p.splits - 1u;
        if (is_last) *ctr = 0u;  // ready for the next launch
    }
    __syncthreads();
    if (p.trace && threadIdx.x == 0) p.trace[cta_linear * 4 + 3] = attn_timer_ns();
    if (!is_last) return;

    // Everything that does not depend on the split weights is requested first: the (max, sum) pairs and the
    // first 16 partial outputs of this thread's four dimensions travel together.
    constexpr int kPre = 32;
    const int n_out4 = G * HD / 4;  // float4 outputs of the group
    float* wsm = &osm[1][0][0];     // [G][splits] weights (splits <= 64: fits the reused buffer)
    float* msm2 = &osm[2][0][0];    // [G][splits] split maxima
    float* lsm2 = &osm[3][0][0];    // [G][splits] split sums
    float2 ml[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int idx = tid + j * kSplitThreads;
        if (idx < G * p.splits) {
            const int r = idx / p.splits, sidx = idx - r * p.splits;
            const size_t slot = ((size_t)b * p.heads + (size_t)kvh * G + r) * p.splits + sidx;
            ml[j] = __ldcg(reinterpret_cast<const float2*>(p.part_ml + slot * 2));
        }
    }
    float4 pre[kPre];
    const float* po0 = nullptr;
    if (tid < n_out4) {
        const int r = tid / (HD / 4), d4 = tid - r * (HD / 4);
        po0 = p.part_o + (((size_t)b * p.heads + (size_t)kvh * G + r) * p.splits) * HD + d4 * 4;
#pragma unroll
        for (int sidx = 0; sidx < kPre; ++sidx)
            if (sidx < p.splits) pre[sidx] = __ldcg(reinterpret_cast<const float4*>(po0 + (size_t)sidx * HD));
    }
    for (int j = 0; j < 2; ++j) {
        const int idx = tid + j * kSplitThreads;
        if (idx < G * p.splits) { msm2[idx] = ml[j].x; lsm2[idx] = ml[j].y; }
    }
    for (int idx = tid + 2 * kSplitThreads; idx < G * p.splits; idx += kSplitThreads) {
        const int r = idx / p.splits, sidx = idx - r * p.splits;
        const size_t slot = ((size_t)b * p.heads + (size_t)kvh * G + r) * p.splits + sidx;
        msm2[idx] = __ldcg(p.part_ml + slot * 2);
        lsm2[idx] = __ldcg(p.part_ml + slot * 2 + 1);
    }
    __syncthreads();
    // weights of the splits: w = 2^(m_s - max), normalised by the total mass; the new token enters with its
    // own score and its unrounded v (Generator/MetalSourceGenerator+Attention.swift:905-907)
    float* inv_den = msm[0];  // reuse: G floats
    float* w_self = msm[1];
    for (int r = warp; r < G; r += kSplitWarps) {
        const float m_self = DECODE ? self_score[r] : -INFINITY;
        float mx = m_self;
        for (int sidx = lane; sidx < p.splits; sidx += 32) mx = fmaxf(mx, msm2[r * p.splits + sidx]);
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float den = 0.f;
        for (int sidx = lane; sidx < p.splits; sidx += 32) {
            const float ms = msm2[r * p.splits + sidx];
            const float w = ms == -INFINITY ? 0.f : exp2f(ms - mx);
            wsm[r * p.splits + sidx] = w;
            den = fmaf(w, lsm2[r * p.splits + sidx], den);
        }
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        const float ws = DECODE ? exp2f(m_self - mx) : 0.f;
        den += ws;
        if (lane == 0) { inv_den[r] = den > 0.f ? 1.0f / den : 0.f; w_self[r] = ws; }
    }
    __syncthreads();
    for (int idx = tid; idx < n_out4; idx += kSplitThreads) {
        const int r = idx / (HD / 4), d4 = idx - r * (HD / 4);
        const float* po = p.part_o + (((size_t)b * p.heads + (size_t)kvh * G + r) * p.splits) * HD + d4 * 4;
        const float* wr = wsm + r * p.splits;
        float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
        if (DECODE) {
            const float ws = w_self[r];
            num = make_float4(ws * vraw[d4 * 4], ws * vraw[d4 * 4 + 1], ws * vraw[d4 * 4 + 2], ws * vraw[d4 * 4 + 3]);
        }
        int s0 = 0;
        if (idx == tid) {  // this thread's first output: its first partials are already in registers
#pragma unroll
            for (int sidx = 0; sidx < kPre; ++sidx)
                if (sidx < p.splits) {
                    const float w = wr[sidx];
                    num.x = fmaf(w, pre[sidx].x, num.x); num.y = fmaf(w, pre[sidx].y, num.y);
                    num.z = fmaf(w, pre[sidx].z, num.z); num.w = fmaf(w, pre[sidx].w, num.w);
                }
            s0 = min(kPre, p.splits);
        }
#pragma unroll 16
        for (int sidx = s0; sidx < p.splits; ++sidx) {
            const float4 v4 = __ldcg(reinterpret_cast<const float4*>(po + (size_t)sidx * HD));
            const float w = wr[sidx];
            num.x = fmaf(w, v4.x, num.x); num.y = fmaf(w, v4.y, num.y);
            num.z = fmaf(w, v4.z, num.z); num.w = fmaf(w, v4.w, num.w);
        }
        const float inv = inv_den[r];
        uint2 packed;
        packed.x = pack_bf16(num.x * inv, num.y * inv);
        packed.y = pack_bf16(num.z * inv, num.w * inv);
        *reinterpret_cast<uint2*>(p.out + (size_t)b * p.out_stride + (size_t)(kvh * G + r) * HD + d4 * 4) = packed;
    }
    if (p.trace) {
        __syncthreads();
        if (threadIdx.x == 0) p.trace[(gridDim.x * gridDim.y * gridDim.z + (blockIdx.z * gridDim.y + blockIdx.y)) * 4] = attn_timer_ns();  // merged
    }
}

// Prompt ingestion: rotate the chunk's k rows (token b at position pos_base + b) and append them and the v rows to
// the cache of sequence 0, rounded to bf16 (Generator/MetalSourceGenerator+Attention.swift:761-805 does the same
// per decode step). One CTA per (token, KV head).
__global__ void __launch_bounds__(128) rope_append_kernel(const AttnParams p, int hd) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float vec[128];
    __shared__ float cs[64], sn[64];
    const int b = blockIdx.x, kvh = blockIdx.y, tid = threadIdx.x;
    const int pos = p.pos_base + b;
    if (pos >= p.max_seq) return;
    for (int i = tid; i < (p.rope_dim >> 1); i += 128) {
        float sv_, cv_;
        sincosf((float)pos * p.inv_freq[i], &sv_, &cv_);
        cs[i] = cv_; sn[i] = sv_;
    }
    for (int d = tid; d < hd; d += 128) vec[d] = __bfloat162float(p.k[(size_t)b * p.k_stride + kvh * hd + d]);
    __syncthreads();
    const size_t row = (size_t)kvh * p.cache_head_stride + (size_t)pos * hd;
    for (int d = tid; d < hd; d += 128) {
        p.kcache[row + d] = __float2bfloat16_rn(rope_elem(vec, d, p.rope_dim, cs, sn));
        p.vcache[row + d] = p.v[(size_t)b * p.v_stride + kvh * hd + d];
    }
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, what);
    return SWLM_OK;
}


// ---- decode attention over a quantized cache (8-bit groups of 32 / 64 / 128, 4-bit groups of 64 / 128) ----------------
// Rows are head_dim / group blocks of fp16 scale | fp16 zero | payload (36 bytes for 8-bit groups of 32), value = scale * q + zero
// (read_kv_element, Generator/MetalSourceGenerator+Attention.swift:1923-1956). Half the bytes of the bf16 cache cross
// HBM. One CTA per (split, KV head, sequence) as in the bf16 kernel; a warp takes one token at a time, every lane
// dequantises its head_dim / 32 consecutive elements of the K row and of the V row and the dot products of the GQA
// group's q rows are reduced across the warp; online softmax in fp32. The new token enters with its unrounded rotated k
// and its v (:866-868, :905-907); split 0 quantises both into the cache (write_kv_quantized_q8, :2057-2101: scale =
// (max - min) / 255 per group, q = round((x - min) / scale), fp16 scale and min stored). The last CTA of a
// (sequence, KV head) to arrive merges the splits.
constexpr int kQ8Warps = 8, kQ8Threads = kQ8Warps * 32;

// One row of head_dim floats into blocks of `group` values with `bits` bits each: a warp per group, a lane takes
// group / 32 consecutive values (write_kv_quantized_q8 / _q4, Generator/MetalSourceGenerator+Attention.swift:2057-2150).
// RESID: resid[i] = src[i] - the value the stored block gives back for it (fp16 scale and zero), the residual that
// qjl_compute_residual (:1983-2013) projects.
template <bool RESID = false>
__device__ __forceinline__ void q8_quantise_row(const float* src, unsigned char* row, int hd, int bits, int group, int warp, int lane, float* resid = nullptr) {
    const int epg = group / 32, bb = 4 + group * bits / 8;
    const float levels = bits == 8 ? 255.0f : 15.0f;
    for (int g = warp; g * group < hd; g += kQ8Warps) {
        float x[4];
        float lo = HUGE_VALF, hi = -HUGE_VALF;
        for (int j = 0; j < epg; ++j) { x[j] = src[g * group + lane * epg + j]; lo = fminf(lo, x[j]); hi = fmaxf(hi, x[j]); }
        for (int o = 16; o > 0; o >>= 1) { lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o)); hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o)); }
        float scale = (hi - lo) / levels;
        if (scale < 1e-10f) scale = 1e-10f;
        unsigned char* blk = row + (size_t)g * bb;
        if (lane == 0) {
            const __half2 hdr = __floats2half2_rn(scale, lo);
            *reinterpret_cast<__half2*>(blk) = hdr;
        }
        int q[4];
        for (int j = 0; j < epg; ++j) q[j] = min(max((int)roundf((x[j] - lo) / scale), 0), (int)levels);
        if (RESID) {
            const float sh = __half2float(__float2half_rn(scale)), zh = __half2float(__float2half_rn(lo));
            for (int j = 0; j < epg; ++j) resid[g * group + lane * epg + j] = x[j] - fmaf(sh, (float)q[j], zh);
        }
        if (bits == 8) {
            for (int j = 0; j < epg; ++j) blk[4 + lane * epg + j] = (unsigned char)q[j];
        } else {   // two values per byte, the even one in the low nibble (epg is 2 or 4)
            for (int j = 0; j < epg; j += 2) blk[4 + (lane * epg + j) / 2] = (unsigned char)(q[j] | (q[j + 1] << 4));
        }
    }
}

// Sandwich product of Cl(3,0) (rotor_sandwich / rotor_sandwich_inverse, Generator/MetalSourceGenerator+Attention.swift:
// 1807-1821): the rotor R = (s, b12, b13, b23) turns (x, y, z) like the unit quaternion (s, b23, -b13, b12), in the
// cross-product form v + s t + p x t with t = 2 p x v; INV uses the conjugate.
template <bool INV>
__device__ __forceinline__ void rotor_turn(const __half* R, float& x, float& y, float& z) {
    const float s = __half2float(R[0]);
    float px = __half2float(R[3]), py = -__half2float(R[2]), pz = __half2float(R[1]);
    if (INV) { px = -px; py = -py; pz = -pz; }
    const float tx = 2.0f * (py * z - pz * y), ty = 2.0f * (pz * x - px * z), tz = 2.0f * (px * y - py * x);
    const float rx = x + s * tx + (py * tz - pz * ty);
    const float ry = y + s * ty + (pz * tx - px * tz);
    const float rz = z + s * tz + (px * ty - py * tx);
    x = rx; y = ry; z = rz;
}
// group g = values 3g .. 3g + 2 of a row of hd floats, in place; values past the row's end enter as zeros and are not
// stored (rotor_apply_forward / _inverse, :1827-1884)
template <bool INV>
__device__ __forceinline__ void rotor_turn_group(float* row, int hd, const __half* rotors, int g) {
    const int base = 3 * g;
    float x = row[base], y = base + 1 < hd ? row[base + 1] : 0.0f, z = base + 2 < hd ? row[base + 2] : 0.0f;
    rotor_turn<INV>(rotors + 4 * g, x, y, z);
    row[base] = x;
    if (base + 1 < hd) row[base + 1] = y;
    if (base + 2 < hd) row[base + 2] = z;
}

// G (query heads per KV head) is a template argument: the per-head dot products, warp reductions and softmax updates of
// a row are then one basic block whose four or eight independent chains the compiler interleaves.
//
// ROTOR (the rotated schemes, :694-930): q, the new k (both after RoPE) and the new v are turned by the KV head's rotors
// before anything else, so the cache holds turned rows and q . k is unchanged; the merged output is turned back. With
// qjl_dim > 0 split 0 also stores Phi . (k - its dequantised row) for the new row, and the score of a cached row gains
// (Phi . q) . (that row's stored values): lane l carries columns l and l + 32 of both into the warp reduction.
// (Up to four query heads per KV head the rotated form is held to 128 registers so that two CTAs share an SM like the
// plain form's, which fits by itself: the kernel is bound by instruction issue and needs both. The plain form states no
// minimum - a minimum of one would let the compiler spread it over 150 registers and halve its occupancy.)
template <int HD, int G, int BITS, bool ROTOR>
__global__ void __launch_bounds__(kQ8Threads, ROTOR && G <= 4 ? 2 : 0) attn_q8_split_kernel(const AttnParams p) {
    constexpr int EPL = HD / 32;           // elements per lane
    constexpr int NG = (HD + 2) / 3;       // rotors per KV head
    const int GROUP = p.kv_group, BB = 4 + GROUP * BITS / 8;   // values and bytes per block (BITS per value)
    const int ROW_BYTES = HD / GROUP * BB;
    pdl_launch_dependents();
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __shared__ float qs[G][HD];
    __shared__ float kcur[HD], vcur[HD];
    __shared__ float osm[kQ8Warps][kMaxGroup][HD];   // (sized for the merge scratch below whatever G is)
    __shared__ float msm[kQ8Warps][kMaxGroup], lsm[kQ8Warps][kMaxGroup];
    __shared__ int is_last;
    __shared__ float kres[ROTOR ? HD : 1];          // the new k row minus its dequantised blocks
    __shared__ float qp[ROTOR ? G : 1][64];         // Phi . q of every head of the group
    const __half* const head_rotors = ROTOR ? p.rotors + (size_t)kvh * NG * 4 : nullptr;
    const int qjl = ROTOR ? p.qjl_dim : 0;
    pdl_wait();
    const int n_ctx = p.position[b];
    for (int idx = tid; idx < G * HD; idx += kQ8Threads)
        qs[idx / HD][idx % HD] = __bfloat162float(p.q[(size_t)b * p.q_stride + (size_t)kvh * G * HD + idx]);
    for (int d = tid; d < HD; d += kQ8Threads) {
        kcur[d] = __bfloat162float(p.k[(size_t)b * p.k_stride + (size_t)kvh * HD + d]);
        vcur[d] = __bfloat162float(p.v[(size_t)b * p.v_stride + (size_t)kvh * HD + d]);
    }
    __syncthreads();
    if (p.rope_dim > 0) {
        // rotate-half RoPE (Generator/MetalSourceGenerator+Attention.swift:596-617): pairs (i, i + rope_dim/2)
        const int pairs = p.rope_dim >> 1;
        for (int idx = tid; idx < (G + 1) * pairs; idx += kQ8Threads) {
            const int r = idx / pairs, i = idx - r * pairs;
            float sn, cs;
            sincosf((float)n_ctx * p.inv_freq[i], &sn, &cs);
            float* row = r < G ? qs[r] : kcur;
            const float lo = row[i], hi = row[i + pairs];
            row[i] = lo * cs - hi * sn;
            row[i + pairs] = lo * sn + hi * cs;
        }
        __syncthreads();
    }
    if (ROTOR) {
        for (int idx = tid; idx < (G + 2) * NG; idx += kQ8Threads) {
            const int r = idx / NG, g = idx - r * NG;
            rotor_turn_group<false>(r < G ? qs[r] : r == G ? kcur : vcur, HD, head_rotors, g);
        }
        __syncthreads();
    }
    const size_t head_bytes = (size_t)p.max_seq * ROW_BYTES;
    unsigned char* kbase = reinterpret_cast<unsigned char*>(p.kcache) + ((size_t)b * p.kv_heads + kvh) * head_bytes;
    unsigned char* vbase = reinterpret_cast<unsigned char*>(p.vcache) + ((size_t)b * p.kv_heads + kvh) * head_bytes;
    const __half* const res_base = ROTOR && qjl > 0 ? p.qjl_res + ((size_t)b * p.kv_heads + kvh) * p.max_seq * qjl : nullptr;
    if (split == 0 && n_ctx < p.max_seq) {
        q8_quantise_row<ROTOR>(kcur, kbase + (size_t)n_ctx * ROW_BYTES, HD, BITS, GROUP, warp, lane, kres);
        q8_quantise_row(vcur, vbase + (size_t)n_ctx * ROW_BYTES, HD, BITS, GROUP, warp, lane);
        if (ROTOR && qjl > 0) {   // (the branch is uniform over the CTA)
            __syncthreads();
            __half* res = p.qjl_res + (((size_t)b * p.kv_heads + kvh) * p.max_seq + n_ctx) * qjl;
            for (int j = warp; j < qjl; j += kQ8Warps) {
                float a = 0.f;
                for (int d = lane; d < HD; d += 32) a = fmaf(kres[d], __half2float(__ldg(p.qjl_matrix + (size_t)d * qjl + j)), a);
                for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                if (lane == 0) res[j] = __float2half_rn(a);
            }
        }
    }
    float qpr[G][2];   // this lane's two columns of Phi . q (zero past qjl_dim)
#pragma unroll
    for (int r = 0; r < G; ++r) qpr[r][0] = qpr[r][1] = 0.f;
    if (ROTOR && qjl > 0) {
        const int cols = ROTOR ? qjl : 1;   // (the plain instantiation never gets here; keeps its dead code free of a constant zero divisor)
        for (int idx = tid; idx < G * qjl; idx += kQ8Threads) {
            const int r = idx / cols, j = idx - r * cols;
            float a = 0.f;
            for (int d = 0; d < HD; ++d) a = fmaf(qs[r][d], __half2float(__ldg(p.qjl_matrix + (size_t)d * qjl + j)), a);
            qp[r][j] = a;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < G; ++r) {
            if (lane < qjl) qpr[r][0] = qp[r][lane];
            if (lane + 32 < qjl) qpr[r][1] = qp[r][lane + 32];
        }
    }
    // this lane's elements e0 .. e0 + EPL - 1 lie in one block; its payload is EPL * BITS / 8 bytes (4, 2 or 1),
    // naturally aligned
    const int e0 = lane * EPL, blk_off = (e0 / GROUP) * BB, pay_off = blk_off + 4 + (e0 % GROUP) * BITS / 8;
    constexpr int pay_bytes = EPL * BITS / 8;
    constexpr unsigned qmask = BITS == 8 ? 0xffu : 0xfu;
    auto load_payload = [&](const unsigned char* ptr) -> unsigned {
        if (pay_bytes == 4) return __ldg(reinterpret_cast<const unsigned*>(ptr));
        if (pay_bytes == 2) return __ldg(reinterpret_cast<const unsigned short*>(ptr));
        return __ldg(ptr);
    };
    float qr[G][EPL];
#pragma unroll
    for (int r = 0; r < G; ++r)
#pragma unroll
        for (int j = 0; j < EPL; ++j) qr[r][j] = qs[r][e0 + j];
    float m_run[G], l_run[G], acc[G][EPL];
#pragma unroll
    for (int r = 0; r < G; ++r) {
        m_run[r] = -INFINITY; l_run[r] = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) acc[r][j] = 0.f;
    }
    // one row's scores (already reduced over the warp, unscaled) and values enter the running softmax of every head
    auto update = [&](const float (&sc)[G], const float (&vf)[EPL]) {
#pragma unroll
        for (int r = 0; r < G; ++r) {
            const float s = sc[r] * p.scale_log2;
            const float m_new = fmaxf(m_run[r], s);
            const float corr = exp2f(m_run[r] - m_new), w = exp2f(s - m_new);
            l_run[r] = l_run[r] * corr + w;
            m_run[r] = m_new;
#pragma unroll
            for (int j = 0; j < EPL; ++j) acc[r][j] = fmaf(w, vf[j], acc[r][j] * corr);
        }
    };
    // the split's share of the cached rows [t_lo, n_ctx): contiguous; a warp takes every fourth row of it
    const int t_lo = p.window > 0 ? max(0, n_ctx + 1 - p.window) : 0;
    const int per = (n_ctx - t_lo + p.splits - 1) / p.splits;
    const int t0 = t_lo + split * per, t1 = min(n_ctx, t0 + per);
    // eight rows per warp are requested before the first is used: one trip to memory per eight rows instead of one per row
    constexpr int UN = 8;
    for (int tb = t0 + warp; tb < t1; tb += kQ8Warps * UN) {
        unsigned kw[UN], vw[UN], khd[UN], vhd[UN];
        unsigned short rz0[ROTOR ? UN : 1], rz1[ROTOR ? UN : 1];   // the row's projected residual, columns lane and lane + 32
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int t = min(tb + u * kQ8Warps, t1 - 1);   // rows past the end repeat the last one and are not absorbed
            const unsigned char* kr = kbase + (size_t)t * ROW_BYTES;
            const unsigned char* vr = vbase + (size_t)t * ROW_BYTES;
            khd[u] = __ldg(reinterpret_cast<const unsigned*>(kr + blk_off));
            vhd[u] = __ldg(reinterpret_cast<const unsigned*>(vr + blk_off));
            kw[u] = load_payload(kr + pay_off);
            vw[u] = load_payload(vr + pay_off);
            if (ROTOR) {
                rz0[u] = rz1[u] = 0;
                if (qjl > 0) {
                    const unsigned short* rr = reinterpret_cast<const unsigned short*>(res_base) + (size_t)t * qjl;
                    if (lane < qjl) rz0[u] = __ldg(rr + lane);
                    if (lane + 32 < qjl) rz1[u] = __ldg(rr + lane + 32);
                }
            }
        }
        // the scores of the eight rows for all heads: 8 x G independent dot products and warp reductions, interleaved
        float sc[UN][G];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const __half2 kh = *reinterpret_cast<const __half2*>(&khd[u]);
            const float ks = __low2float(kh), kz = __high2float(kh);
            float kf[EPL];
#pragma unroll
            for (int j = 0; j < EPL; ++j) kf[j] = fmaf(ks, (float)((kw[u] >> (BITS * j)) & qmask), kz);
#pragma unroll
            for (int r = 0; r < G; ++r) {
                sc[u][r] = 0.f;
#pragma unroll
                for (int j = 0; j < EPL; ++j) sc[u][r] = fmaf(qr[r][j], kf[j], sc[u][r]);
            }
            if (ROTOR) {
                const float r0 = __half2float(__ushort_as_half(rz0[u])), r1 = __half2float(__ushort_as_half(rz1[u]));
#pragma unroll
                for (int r = 0; r < G; ++r) sc[u][r] = fmaf(qpr[r][1], r1, fmaf(qpr[r][0], r0, sc[u][r]));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < UN; ++u)
#pragma unroll
                for (int r = 0; r < G; ++r) sc[u][r] += __shfl_xor_sync(0xffffffffu, sc[u][r], o);
        // the eight rows enter the running softmax together: one new maximum and one rescale per head for the lot
        // (rows past the end carry the score -inf, i.e. weight 0)
        float vfu[UN][EPL];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const __half2 vh = *reinterpret_cast<const __half2*>(&vhd[u]);
            const float vs = __low2float(vh), vz = __high2float(vh);
#pragma unroll
            for (int j = 0; j < EPL; ++j) vfu[u][j] = fmaf(vs, (float)((vw[u] >> (BITS * j)) & qmask), vz);
        }
#pragma unroll
        for (int r = 0; r < G; ++r) {
            float m_new = m_run[r];
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                sc[u][r] = tb + u * kQ8Warps < t1 ? sc[u][r] * p.scale_log2 : -INFINITY;
                m_new = fmaxf(m_new, sc[u][r]);
            }
            const float corr = exp2f(m_run[r] - m_new);   // m_new is finite: the batch's first row is inside the range
            float wsum = 0.f;
#pragma unroll
            for (int j = 0; j < EPL; ++j) acc[r][j] *= corr;
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const float w = exp2f(sc[u][r] - m_new);
                wsum += w;
#pragma unroll
                for (int j = 0; j < EPL; ++j) acc[r][j] = fmaf(w, vfu[u][j], acc[r][j]);
            }
            l_run[r] = l_run[r] * corr + wsum;
            m_run[r] = m_new;
        }
    }
    if (split == 0 && warp == 0) {   // the new token: unrounded rotated k, v as given
        float vf[EPL], sc[G];
#pragma unroll
        for (int j = 0; j < EPL; ++j) vf[j] = vcur[e0 + j];
#pragma unroll
        for (int r = 0; r < G; ++r) {
            sc[r] = 0.f;
#pragma unroll
            for (int j = 0; j < EPL; ++j) sc[r] = fmaf(qr[r][j], kcur[e0 + j], sc[r]);
            for (int o = 16; o > 0; o >>= 1) sc[r] += __shfl_xor_sync(0xffffffffu, sc[r], o);
        }
        update(sc, vf);
    }
    // ---- merge the warps, publish the split's partial ----------------------------------------------------
#pragma unroll
    for (int r = 0; r < G; ++r) {
#pragma unroll
        for (int j = 0; j < EPL; ++j) osm[warp][r][e0 + j] = acc[r][j];
        if (lane == 0) { msm[warp][r] = m_run[r]; lsm[warp][r] = l_run[r]; }
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += kQ8Threads) {
        const int r = idx / HD, d = idx - r * HD;
        float mx = -INFINITY;
        for (int w = 0; w < kQ8Warps; ++w) mx = fmaxf(mx, msm[w][r]);
        float o = 0.f, l = 0.f;
        for (int w = 0; w < kQ8Warps; ++w) {
            const float wgt = msm[w][r] == -INFINITY ? 0.f : exp2f(msm[w][r] - mx);
            o = fmaf(wgt, osm[w][r][d], o);
            l = fmaf(wgt, lsm[w][r], l);
        }
        const size_t slot = ((size_t)b * p.heads + (size_t)kvh * G + r) * p.splits + split;
        __stcg(p.part_o + slot * HD + d, o);
        if (d == 0) { __stcg(p.part_ml + slot * 2, mx); __stcg(p.part_ml + slot * 2 + 1, l); }
    }
    __syncthreads();
    if (tid == 0) {
        unsigned* ctr = p.counters + (size_t)b * p.kv_heads + kvh;
        unsigned prev;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(ctr) : "memory");
        is_last = prev == (unsigned)p.splits - 1u;
        if (is_last) *ctr = 0u;
    }
    __syncthreads();
    if (!is_last) return;
    // the merge: all (max, sum) pairs travel together, then every thread adds up one float4 of one head's output over
    // the splits with the loads of eight splits in flight at a time (rolled loops of dependent L2 round trips made this
    // the longest part of the kernel)
    float* wsm = &osm[0][0][0];              // [G][splits] weights (splits <= 64)
    float* lsm2 = &osm[1][0][0];             // [G][splits] sums
    __shared__ float inv_den[kMaxGroup];
    for (int idx = tid; idx < G * p.splits; idx += kQ8Threads) {
        const int r = idx / p.splits, sidx = idx - r * p.splits;
        const size_t slot = ((size_t)b * p.heads + (size_t)kvh * G + r) * p.splits + sidx;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + slot * 2));
        wsm[idx] = ml.x; lsm2[idx] = ml.y;
    }
    __syncthreads();
    for (int r = warp; r < G; r += kQ8Warps) {
        float mx = -INFINITY;
        for (int sidx = lane; sidx < p.splits; sidx += 32) mx = fmaxf(mx, wsm[r * p.splits + sidx]);
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float den = 0.f;
        for (int sidx = lane; sidx < p.splits; sidx += 32) {
            const float ms = wsm[r * p.splits + sidx];
            const float w = ms == -INFINITY ? 0.f : exp2f(ms - mx);
            wsm[r * p.splits + sidx] = w;
            den = fmaf(w, lsm2[r * p.splits + sidx], den);
        }
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        if (lane == 0) inv_den[r] = den > 0.f ? 1.0f / den : 0.f;
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD / 4; idx += kQ8Threads) {
        const int r = idx / (HD / 4), d4 = idx - r * (HD / 4);
        const float* po = p.part_o + (((size_t)b * p.heads + (size_t)kvh * G + r) * p.splits) * HD + d4 * 4;
        const float* wr = wsm + r * p.splits;
        float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int sidx = 0; sidx < p.splits; ++sidx) {
            const float4 v4 = __ldcg(reinterpret_cast<const float4*>(po + (size_t)sidx * HD));
            const float w = wr[sidx];
            num.x = fmaf(w, v4.x, num.x); num.y = fmaf(w, v4.y, num.y); num.z = fmaf(w, v4.z, num.z); num.w = fmaf(w, v4.w, num.w);
        }
        const float inv = inv_den[r];
        if (ROTOR) {   // normalised, still in the turned basis
            qs[r][d4 * 4 + 0] = num.x * inv; qs[r][d4 * 4 + 1] = num.y * inv;
            qs[r][d4 * 4 + 2] = num.z * inv; qs[r][d4 * 4 + 3] = num.w * inv;
            continue;
        }
        __nv_bfloat16* o = p.out + (size_t)b * p.out_stride + (size_t)(kvh * G + r) * HD + d4 * 4;
        o[0] = __float2bfloat16_rn(num.x * inv); o[1] = __float2bfloat16_rn(num.y * inv);
        o[2] = __float2bfloat16_rn(num.z * inv); o[3] = __float2bfloat16_rn(num.w * inv);
    }
    if (ROTOR) {
        __syncthreads();
        for (int idx = tid; idx < G * NG; idx += kQ8Threads) rotor_turn_group<true>(qs[idx / NG], HD, head_rotors, idx % NG);
        __syncthreads();
        for (int idx = tid; idx < G * HD; idx += kQ8Threads)
            p.out[(size_t)b * p.out_stride + (size_t)kvh * G * HD + idx] = __float2bfloat16_rn(qs[idx / HD][idx % HD]);
    }
}

template <int MODE>
int launch_both(const AttnParams& p, int m, int hd, cudaStream_t s) {
    const dim3 grid(p.splits, p.kv_heads, m);
    if (hd == 128) {
        launch_k(attn_split_kernel<128, MODE>, dim3(grid), dim3(kSplitThreads), 0, s, p);
    } else if (hd == 64) {
        launch_k(attn_split_kernel<64, MODE>, dim3(grid), dim3(kSplitThreads), 0, s, p);
    } else {
        set_error("attention: head_dim %d not supported (64 or 128)", hd);
        return SWLM_ERR_UNSUPPORTED;
    }
    return check_launch("attention launch");
}

}  // namespace

// ---- prompt ingestion: tiled causal attention over the cache ----------------------------------------------
// The chunk's k/v rows are already in the cache (rope_append_kernel); token b of the chunk attends rows
// 0..pos_base+b. One CTA serves 64 query rows = (64 / G) consecutive tokens x the G query heads of one KV head, so
// a K/V tile is read once per 64 rows instead of once per token (the reference's prefill attention walks the
// context once per query head and position, Generator/MetalSourceGenerator+Attention.swift:551-930). K/V tiles of
// 64 rows go through shared memory (cp.async, two stages, ldmatrix); arithmetic as in the decode kernel: q is
// rotated in fp32 and fed as a bf16 hi + lo pair in rows g / g + 8 of the A fragment, as are the probabilities;
// scores, softmax and the output accumulate in fp32.
constexpr int kPfWarps = 8, kPfThreads = kPfWarps * 32, kPfRows = kPfWarps * 8, kPfTile = 64;

template <int HD>
constexpr size_t attn_prefill_smem() {
    return (size_t)4 * kPfTile * (HD * 2 + 16) + (size_t)kPfRows * (HD + 2) * 4 + (size_t)kPfRows * HD * 4;
}

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <int HD>
__global__ void __launch_bounds__(kPfThreads) attn_prefill_kernel(const AttnParams p) {
    constexpr int PK = HD * 2 + 16;       // bytes per K/V row in shared memory: 8 rows of an ldmatrix hit 8 different 16-byte bank groups
    constexpr int TILE_BYTES = kPfTile * PK;
    constexpr int QP = HD + 2;            // floats per q row
    constexpr int KS = HD / 16;           // k-steps of q . K^T
    extern __shared__ __align__(16) unsigned char pf_smem[];
    unsigned char* kv_sm = pf_smem;                                          // [2 stages][K tile | V tile]
    float* q_sm = reinterpret_cast<float*>(pf_smem + 4 * TILE_BYTES);        // [64 rows][QP]
    float* cs_sm = q_sm + kPfRows * QP;                                      // [tokens][HD / 2] cos, then the same for sin
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int G = p.heads / p.kv_heads;   // 1, 2, 4 or 8
    const int TQ = kPfRows / G;           // tokens per CTA
    const int qt = gridDim.x - 1 - blockIdx.x, kvh = blockIdx.y;   // the longest rows first
    const int tok0 = qt * TQ;
    const int n_tok = min(TQ, p.chunk_tokens - tok0);
    const int pairs = p.rope_dim >> 1;
    float* sn_sm = cs_sm + TQ * (HD / 2);
    pdl_wait();

    const __nv_bfloat16* kbase = p.kcache + (size_t)kvh * p.cache_head_stride;
    const __nv_bfloat16* vbase = p.vcache + (size_t)kvh * p.cache_head_stride;
    const int last_row = p.pos_base + p.chunk_tokens - 1;              // last cache row that holds data
    const int n_tiles = (p.pos_base + tok0 + n_tok - 1) / kPfTile + 1; // tiles the CTA's last token attends
    // sliding window: the CTA's first token reaches back furthest
    const int tile_lo = p.window > 0 ? max(0, p.pos_base + tok0 - p.window + 1) / kPfTile : 0;
    auto load_tile = [&](int tile, int stage) {
        unsigned char* kd = kv_sm + (size_t)stage * 2 * TILE_BYTES;
        unsigned char* vd = kd + TILE_BYTES;
        constexpr int CPR = HD / 8;  // 16-byte chunks per row
        for (int idx = tid; idx < kPfTile * CPR; idx += kPfThreads) {
            const int r = idx / CPR, c = idx - r * CPR;
            const size_t src = (size_t)min(tile * kPfTile + r, last_row) * HD + c * 8;
            const unsigned kdst = (unsigned)__cvta_generic_to_shared(kd + r * PK + c * 16);
            const unsigned vdst = (unsigned)__cvta_generic_to_shared(vd + r * PK + c * 16);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kdst), "l"(kbase + src) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vdst), "l"(vbase + src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_tile(tile_lo, tile_lo & 1);

    // ---- prologue: q rows (row = token * G + head) to shared memory as floats, rotation table, rotation ----
    for (int idx = tid; idx < kPfRows * (HD / 8); idx += kPfThreads) {
        const int rr = idx / (HD / 8), c = idx - rr * (HD / 8);
        const int tl = rr / G, head = rr - tl * G;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tl < n_tok) v = *reinterpret_cast<const uint4*>(p.q + (size_t)(tok0 + tl) * p.q_stride + (size_t)(kvh * G + head) * HD + c * 8);
        const unsigned u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
            *reinterpret_cast<float2*>(q_sm + rr * QP + c * 8 + 2 * j) = make_float2(__uint_as_float(u[j] << 16), __uint_as_float(u[j] & 0xffff0000u));
    }
    for (int idx = tid; idx < n_tok * pairs; idx += kPfThreads) {
        const int tl = idx / pairs, i = idx - tl * pairs;
        float sv_, cv_;
        sincosf((float)(p.pos_base + tok0 + tl) * p.inv_freq[i], &sv_, &cv_);
        cs_sm[tl * (HD / 2) + i] = cv_; sn_sm[tl * (HD / 2) + i] = sv_;
    }
    __syncthreads();
    // rotate-half RoPE (Generator/MetalSourceGenerator+Attention.swift:596-617): pairs (i, i + rope_dim/2)
    for (int idx = tid; idx < n_tok * G * pairs; idx += kPfThreads) {
        const int rr = idx / pairs, i = idx - rr * pairs;
        const int tl = rr / G;
        const float c = cs_sm[tl * (HD / 2) + i], sn = sn_sm[tl * (HD / 2) + i];
        const float lo = q_sm[rr * QP + i], hi = q_sm[rr * QP + i + pairs];
        q_sm[rr * QP + i] = lo * c - hi * sn;
        q_sm[rr * QP + i + pairs] = lo * sn + hi * c;
    }
    __syncthreads();
    // A fragments of this warp's 8 rows: rows g carry the high bf16 parts, rows g + 8 the low parts
    unsigned qa[KS][4];
    {
        const float* qrow = q_sm + (warp * 8 + g) * QP;
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
            const float2 x0 = *reinterpret_cast<const float2*>(qrow + 16 * kk + 2 * t);
            const float2 x1 = *reinterpret_cast<const float2*>(qrow + 16 * kk + 8 + 2 * t);
            const float h0 = __bfloat162float(__float2bfloat16_rn(x0.x)), h1 = __bfloat162float(__float2bfloat16_rn(x0.y));
            const float h2 = __bfloat162float(__float2bfloat16_rn(x1.x)), h3 = __bfloat162float(__float2bfloat16_rn(x1.y));
            qa[kk][0] = pack_bf16(h0, h1); qa[kk][1] = pack_bf16(x0.x - h0, x0.y - h1);
            qa[kk][2] = pack_bf16(h2, h3); qa[kk][3] = pack_bf16(x1.x - h2, x1.y - h3);
        }
    }
    // position of this lane's row; rows past the chunk's end repeat the last token (their output is dropped)
    const int row_tl = min((warp * 8 + g) / G, n_tok - 1);
    const int pos_row = p.pos_base + tok0 + row_tl;
    const int warp_last_pos = p.pos_base + tok0 + min((warp * 8 + 7) / G, n_tok - 1);

    float m_run = -INFINITY, l_run = 0.f;
    float oacc[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) oacc[j][0] = oacc[j][1] = oacc[j][2] = oacc[j][3] = 0.f;

    const int row_lo = p.window > 0 ? pos_row - p.window + 1 : 0;   // first key this lane's row attends
    for (int tile = tile_lo; tile < n_tiles; ++tile) {
        if (tile + 1 < n_tiles) load_tile(tile + 1, (tile + 1) & 1);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        if (tile * kPfTile <= warp_last_pos) {
            const unsigned kb = (unsigned)__cvta_generic_to_shared(kv_sm + (size_t)(tile & 1) * 2 * TILE_BYTES);
            const unsigned vb = kb + TILE_BYTES;
            // S = q . K^T: 8 key tiles of 8
            float sacc[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
#pragma unroll
                for (int k2 = 0; k2 < KS / 2; ++k2) {
                    unsigned b[4];
                    ldsm_x4(b, kb + (unsigned)((8 * j + (lane & 7)) * PK + (32 * k2 + 8 * (lane >> 3)) * 2));
                    mma_bf16(sacc[j], qa[2 * k2][0], qa[2 * k2][1], qa[2 * k2][2], qa[2 * k2][3], b[0], b[1]);
                    mma_bf16(sacc[j], qa[2 * k2 + 1][0], qa[2 * k2 + 1][1], qa[2 * k2 + 1][2], qa[2 * k2 + 1][3], b[2], b[3]);
                }
            }
            // causal mask, online softmax in the log2 domain; row g lives in the four lanes t = 0..3
            float rmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = tile * kPfTile + 8 * j + 2 * t + e;
                    const float v = key <= pos_row && key >= row_lo ? (sacc[j][e] + sacc[j][2 + e]) * p.scale_log2 : -INFINITY;
                    sacc[j][e] = v;
                    rmax = fmaxf(rmax, v);
                }
            rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 1));
            rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
            const float m_new = fmaxf(m_run, rmax);
            const float m_ref = m_new == -INFINITY ? 0.f : m_new;   // a tile wholly outside this row's window: all weights 0
            const float corr = exp2f(m_run - m_ref);
            float psum = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) { sacc[j][e] = exp2f(sacc[j][e] - m_ref); psum += sacc[j][e]; }
            l_run = l_run * corr + psum;
            m_run = m_new;
            if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                for (int j = 0; j < HD / 8; ++j) { oacc[j][0] *= corr; oacc[j][1] *= corr; oacc[j][2] *= corr; oacc[j][3] *= corr; }
            }
            // O += P . V over 4 steps of 16 keys; P as hi + lo in rows g / g + 8
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                unsigned pa[4];
                {
                    const float a0 = sacc[2 * kk][0], a1 = sacc[2 * kk][1], c0 = sacc[2 * kk + 1][0], c1 = sacc[2 * kk + 1][1];
                    const float ah0 = __bfloat162float(__float2bfloat16_rn(a0)), ah1 = __bfloat162float(__float2bfloat16_rn(a1));
                    const float ch0 = __bfloat162float(__float2bfloat16_rn(c0)), ch1 = __bfloat162float(__float2bfloat16_rn(c1));
                    pa[0] = pack_bf16(ah0, ah1); pa[1] = pack_bf16(a0 - ah0, a1 - ah1);
                    pa[2] = pack_bf16(ch0, ch1); pa[3] = pack_bf16(c0 - ch0, c1 - ch1);
                }
#pragma unroll
                for (int jj = 0; jj < HD / 16; ++jj) {
                    unsigned b[4];
                    ldsm_x4_trans(b, vb + (unsigned)((16 * kk + (lane & 7) + 8 * ((lane >> 3) & 1)) * PK + (16 * jj + 8 * (lane >> 4)) * 2));
                    mma_bf16(oacc[2 * jj], pa[0], pa[1], pa[2], pa[3], b[0], b[1]);
                    mma_bf16(oacc[2 * jj + 1], pa[0], pa[1], pa[2], pa[3], b[2], b[3]);
                }
            }
        }
        __syncthreads();  // the stage is rewritten by the next iteration's copies
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    const int rr = warp * 8 + g;
    const int tl = rr / G, head = rr - tl * G;
    if (tl < n_tok) {
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        __nv_bfloat16* orow = p.out + (size_t)(tok0 + tl) * p.out_stride + (size_t)(kvh * G + head) * HD;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j)
            *reinterpret_cast<unsigned*>(orow + 8 * j + 2 * t) = pack_bf16((oacc[j][0] + oacc[j][2]) * inv, (oacc[j][1] + oacc[j][3]) * inv);
    }
}

int attn_init() {
    SWLM_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_prefill_smem<128>()));
    SWLM_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_prefill_smem<64>()));
    return SWLM_OK;
}

int attn_pick_splits(int m, int kv_heads, int max_ctx) {
    static const int forced = [] { const char* v = getenv("SWLM_ATTN_SPLITS"); return v ? atoi(v) : 0; }();
    if (forced >= 1 && forced <= 64) return forced;
    if (m <= 0 || kv_heads <= 0) return 1;
    int s = 300 / (m * kv_heads);
    const int cap = max_ctx / 128;
    if (s > 32) s = 32;
    if (s > cap) s = cap;
    if (s < 1) s = 1;
    return s;
}

size_t attn_scratch_floats(int m, int heads, int head_dim, int splits) {
    return (size_t)m * heads * splits * (head_dim + 2);
}

static int check_group(int heads, int kv_heads) {
    if (kv_heads <= 0 || heads % kv_heads || heads / kv_heads > kMaxGroup) {
        set_error("attention: %d query heads per KV head not supported (max %d)", kv_heads ? heads / kv_heads : 0, kMaxGroup);
        return SWLM_ERR_UNSUPPORTED;
    }
    return SWLM_OK;
}

int launch_attn_decode(const AttnLaunch& a, cudaStream_t s) {
    int rc = check_group(a.heads, a.kv_heads);
    if (rc) return rc;
    if (a.rope_dim > a.head_dim || (a.rope_dim & 1)) { set_error("attention: bad rope_dim"); return SWLM_ERR_INVALID; }
    if (((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v) | reinterpret_cast<uintptr_t>(a.out)) & 15) ||
        ((a.q_stride | a.k_stride | a.v_stride | a.out_stride) & 7)) {
        set_error("attention: q, k, v and out rows must be 16-byte aligned");
        return SWLM_ERR_INVALID;
    }
    AttnParams p{};
    p.heads = a.heads; p.kv_heads = a.kv_heads; p.rope_dim = a.rope_dim; p.max_seq = a.max_seq; p.splits = a.splits;
    p.scale_log2 = a.scale * kLog2e;
    p.inv_freq = a.inv_freq;
    p.q = a.q; p.q_stride = a.q_stride; p.k = a.k; p.k_stride = a.k_stride; p.v = a.v; p.v_stride = a.v_stride;
    p.kcache = a.kcache; p.vcache = a.vcache;
    p.cache_head_stride = (size_t)a.max_seq * a.head_dim;
    p.cache_seq_stride = p.cache_head_stride * a.kv_heads;
    p.position = a.position; p.ctx_len = 0; p.window = a.window > 0 ? a.window : 0;
    static const int q_first = [] { const char* v = getenv("SWLM_ATTN_QFIRST"); return v ? atoi(v) : 0; }();
    p.q_first = q_first;
    p.out = a.out; p.out_stride = a.out_stride;
    p.part_o = a.scratch;
    p.part_ml = a.scratch + (size_t)a.m * a.heads * a.splits * a.head_dim;
    p.counters = a.counters;
    p.prefetch = a.prefetch;
    if (a.pos_base < 0 && a.m * a.kv_heads * a.splits + a.m * a.kv_heads <= 512)
        p.trace = qgemv_trace_slot(a.m * a.kv_heads * a.splits, -a.kv_heads * a.m, a.splits, 9, 0);
    if (swlm_kv_bits(a.kv_scheme)) {
        if (a.pos_base >= 0) { set_error("attention: prompt chunks over a quantized cache are not supported"); return SWLM_ERR_UNSUPPORTED; }
        p.kv_bits = swlm_kv_bits(a.kv_scheme); p.kv_group = swlm_kv_group(a.kv_scheme);
        if (p.kv_group > a.head_dim) { set_error("attention: cache groups of %d values exceed head_dim %d", p.kv_group, a.head_dim); return SWLM_ERR_UNSUPPORTED; }
        const dim3 grid(p.splits, p.kv_heads, a.m);
        const int G = a.heads / a.kv_heads;
        if (a.head_dim != 64 && a.head_dim != 128) { set_error("attention: head_dim %d not supported over an 8-bit cache (64 or 128)", a.head_dim); return SWLM_ERR_UNSUPPORTED; }
        if (G != 1 && G != 2 && G != 4 && G != 8) { set_error("attention over an 8-bit cache: %d query heads per KV head (1, 2, 4 or 8)", G); return SWLM_ERR_UNSUPPORTED; }
        const bool rotor = swlm_kv_is_rotor(a.kv_scheme);
        if (rotor) {
            if (!a.rotors || a.qjl_dim < 0 || a.qjl_dim > 64 || (a.qjl_dim > 0 && (!a.qjl_matrix || !a.qjl_res))) {
                set_error("attention over a rotated cache: rotors, projection matrix or residual rows missing (qjl_dim %d)", a.qjl_dim);
                return SWLM_ERR_INVALID;
            }
            p.rotors = a.rotors; p.qjl_matrix = a.qjl_matrix; p.qjl_res = a.qjl_res; p.qjl_dim = a.qjl_dim;
        }
#define SWLM_Q8_CASE(HDV, GV) if (a.head_dim == HDV && G == GV) { \
            if (rotor) { \
                if (p.kv_bits == 8) launch_k(attn_q8_split_kernel<HDV, GV, 8, true>, grid, dim3(kQ8Threads), 0, s, p); \
                else launch_k(attn_q8_split_kernel<HDV, GV, 4, true>, grid, dim3(kQ8Threads), 0, s, p); \
            } else if (p.kv_bits == 8) launch_k(attn_q8_split_kernel<HDV, GV, 8, false>, grid, dim3(kQ8Threads), 0, s, p); \
            else launch_k(attn_q8_split_kernel<HDV, GV, 4, false>, grid, dim3(kQ8Threads), 0, s, p); }
        SWLM_Q8_CASE(128, 1); SWLM_Q8_CASE(128, 2); SWLM_Q8_CASE(128, 4); SWLM_Q8_CASE(128, 8);
        SWLM_Q8_CASE(64, 1); SWLM_Q8_CASE(64, 2); SWLM_Q8_CASE(64, 4); SWLM_Q8_CASE(64, 8);
#undef SWLM_Q8_CASE
        return check_launch("attention (8-bit cache) launch");
    }
    if (a.pos_base >= 0) {
        // prompt ingestion: rows of q/k/v are consecutive tokens of sequence 0
        if (a.head_dim > 128) { set_error("attention: head_dim %d not supported", a.head_dim); return SWLM_ERR_UNSUPPORTED; }
        p.pos_base = a.pos_base;
        p.chunk_tokens = a.m;
        cudaError_t e = launch_k(rope_append_kernel, dim3(a.m, a.kv_heads, 1), dim3(128), 0, s, p, a.head_dim);
        if (e != cudaSuccess) return cuda_fail(e, "rope_append launch");
        // tiled causal kernel when the GQA group fills the 8 rows of a warp evenly; SWLM_PREFILL_ATTN=0 keeps the
        // per-token kernel (for comparisons)
        static const bool tiled = [] { const char* v = getenv("SWLM_PREFILL_ATTN"); return !(v && v[0] == '0'); }();
        const int G = a.heads / a.kv_heads;
        if (tiled && (G == 1 || G == 2 || G == 4 || G == 8) && (a.head_dim == 64 || a.head_dim == 128) && a.rope_dim <= a.head_dim) {
            const dim3 grid((unsigned)((a.m + kPfRows / G - 1) / (kPfRows / G)), (unsigned)a.kv_heads, 1);
            e = a.head_dim == 128 ? launch_k(attn_prefill_kernel<128>, grid, dim3(kPfThreads), attn_prefill_smem<128>(), s, p)
                                  : launch_k(attn_prefill_kernel<64>, grid, dim3(kPfThreads), attn_prefill_smem<64>(), s, p);
            if (e != cudaSuccess) return cuda_fail(e, "attn_prefill launch");
            return SWLM_OK;
        }
        return launch_both<2>(p, a.m, a.head_dim, s);
    }
    return launch_both<1>(p, a.m, a.head_dim, s);
}

int launch_flash_decode_plain(int m, int heads, int kv_heads, int hd, int ctx_len, int ctx_stride, float scale,
                              const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                              __nv_bfloat16* out, float* scratch, unsigned* counters, int splits, cudaStream_t s) {
    int rc = check_group(heads, kv_heads);
    if (rc) return rc;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15) { set_error("flash-decode: q and out must be 16-byte aligned"); return SWLM_ERR_INVALID; }
    AttnParams p{};
    p.heads = heads; p.kv_heads = kv_heads; p.rope_dim = 0; p.max_seq = ctx_stride; p.splits = splits;
    p.scale_log2 = scale * kLog2e;
    p.q = q; p.q_stride = heads * hd;
    p.kcache = const_cast<__nv_bfloat16*>(k); p.vcache = const_cast<__nv_bfloat16*>(v);
    p.cache_head_stride = (size_t)ctx_stride * hd;
    p.cache_seq_stride = p.cache_head_stride * kv_heads;
    p.position = nullptr; p.ctx_len = ctx_len;
    p.out = out; p.out_stride = heads * hd;
    p.part_o = scratch;
    p.part_ml = scratch + (size_t)m * heads * splits * hd;
    p.counters = counters;
    return launch_both<0>(p, m, hd, s);
}

// ---- allocation-free flash-decode ---------------------------------------------------------------------
// Some embedders may not allocate device memory once they are running: a serving loop that reserved its
// whole memory budget at start-up and treats any later cudaMalloc as a bug (it synchronises the device and
// can fail under memory pressure), or a host runtime that owns the allocator and hands this library no
// pool of its own. For them the partial results and arrival counters of the split kernel live in a fixed
// array that is part of the loaded module instead of in caller- or library-allocated scratch.
//
// The array is 8 MiB on every GPU that loads the library, for the life of the process. All calls share it
// and it keeps the previous call's contents: the counters are cleared (asynchronously, on the call's
// stream) before every launch, the partials are overwritten before they are read. Two calls that overlap
// on the GPU (different streams, no ordering between them) would race on it; serialise them.
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_flash_static_scratch[kStaticScratchBytes];
// device address of the array, per device ordinal. Written by whichever thread calls first on a device; every writer
// stores the same value, and the slot is an atomic so that concurrent first calls are a defined program.
static std::atomic<void*> g_flash_static_addr[64];

size_t flash_decode_static_capacity() { return kStaticScratchBytes; }

int launch_flash_decode_static(int device, int m, int heads, int kv_heads, int hd, int ctx_len, int ctx_stride, float scale,
                               const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, __nv_bfloat16* out,
                               cudaStream_t s) {
    if (device < 0 || device >= 64) { set_error("flash-decode (static scratch): device ordinal %d out of range", device); return SWLM_ERR_INVALID; }
    if (!g_flash_static_addr[device].load(std::memory_order_acquire)) {
        // In host code the array's name is only a handle; the kernel needs the device address, which the
        // runtime resolves for the device that is current now. Done once per device, on the first call.
        void* addr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&addr, g_flash_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(flash-decode static scratch)");
        g_flash_static_addr[device].store(addr, std::memory_order_release);
    }
    const int splits = attn_pick_splits(m, kv_heads, ctx_len);
    const size_t counter_bytes = (((size_t)m * kv_heads * sizeof(unsigned)) + 255) / 256 * 256;
    const size_t need = counter_bytes + attn_scratch_floats(m, heads, hd, splits) * sizeof(float);
    if (need > kStaticScratchBytes) {
        set_error("flash-decode (static scratch): batch %d x %d heads x %d splits needs %zu bytes, the built-in scratch holds %zu",
                  m, heads, splits, need, kStaticScratchBytes);
        return SWLM_ERR_INVALID;
    }
    unsigned char* base = static_cast<unsigned char*>(g_flash_static_addr[device].load(std::memory_order_acquire));
    SWLM_CUDA(cudaMemsetAsync(base, 0, counter_bytes, s));  // arrival counters must start at zero
    return launch_flash_decode_plain(m, heads, kv_heads, hd, ctx_len, ctx_stride, scale, q, k, v, out,
                                     reinterpret_cast<float*>(base + counter_bytes), reinterpret_cast<unsigned*>(base), splits, s);
}

}  // namespace swlm
