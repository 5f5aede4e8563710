// Latency-bound glue kernels of the decode step: fused residual/RMSNorm, per-head QK norm,
// embedding gather, SwiGLU, gated short-conv state update, greedy argmax. Each is a few KB of
// traffic; the design goal is one launch where the reference needs two or three, 128-bit accesses,
// and bf16 rounding at exactly the points where the reference stores to a bf16 buffer.
#include "swlm_internal.h"

namespace swlm {
namespace {

__device__ __forceinline__ float bf_lo(unsigned w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(unsigned w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ unsigned pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<unsigned*>(&v);
}

__device__ __forceinline__ float block_sum(float v, float* red) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < nw; ++i) total += red[i];  // same order in every thread
    __syncthreads();
    return total;
}

// Replaces fused_copy_rms_norm / fused_residual_add_copy_rms_norm / fused_residual_add_rms_norm
// (Primitives/Reduction.swift:74-115 synthesized with CopyFragment and ResidualAddFragment,
// Compiler/MetalEntryCollector.swift:143-218). One CTA per sequence; h is kept in shared memory
// in fp32 so the norm sees the unrounded sum, as the reference's fused kernel does.
template <int MODE>  // 0 copy+norm, 1 add+copy+norm, 2 add+norm
__global__ void __launch_bounds__(256) rmsnorm_kernel(int dim, const __nv_bfloat16* in, int in_stride,
                                                     __nv_bfloat16* residual, int res_stride,
                                                     const __nv_bfloat16* weight, float eps, float weight_bias,
                                                     __nv_bfloat16* out, int out_stride) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float hbuf[];
    __shared__ float red[8];
    const int b = blockIdx.x;
    const uint4* in4 = reinterpret_cast<const uint4*>(in + (size_t)b * in_stride);
    uint4* res4 = reinterpret_cast<uint4*>(residual + (size_t)b * res_stride);
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) {
        const uint4 v = in4[i];
        float h[8] = {bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y), bf_lo(v.z), bf_hi(v.z), bf_lo(v.w), bf_hi(v.w)};
        if (MODE != 0) {
            const uint4 r = res4[i];
            h[0] += bf_lo(r.x); h[1] += bf_hi(r.x); h[2] += bf_lo(r.y); h[3] += bf_hi(r.y);
            h[4] += bf_lo(r.z); h[5] += bf_hi(r.z); h[6] += bf_lo(r.w); h[7] += bf_hi(r.w);
        }
        if (MODE != 2) res4[i] = make_uint4(pack_bf16(h[0], h[1]), pack_bf16(h[2], h[3]), pack_bf16(h[4], h[5]), pack_bf16(h[6], h[7]));
#pragma unroll
        for (int e = 0; e < 8; ++e) { hbuf[i * 8 + e] = h[e]; ss = fmaf(h[e], h[e], ss); }
    }
    const float total = block_sum(ss, red);
    const float rs = rsqrtf(total / (float)dim + eps);
    const uint4* w4 = reinterpret_cast<const uint4*>(weight);
    uint4* out4 = reinterpret_cast<uint4*>(out + (size_t)b * out_stride);
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) {
        const uint4 w = w4[i];
        const float wf[8] = {bf_lo(w.x), bf_hi(w.x), bf_lo(w.y), bf_hi(w.y), bf_lo(w.z), bf_hi(w.z), bf_lo(w.w), bf_hi(w.w)};
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = hbuf[i * 8 + e] * rs * (wf[e] + weight_bias);
        out4[i] = make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
    }
}

// batched_qk_rms_norm_2 (Generator/MetalSourceGenerator+Batched.swift:681-760): one warp per head.
__global__ void qk_norm_kernel(int heads, int kv_heads, int head_dim, __nv_bfloat16* q, int q_stride,
                               __nv_bfloat16* k, int k_stride, const __nv_bfloat16* wq, const __nv_bfloat16* wk,
                               float eps, float weight_bias) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int head = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (head >= heads + kv_heads) return;
    __nv_bfloat16* data = head < heads ? q + (size_t)b * q_stride + (size_t)head * head_dim
                                       : k + (size_t)b * k_stride + (size_t)(head - heads) * head_dim;
    const __nv_bfloat16* w = head < heads ? wq : wk;
    float ss = 0.f;
    for (int i = lane; i < head_dim; i += 32) { const float v = __bfloat162float(data[i]); ss = fmaf(v, v, ss); }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rs = rsqrtf(ss / (float)head_dim + eps);
    for (int i = lane; i < head_dim; i += 32)
        data[i] = __float2bfloat16_rn(__bfloat162float(data[i]) * rs * (__bfloat162float(w[i]) + weight_bias));
}

// embedding_lookup_bf16 (Generator/MetalSourceGenerator+Embedding.swift:3-48).
__global__ void embed_kernel(int dim, const int32_t* tokens, int vocab, const __nv_bfloat16* table,
                             __nv_bfloat16* out, int out_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    int tok = tokens[b];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)tok * dim);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)b * out_stride);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < dim / 8) dst[i] = src[i];
}

// embedding_lookup_q4 (Generator/MetalSourceGenerator+Embedding.swift:79-154): row gather from a Q4 group-64 table in
// the packed source layout, value = bf16(q * scale + zero). One thread per 8 consecutive elements (one packed word).
__global__ void embed_q4_kernel(int dim, const int32_t* tokens, int vocab, const uint32_t* w, const uint16_t* scales,
                                const uint16_t* zeros, int sb_f16, __nv_bfloat16* out, int out_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    int tok = tokens[b];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;   // word index in the row
    if (i >= dim / 8) return;
    const unsigned word = w[(size_t)tok * (dim / 8) + i];
    const size_t g = (size_t)tok * (dim / 64) + (i >> 3);
    const float s = sb_f16 ? __half2float(__ushort_as_half(scales[g])) : __uint_as_float((unsigned)scales[g] << 16);
    const float z = sb_f16 ? __half2float(__ushort_as_half(zeros[g])) : __uint_as_float((unsigned)zeros[g] << 16);
    unsigned o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(fmaf((float)((word >> (8 * j)) & 0xFu), s, z),
                                                       fmaf((float)((word >> (8 * j + 4)) & 0xFu), s, z));
        o[j] = *reinterpret_cast<const unsigned*>(&v);
    }
    reinterpret_cast<uint4*>(out + (size_t)b * out_stride)[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

// swiglu (Primitives/ElementwiseFragment.swift:49-54); used only when the plan cannot fold it
// into the gate/up GEMV epilogue.
__global__ void swiglu_kernel(int n, const __nv_bfloat16* gate, int g_stride, const __nv_bfloat16* up, int u_stride,
                              __nv_bfloat16* out, int o_stride, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = __bfloat162float(gate[(size_t)b * g_stride + i]);
    const float u = __bfloat162float(up[(size_t)b * u_stride + i]);
    out[(size_t)b * o_stride + i] = __float2bfloat16_rn(gated_activation(g, u, act));
}

// the same, eight elements per thread with 128-bit accesses (rows of many tokens in prompt ingestion)
__global__ void swiglu8_kernel(int n8, const uint4* gate, int g_stride8, const uint4* up, int u_stride8, uint4* out, int o_stride8, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const uint4 gv = gate[(size_t)b * g_stride8 + i], uv = up[(size_t)b * u_stride8 + i];
    const unsigned gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
    unsigned ow[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float g0 = __uint_as_float(gw[j] << 16), g1 = __uint_as_float(gw[j] & 0xffff0000u);
        const float u0 = __uint_as_float(uw[j] << 16), u1 = __uint_as_float(uw[j] & 0xffff0000u);
        const __nv_bfloat162 o = __floats2bfloat162_rn(gated_activation(g0, u0, act), gated_activation(g1, u1, act));
        ow[j] = *reinterpret_cast<const unsigned*>(&o);
    }
    out[(size_t)b * o_stride8 + i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

// conv_state_update_bf16 (Generator/MetalSourceGenerator+ConvAndState.swift:27-70): in = B|C|x,
// state [kernel][dim] bf16 shifted by one, newest entry stored rounded but used unrounded.
__global__ void conv_step_kernel(int dim, int kernel, __nv_bfloat16* state, size_t state_seq_stride,
                                 const __nv_bfloat16* in, int in_stride, const __nv_bfloat16* weight,
                                 __nv_bfloat16* out, int out_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= dim) return;
    const __nv_bfloat16* x = in + (size_t)b * in_stride;
    __nv_bfloat16* st = state + (size_t)b * state_seq_stride;
    const float B = __bfloat162float(x[c]), C = __bfloat162float(x[dim + c]), xv = __bfloat162float(x[2 * dim + c]);
    const float Bx = B * xv;
    float acc = 0.f;
    for (int k = 0; k + 1 < kernel; ++k) {
        const __nv_bfloat16 s = st[(size_t)(k + 1) * dim + c];
        st[(size_t)k * dim + c] = s;
        acc += __bfloat162float(s) * __bfloat162float(weight[(size_t)c * kernel + k]);
    }
    st[(size_t)(kernel - 1) * dim + c] = __float2bfloat16_rn(Bx);
    acc += Bx * __bfloat162float(weight[(size_t)c * kernel + (kernel - 1)]);
    out[(size_t)b * out_stride + c] = __float2bfloat16_rn(C * acc);
}

// The same update over `tokens` consecutive prompt tokens of one sequence: a thread keeps its channel's window in
// registers and walks the tokens in order, so every intermediate value (and the state left behind) is bit for bit
// what `tokens` single steps produce.
constexpr int kConvMaxKernel = 8;
__global__ void conv_prefill_kernel(int dim, int kernel, int tokens, __nv_bfloat16* state, const __nv_bfloat16* in,
                                    int in_stride, const __nv_bfloat16* weight, __nv_bfloat16* out, int out_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= dim) return;
    float win[kConvMaxKernel], w[kConvMaxKernel];
#pragma unroll
    for (int k = 0; k < kConvMaxKernel; ++k) {
        win[k] = k < kernel ? __bfloat162float(state[(size_t)k * dim + c]) : 0.f;
        w[k] = k < kernel ? __bfloat162float(weight[(size_t)c * kernel + k]) : 0.f;
    }
    for (int tkn = 0; tkn < tokens; ++tkn) {
        const __nv_bfloat16* x = in + (size_t)tkn * in_stride;
        const float B = __bfloat162float(x[c]), C = __bfloat162float(x[dim + c]), xv = __bfloat162float(x[2 * dim + c]);
        const float Bx = B * xv;
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k + 1 < kConvMaxKernel; ++k)
            if (k + 1 < kernel) { win[k] = win[k + 1]; acc += win[k] * w[k]; }
#pragma unroll
        for (int k = 0; k < kConvMaxKernel; ++k)
            if (k == kernel - 1) { win[k] = __bfloat162float(__float2bfloat16_rn(Bx)); acc += Bx * w[k]; }
        out[(size_t)tkn * out_stride + c] = __float2bfloat16_rn(C * acc);
    }
#pragma unroll
    for (int k = 0; k < kConvMaxKernel; ++k)
        if (k < kernel) state[(size_t)k * dim + c] = __float2bfloat16_rn(win[k]);
}

// ---- argmax -----------------------------------------------------------------------------------------
// Replaces the single-threadgroup `argmax` (Generator/MetalSourceGenerator+Sampling.swift:62-107) with a
// two-level reduction. Lowest index wins among equal maxima.
constexpr int kArgmaxBlocks = 128;

__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

__global__ void __launch_bounds__(256) argmax_partial_kernel(int n, const __nv_bfloat16* logits, int stride,
                                                            float* pval, int32_t* pidx) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const __nv_bfloat16* row = logits + (size_t)b * stride;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = __bfloat162float(row[i]);
        if (v > best) { best = v; bi = i; }   // i ascends within a thread: first maximum is kept
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_merge(best, bi, ov, oi);
    }
    __shared__ float sv[8];
    __shared__ int si[8];
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) argmax_merge(best, bi, sv[w], si[w]);
        pval[b * kArgmaxBlocks + blockIdx.x] = best;
        pidx[b * kArgmaxBlocks + blockIdx.x] = bi;
    }
}

// one warp per sequence; finally thread 0 advances the device-side position and step counter.
// Tensor parallel (vocabulary sharded): every rank pushes its local (max, global index) per sequence into
// every rank's exchange buffer, waits (bounded) for the others and takes the best pair, lowest index first
// among equal maxima, so all ranks continue with the same token.
__global__ void argmax_final_kernel(int m, const float* pval, const int32_t* pidx, int32_t* token_out,
                                    int32_t* token_in_next, int32_t* ring, int32_t* step_counter, int ring_cap,
                                    int32_t* position, int advance, TpParams tp, int32_t* am_epoch, int shard_offset) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ float best_v[kMaxSequences];
    __shared__ int best_i[kMaxSequences];
    for (int b = warp; b < m; b += (blockDim.x >> 5)) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = lane; i < kArgmaxBlocks; i += 32) argmax_merge(best, bi, pval[b * kArgmaxBlocks + i], pidx[b * kArgmaxBlocks + i]);
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_merge(best, bi, ov, oi);
        }
        if (lane == 0) {
            if (bi == 0x7fffffff) bi = 0;
            best_v[b] = best; best_i[b] = bi + shard_offset;
        }
    }
    __syncthreads();
    if (tp.tp > 1) {
        const int epoch = *am_epoch + 1, par = epoch & 1;
        for (int idx = threadIdx.x; idx < m * tp.tp; idx += blockDim.x) {
            const int b = idx / tp.tp, r = idx - b * tp.tp;
            float2* dst = reinterpret_cast<float2*>(tp.peer[r] + tp.lay.recv_am(par, tp.rank, b));
            *dst = make_float2(best_v[b], __int_as_float(best_i[b]));
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x < tp.tp)
            st_release_sys(reinterpret_cast<unsigned*>(tp.peer[threadIdx.x] + tp.lay.flags_am(par, tp.rank)), (unsigned)epoch);
        tp_wait_flags(tp, tp.peer[tp.rank], tp.lay.flags_am(par, 0), epoch, threadIdx.x);
        __syncthreads();
        if (threadIdx.x < m) {
            const int b = threadIdx.x;
            float best = -INFINITY;
            int bi = 0x7fffffff;
            for (int src = 0; src < tp.tp; ++src) {
                const float2 v = __ldcg(reinterpret_cast<const float2*>(tp.peer[tp.rank] + tp.lay.recv_am(par, src, b)));
                argmax_merge(best, bi, v.x, __float_as_int(v.y));
            }
            best_v[b] = best; best_i[b] = bi == 0x7fffffff ? 0 : bi;
        }
        __syncthreads();
        if (threadIdx.x == 0) *am_epoch = epoch;
    }
    if (threadIdx.x < m) {
        const int b = threadIdx.x, bi = best_i[b];
        token_out[b] = bi;
        if (token_in_next) token_in_next[b] = bi;
        if (ring) ring[(size_t)(step_counter[0] % ring_cap) * m + b] = bi;
    }
    __syncthreads();
    if (advance) {   // every sequence has its own position
        if (threadIdx.x < m) position[threadIdx.x] += 1;
        if (threadIdx.x == 0) step_counter[0] += 1;
    }
}

__global__ void fill_u32_kernel(uint32_t* p, size_t n, uint32_t v) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}
__global__ void advance_kernel(int m, int32_t* position, int32_t* step_counter) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x < m) position[threadIdx.x] += 1;
    if (step_counter && threadIdx.x == 0) step_counter[0] += 1;
}

// ---- tensor parallel: all-reduce of a prompt chunk's partial rows ------------------------------------------------
// Push: rows x hidden bf16 of this rank into slot [parity][this rank] of every rank's exchange buffer (plain peer
// stores, 16 bytes each); the last CTA to finish raises the flag on every rank.
__global__ void tp_rows_push_kernel(TpParams tp, const __nv_bfloat16* x, int x_stride, int rows, int hidden, int epoch,
                                    unsigned* done_counter) {
    pdl_launch_dependents();
    pdl_wait();
    const int par = epoch & 1, vec_per_row = hidden / 8;
    const size_t n_vec = (size_t)rows * vec_per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / vec_per_row), c = (int)(i - (size_t)r * vec_per_row);
        const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)r * x_stride + (size_t)c * 8);
        for (int dst = 0; dst < tp.tp; ++dst)
            *reinterpret_cast<uint4*>(tp.peer[dst] + tp.lay.recv_rows(par, tp.rank) + ((size_t)r * hidden + (size_t)c * 8) * 2) = v;
    }
    __threadfence_system();
    __syncthreads();
    __shared__ int last;
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(done_counter, 1u);
        last = prev == gridDim.x - 1;
        if (last) *done_counter = 0u;   // ready for the next exchange
    }
    __syncthreads();
    if (last && threadIdx.x < tp.tp)
        st_release_sys(reinterpret_cast<unsigned*>(tp.peer[threadIdx.x] + tp.lay.flags_rows(par, tp.rank)), (unsigned)epoch);
}

// Reduce: wait (bounded) for every rank's flag, then x = bf16(sum over ranks, in rank order, in fp32).
__global__ void tp_rows_reduce_kernel(TpParams tp, __nv_bfloat16* x, int x_stride, int rows, int hidden, int epoch) {
    pdl_launch_dependents();
    pdl_wait();
    const int par = epoch & 1, vec_per_row = hidden / 8;
    const unsigned char* own = tp.peer[tp.rank];
    if (*reinterpret_cast<volatile int*>(tp.status) == 0) tp_wait_flags(tp, own, tp.lay.flags_rows(par, 0), epoch, threadIdx.x);
    __syncthreads();
    const size_t n_vec = (size_t)rows * vec_per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / vec_per_row), c = (int)(i - (size_t)r * vec_per_row);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int src = 0; src < tp.tp; ++src) {
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(own + tp.lay.recv_rows(par, src) + ((size_t)r * hidden + (size_t)c * 8) * 2));
            const unsigned u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) { acc[2 * j] += __uint_as_float(u[j] << 16); acc[2 * j + 1] += __uint_as_float(u[j] & 0xffff0000u); }
        }
        uint4 o;
        o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
        o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(x + (size_t)r * x_stride + (size_t)c * 8) = o;
    }
}

// ssm_recurrence (Generator/MetalSourceGenerator+ConvAndState.swift:347-497): one block per (key group, sequence). The
// block's channels (q and k of the group, v of its heads) go through the conv shift + SiLU into shared memory; then
// one thread per (head, value dimension) walks the key dimension of the fp32 state twice (decay + read, then the full
// write), so consecutive threads touch consecutive state elements; then the RMS norm over the value dimension and the
// z gate. The arithmetic keeps the reference's order; the un-normalised output is rounded to the buffer type before
// the norm, as there.
__device__ __forceinline__ float ssm_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float ssm_softplus(float x) { return fmaxf(x, 0.0f) + logf(1.0f + expf(-fabsf(x))); }

__global__ void ssm_recurrence_kernel(const SsmLaunch a) {
    pdl_launch_dependents();
    extern __shared__ float ssm_smem[];
    const int tid = threadIdx.x, T = blockDim.x;
    const int dk = a.key_dim, dv = a.value_dim, K = a.kernel;
    const int groups = gridDim.x, hpg = a.heads / groups;
    const int kgd = groups * dk, conv_dim = 2 * kgd + a.heads * dv;
    const int g = blockIdx.x, b = blockIdx.y, head0 = g * hpg;
    const int local_dim = 2 * dk + hpg * dv;
    float* act = ssm_smem;                   // [local_dim]: q, k, then v of the group's heads
    float* dots = act + local_dim;           // [hpg * dv]: un-normalised outputs as stored
    float* partial = dots + hpg * dv;        // [T]
    pdl_wait();
    __nv_bfloat16* cstate = a.conv_state + (size_t)b * a.conv_seq_stride;
    const int tph = min(T / hpg, dv), active = hpg * tph;   // threads per head
    const int lh = tid / tph, head = head0 + lh, lt = tid - lh * tph;
    const int chunk = dv / tph, d0 = lt * chunk, d1 = lt + 1 == tph ? dv : d0 + chunk;
    // every channel, state column and output element belongs to the same thread at every token, so walking a chunk's
    // tokens in order needs no synchronisation beyond the barriers of one step
    for (int tok = 0; tok < a.tokens; ++tok) {
    const int row = b + tok;   // decode: sequence b; prompt chunk: token `tok` of the one sequence
    const __nv_bfloat16* qkv = a.qkv + (size_t)row * a.qkv_stride;
    for (int lc = tid; lc < local_dim; lc += T) {
        const int ch = lc < dk ? g * dk + lc : lc < 2 * dk ? kgd + g * dk + (lc - dk) : 2 * kgd + head0 * dv + (lc - 2 * dk);
        float sum = 0.f;
        for (int k = 0; k + 1 < K; ++k) {
            const __nv_bfloat16 v = cstate[(size_t)(k + 1) * conv_dim + ch];
            cstate[(size_t)k * conv_dim + ch] = v;
            sum += __bfloat162float(v) * __bfloat162float(a.conv_weight[(size_t)ch * K + k]);
        }
        const __nv_bfloat16 nv = qkv[ch];
        cstate[(size_t)(K - 1) * conv_dim + ch] = nv;
        sum += __bfloat162float(nv) * __bfloat162float(a.conv_weight[(size_t)ch * K + (K - 1)]);
        act[lc] = sum * ssm_sigmoid(sum);
    }
    __syncthreads();
    partial[tid] = 0.f;
    if (tid < active) {
        const float decay = expf(-expf(a.a_log[head]) * ssm_softplus(__bfloat162float(a.alpha[(size_t)row * a.alpha_stride + head]) + __bfloat162float(a.dt_bias[head])));
        const float beta = ssm_sigmoid(__bfloat162float(a.beta[(size_t)row * a.beta_stride + head]));
        float* S = a.state + (size_t)b * a.state_seq_stride + (size_t)head * dk * dv;
        const float* Q = act;
        const float* Kk = act + dk;
        const float* V = act + 2 * dk + lh * dv;
        float qn = 0.f, kn = 0.f, kq = 0.f;
        for (int j = 0; j < dk; ++j) { qn += Q[j] * Q[j]; kn += Kk[j] * Kk[j]; kq += Q[j] * Kk[j]; }
        const float q_inv = rsqrtf(qn + 1e-6f) * rsqrtf((float)dk), k_inv = rsqrtf(kn + 1e-6f);
        float norm_sq = 0.f;
        for (int d = d0; d < d1; ++d) {
            float kvmem = 0.f, sq = 0.f;
            for (int j = 0; j < dk; ++j) {
                const float sv = S[(size_t)j * dv + d] * decay;
                kvmem += sv * Kk[j];
                sq += sv * Q[j];
            }
            const float delta = beta * (V[d] - kvmem * k_inv);
            const float kid = k_inv * delta;
            const float dot = (sq + kid * kq) * q_inv;
            for (int j = 0; j < dk; ++j) S[(size_t)j * dv + d] = S[(size_t)j * dv + d] * decay + Kk[j] * kid;
            dots[lh * dv + d] = __bfloat162float(__float2bfloat16_rn(dot));
            norm_sq += dot * dot;
        }
        partial[tid] = norm_sq;
    }
    __syncthreads();
    if (tid < active) {
        float total = 0.f;
        for (int t = 0; t < tph; ++t) total += partial[lh * tph + t];
        const float rms = rsqrtf(total / (float)dv + 1e-6f);
        for (int d = d0; d < d1; ++d) {
            const float normed = dots[lh * dv + d] * rms * a.norm_weight[d];
            const float z = __bfloat162float(a.z[(size_t)row * a.z_stride + (size_t)head * dv + d]);
            a.out[(size_t)row * a.out_stride + (size_t)head * dv + d] = __float2bfloat16_rn(normed * z * ssm_sigmoid(z));
        }
    }
    __syncthreads();   // shared memory is reused by the next token
    }
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, what);
    return SWLM_OK;
}

}  // namespace

int launch_rmsnorm(int mode, int m, int dim, const __nv_bfloat16* in, int in_stride, __nv_bfloat16* residual,
                   int res_stride, const __nv_bfloat16* weight, float eps, float weight_bias, __nv_bfloat16* out,
                   int out_stride, cudaStream_t s) {
    if (dim % 8 || in_stride % 8 || res_stride % 8 || out_stride % 8 || dim > 12288) {
        set_error("rmsnorm: dim=%d must be a multiple of 8 and <= 12288 with 16-byte aligned rows", dim);
        return SWLM_ERR_INVALID;
    }
    const size_t smem = (size_t)dim * 4;
    switch (mode) {
    case SWLM_STEP_COPY_RMSNORM:
        launch_k(rmsnorm_kernel<0>, m, 256, smem, s, dim, in, in_stride, residual, res_stride, weight, eps, weight_bias, out, out_stride);
        break;
    case SWLM_STEP_RESADD_COPY_RMSNORM:
        launch_k(rmsnorm_kernel<1>, m, 256, smem, s, dim, in, in_stride, residual, res_stride, weight, eps, weight_bias, out, out_stride);
        break;
    case SWLM_STEP_RESADD_RMSNORM:
        launch_k(rmsnorm_kernel<2>, m, 256, smem, s, dim, in, in_stride, residual, res_stride, weight, eps, weight_bias, out, out_stride);
        break;
    default:
        set_error("rmsnorm: bad mode %d", mode);
        return SWLM_ERR_INVALID;
    }
    return check_launch("rmsnorm launch");
}

int launch_qk_norm(int m, int heads, int kv_heads, int head_dim, __nv_bfloat16* q, int q_stride, __nv_bfloat16* k,
                   int k_stride, const __nv_bfloat16* wq, const __nv_bfloat16* wk, float eps, float weight_bias,
                   cudaStream_t s) {
    const int total = heads + kv_heads;
    launch_k(qk_norm_kernel, dim3((total + 3) / 4, m), 128, 0, s, heads, kv_heads, head_dim, q, q_stride, k, k_stride, wq, wk, eps, weight_bias);
    return check_launch("qk_norm launch");
}

int launch_embed(int m, int dim, const int32_t* tokens, int vocab, const __nv_bfloat16* table, __nv_bfloat16* out,
                 int out_stride, cudaStream_t s) {
    if (dim % 8 || out_stride % 8) { set_error("embed: dim must be a multiple of 8"); return SWLM_ERR_INVALID; }
    launch_k(embed_kernel, dim3((dim / 8 + 127) / 128, m), 128, 0, s, dim, tokens, vocab, table, out, out_stride);
    return check_launch("embed launch");
}

int launch_embed_q4(int m, int dim, const int32_t* tokens, const Q4Raw& table, __nv_bfloat16* out, int out_stride, cudaStream_t s) {
    if (dim % 64 || out_stride % 8 || table.k != dim) { set_error("embed (q4): the table's width must equal the hidden size, a multiple of 64"); return SWLM_ERR_INVALID; }
    launch_k(embed_q4_kernel, dim3((dim / 8 + 127) / 128, m), 128, 0, s, dim, tokens, table.n, table.w, table.scales, table.biases,
             table.sb_f16 ? 1 : 0, out, out_stride);
    return check_launch("embed (q4) launch");
}

int launch_swiglu(int m, int n, const __nv_bfloat16* gate, int g_stride, const __nv_bfloat16* up, int u_stride,
                  __nv_bfloat16* out, int o_stride, int act, cudaStream_t s) {
    const bool vec = !((n | g_stride | u_stride | o_stride) & 7) &&
                     !((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(out)) & 15);
    if (vec)
        launch_k(swiglu8_kernel, dim3((n / 8 + 255) / 256, m), 256, 0, s, n / 8, reinterpret_cast<const uint4*>(gate), g_stride / 8,
                 reinterpret_cast<const uint4*>(up), u_stride / 8, reinterpret_cast<uint4*>(out), o_stride / 8, act);
    else
        launch_k(swiglu_kernel, dim3((n + 255) / 256, m), 256, 0, s, n, gate, g_stride, up, u_stride, out, o_stride, act);
    return check_launch("swiglu launch");
}

int launch_ssm_recurrence(const SsmLaunch& a, cudaStream_t s) {
    const int groups = a.groups > 0 ? a.groups : 1;
    if (a.heads <= 0 || a.heads % groups || a.key_dim <= 0 || a.value_dim <= 0 || a.kernel < 1 || a.m < 1 || a.tokens < 1 ||
        (a.tokens > 1 && a.m != 1)) { set_error("ssm recurrence: bad head layout"); return SWLM_ERR_INVALID; }
    const int hpg = a.heads / groups, local_dim = 2 * a.key_dim + hpg * a.value_dim;
    // a block owns one key group: enough threads for its channels and for one thread per (head, value dimension)
    int threads = std::max(local_dim, hpg * std::min(a.value_dim, 256));
    threads = std::min(1024, (threads + 31) / 32 * 32);
    if (threads / hpg < 1) { set_error("ssm recurrence: %d heads per key group exceed a block", hpg); return SWLM_ERR_UNSUPPORTED; }
    const size_t smem = ((size_t)local_dim + (size_t)hpg * a.value_dim + (size_t)threads) * sizeof(float);
    if (smem > 48 * 1024) { set_error("ssm recurrence: a key group of %d channels does not fit shared memory", local_dim); return SWLM_ERR_UNSUPPORTED; }
    launch_k(ssm_recurrence_kernel, dim3((unsigned)groups, (unsigned)a.m), dim3((unsigned)threads), smem, s, a);
    return check_launch("ssm recurrence launch");
}

int launch_conv_step(int m, int dim, int kernel, __nv_bfloat16* state, size_t state_seq_stride,
                     const __nv_bfloat16* in, int in_stride, const __nv_bfloat16* weight, __nv_bfloat16* out,
                     int out_stride, cudaStream_t s) {
    launch_k(conv_step_kernel, dim3((dim + 255) / 256, m), 256, 0, s, dim, kernel, state, state_seq_stride, in, in_stride, weight, out, out_stride);
    return check_launch("conv_step launch");
}

int launch_conv_prefill(int tokens, int dim, int kernel, __nv_bfloat16* state, const __nv_bfloat16* in, int in_stride,
                        const __nv_bfloat16* weight, __nv_bfloat16* out, int out_stride, cudaStream_t s) {
    if (kernel > kConvMaxKernel) { set_error("conv: kernel size %d not supported for prompt ingestion (max %d)", kernel, kConvMaxKernel); return SWLM_ERR_UNSUPPORTED; }
    launch_k(conv_prefill_kernel, dim3((dim + 127) / 128), 128, 0, s, dim, kernel, tokens, state, in, in_stride, weight, out, out_stride);
    return check_launch("conv_prefill launch");
}

size_t argmax_scratch_elems(int m) { return (size_t)m * kArgmaxBlocks; }

int launch_argmax(int m, int n, const __nv_bfloat16* logits, int stride, int32_t* token_out, int32_t* token_in_next,
                  int32_t* ring, int32_t* step_counter, int ring_cap, int32_t* position, int advance,
                  float* scratch_val, int32_t* scratch_idx, const TpParams& tp, int32_t* am_epoch, int shard_offset,
                  cudaStream_t s) {
    launch_k(argmax_partial_kernel, dim3(kArgmaxBlocks, m), 256, 0, s, n, logits, stride, scratch_val, scratch_idx);
    launch_k(argmax_final_kernel, 1, 256, 0, s, m, scratch_val, scratch_idx, token_out, token_in_next, ring, step_counter,
                                          ring_cap, position, advance, tp, am_epoch, shard_offset);
    return check_launch("argmax launch");
}

int launch_tp_rows_allreduce(const TpParams& tp, __nv_bfloat16* x, int x_stride, int rows, int hidden, int epoch,
                             unsigned* done_counter, cudaStream_t s) {
    if (tp.tp < 2 || rows < 1 || rows > tp.lay.rows || hidden != tp.lay.hidden || (hidden & 7) || (x_stride & 7) ||
        (reinterpret_cast<uintptr_t>(x) & 15)) {
        set_error("tensor-parallel row exchange: %d rows x %d (capacity %d x %d)", rows, hidden, tp.lay.rows, tp.lay.hidden);
        return SWLM_ERR_INVALID;
    }
    const size_t n_vec = (size_t)rows * (hidden / 8);
    const unsigned grid = (unsigned)std::min<size_t>(148, (n_vec + 1023) / 1024);
    launch_k(tp_rows_push_kernel, grid, 256, 0, s, tp, (const __nv_bfloat16*)x, x_stride, rows, hidden, epoch, done_counter);
    launch_k(tp_rows_reduce_kernel, grid, 256, 0, s, tp, x, x_stride, rows, hidden, epoch);
    return check_launch("tp rows all-reduce launch");
}

int launch_fill_u32(uint32_t* p, size_t n, uint32_t v, cudaStream_t s) {
    if (n == 0) return SWLM_OK;
    launch_k(fill_u32_kernel, (unsigned)((n + 255) / 256), 256, 0, s, p, n, v);
    return check_launch("fill launch");
}
int launch_advance(int m, int32_t* position, int32_t* step_counter, cudaStream_t s) {
    launch_k(advance_kernel, 1, kMaxSequences, 0, s, m, position, step_counter);
    return check_launch("advance launch");
}

}  // namespace swlm
