// Q4 group-64 affine GEMV / small-M GEMM for sm_100a.
//
// Replaces the reference's `gemv_q4_g64` (Generator/MetalSourceGenerator+Quantized.swift:496-575,
// one SIMD-group per output row, one byte load per weight) and, for 1 < M <= 16, its
// `gemm_q4_g64` (:88-156, which re-reads the weights once per sequence position).
//
// Design: the kernel is HBM-bound on the 0.5625 bytes/weight stream, and on B200 the
// per-weight instruction budget is the second limit, so
//   * weights are re-tiled at upload into 512-byte tiles (16 rows x 64 columns) laid out in
//     mma.m16n8k16 A-fragment order: one 16-byte load per lane per tile, no shuffles. The contraction
//     order inside a group is free, so k-step j of lane t is defined to cover columns 16t+4j..16t+4j+3:
//     the matching B fragments are then 16 consecutive activations, read as they lie in memory;
//   * the grid is persistent (at most three CTAs per SM, all resident) and the matrix is cut into
//     (row tile, k-slice) units of a few KB that are dealt out evenly, so every SM streams the same
//     number of bytes and nothing is left for a second wave; activations are staged once per CTA;
//     partial sums of a row tile meet in global scratch and the last warp to arrive adds them in
//     slice order, which keeps the result independent of scheduling;
//   * every warp streams its units through a private cp.async ring in shared memory (kStages deep)
//     that runs ahead across unit boundaries, so loads stay in flight independent of register pressure;
//   * a nibble pair becomes two fp16 values 1024+q (low nibbles) or 1024+16q (high nibbles) with one
//     LOP3 ((w & mask) | 0x64006400), one shift per four pairs; activations are converted bf16 -> fp16
//     times a per-column power of two, which is exact; the tensor core forms sum((1024+q)*x) per group
//     in fp32, and the group epilogue applies scale*(acc - 1024*sum(x)) + zero*sum(x) in fp32 —
//     algebraically the reference's sum((scale*q+zero)*x), with q and x exact and products exact in fp32;
//   * the B operand holds up to 16 sequences (columns), so batch <= 16 costs the same weight traffic.
//
// The single-sequence product (qgemv1_kernel, further down) keeps the tiles, the per-warp ring and the even
// deal, but holds the activations as block floating point (one exponent per group of 64, two signed 8-bit
// digits per element) and contracts them with the nibbles on the int8 tensor-core shape (mma.m16n8k32 u8 x s8):
// rows g of a tile take the masked low nibbles, rows g + 8 the bytes as they are, and one subtraction
// recovers the high nibbles. One CTA per SM of up to three 8-warp groups shares one copy of the activations.
// Order in the SM's memory pipeline matters: the activation loads are issued first after the wait for the
// preceding kernel and the ring stages only after them, because the product cannot start before its
// activations and a load issued behind 100 KB of weights arrives late.
#include <algorithm>
#include <cstdio>
#include <cstdlib>

#include "swlm_internal.h"
#include "tp_device.cuh"
#include "qgemv_common.cuh"

namespace swlm {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 3;                 // ring depth per warp; one stage = 4 k-tiles + their scales
constexpr int kStageBytes = 4 * 512 + 256;
constexpr int kRingBytes = kWarps * kStages * kStageBytes;
// Batch-1 kernel: a CTA is up to three groups of eight warps. The groups share one copy of the quantised
// activations (prepared once per SM instead of once per group) and otherwise behave like separate CTAs.
constexpr int kMaxGroups = 3;
constexpr int kMaxWarps1 = kMaxGroups * kWarps;
constexpr int kXPad = 8;                   // bf16 elements of padding per x row (bank skew)
constexpr int kTraceRows = 512;            // rows of four stamps per traced launch
constexpr int kL2Ahead = 10;               // stages (2.3 KB each) a warp prefetches into L2 ahead of its ring

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ uint4 lds128b(unsigned sa) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(sa));
    return v;
}
__device__ __forceinline__ float2 lds64fb(unsigned sa) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(sa));
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// one instruction asks for `bytes` (a multiple of 16, 16-byte aligned) to be brought from HBM into L2
__device__ __forceinline__ void prefetch_l2_bulk(const void* p, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
constexpr int kBulkPiece = 8;        // stages per bulk prefetch instruction (16 KB of tiles + 2 KB of pairs)
constexpr int kBulkMaxStages = 8;    // at most 18 KB per CTA requested up front (the rolling prefetch does the rest); measured:
                                     // 0 -> 582, 8 -> 585, 16 -> 575, 32 -> 563, 64 -> 541 tok/s on the Llama-3-8B shape
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_f16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                        unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float half_bits_to_float(unsigned bits16, int is_f16) {
    return is_f16 ? __half2float(__ushort_as_half((unsigned short)bits16)) : __uint_as_float(bits16 << 16);
}
// (scale, zero) pair of one row and group: scale in the low half-word, zero in the high one
template <bool F16SB>
__device__ __forceinline__ float sb_scale(unsigned pair) {
    return F16SB ? __half2float(__ushort_as_half((unsigned short)(pair & 0xFFFFu))) : __uint_as_float(pair << 16);
}
template <bool F16SB>
__device__ __forceinline__ float sb_zero(unsigned pair) {
    return F16SB ? __half2float(__ushort_as_half((unsigned short)(pair >> 16))) : __uint_as_float(pair & 0xFFFF0000u);
}


// Fused fused_copy_rms_norm / fused_residual_add_copy_rms_norm / fused_residual_add_rms_norm
// (Primitives/Reduction.swift:74-115 with CopyFragment / ResidualAddFragment,
// Compiler/MetalEntryCollector.swift:143-218) as the prologue of the product that consumes it.
// Every thread owns the run of 16 elements k0..k0+15 of row `b` (dimension <= 4096): h = in (+ residual)
// in fp32, residual_out = bf16(h) (written by one CTA only), then bf16(h * rsqrt(mean(h^2)+eps) * (w+bias))
// returned as eight packed bf16 pairs. The norm sees the unrounded sum, as the reference's fused kernel does.
// res_in and res_out are different buffers: other CTAs read res_in while one writes res_out.
__device__ __forceinline__ void fused_norm_run(const QGemvParams& p, int b, int k0, bool in_range, bool writer,
                                               float* red, unsigned (&w)[8], int tp_epoch, int nwarps = kWarps) {
    float h[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) h[i] = 0.f;
    if (in_range) {
        if (p.in_tp) {
            // all-reduce, consuming side: partial sums of every rank, added in rank order, rounded once to
            // bf16 (the value a single GPU would have stored to the hidden buffer)
            const int par = tp_epoch & 1;
#pragma unroll 1
            for (int src = 0; src < p.tp.tp; ++src) {
                const unsigned char* r = p.tp.peer[p.tp.rank] + p.tp.lay.recv_ar(par, src, b) + (size_t)k0 * 8;
                tp_add_tagged<4>(p.tp, r, tp_epoch, h);
                tp_add_tagged<4>(p.tp, r + 64, tp_epoch, h + 8);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) h[i] = __bfloat162float(__float2bfloat16_rn(h[i]));
        } else {
            const uint4* src = reinterpret_cast<const uint4*>(p.x + (size_t)b * p.x_stride + k0);
            const uint4 v0 = __ldcg(src), v1 = __ldcg(src + 1);
            const unsigned vw[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) { h[2 * i] = __uint_as_float(vw[i] << 16); h[2 * i + 1] = __uint_as_float(vw[i] & 0xFFFF0000u); }
        }
        if (p.norm_mode != SWLM_STEP_COPY_RMSNORM) {
            const uint4* rs = reinterpret_cast<const uint4*>(p.res_in + (size_t)b * p.res_stride + k0);
            const uint4 r0 = __ldcg(rs), r1 = __ldcg(rs + 1);
            const unsigned rw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) { h[2 * i] += __uint_as_float(rw[i] << 16); h[2 * i + 1] += __uint_as_float(rw[i] & 0xFFFF0000u); }
        }
        if (writer && p.norm_mode != SWLM_STEP_RESADD_RMSNORM) {
            unsigned o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const __nv_bfloat162 v = __floats2bfloat162_rn(h[2 * i], h[2 * i + 1]);
                o[i] = *reinterpret_cast<const unsigned*>(&v);
            }
            uint4* dst = reinterpret_cast<uint4*>(p.res_out + (size_t)b * p.res_stride + k0);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
    }
    // the norm weights do not depend on the sum below: requested now, used after the barriers
    uint4 n0 = make_uint4(0, 0, 0, 0), n1 = n0;
    if (in_range) {
        const uint4* ws = reinterpret_cast<const uint4*>(p.norm_w + k0);
        n0 = __ldg(ws); n1 = __ldg(ws + 1);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) ss = fmaf(h[i], h[i], ss);
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();  // red may still be read from the previous row
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < nwarps; ++i) total += red[i];
    const float rs = rsqrtf(total / (float)p.k + p.eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = 0u;
    if (in_range) {
        const unsigned nw[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(h[2 * i] * rs * (__uint_as_float(nw[i] << 16) + p.weight_bias),
                                                           h[2 * i + 1] * rs * (__uint_as_float(nw[i] & 0xFFFF0000u) + p.weight_bias));
            w[i] = *reinterpret_cast<const unsigned*>(&v);
        }
    }
}

// All-reduce, producing side: one fp32 value of row `row`, sequence `col`, into every rank's buffer.
__device__ __forceinline__ void tp_push_value(const QGemvParams& p, int epoch, int row, int col, float v) {
    const size_t off = p.tp.lay.recv_ar(epoch & 1, p.tp.rank, col) + (size_t)row * 8;
#pragma unroll 1
    for (int r = 0; r < p.tp.tp; ++r) tp_store_tagged(p.tp.peer[r] + off, v, epoch);
}
// Called by one whole warp after it pushed a row tile: the warp that completes the count advances the local
// epoch for the kernels that follow (the pushed elements carry the number themselves and need no fence).
__device__ __forceinline__ void tp_row_tile_done(const QGemvParams& p, int epoch, int lane) {
    if (lane == 0) {
        const unsigned prev = atomicAdd(p.tp.done, 1u);
        if (prev == (unsigned)p.row_tiles - 1u) {
            *p.tp.done = 0u;
            *p.tp.epoch = epoch;
        }
    }
}

// One unit of work = (row tile rt, k-slice s): 16 output rows x a contiguous run of stages.
struct UnitCursor {
    int u, u_end;     // current unit and end of this warp's sequence (stride kWarps)
    int st, st_end;   // current stage (in units of 4 k-tiles) and end of the current unit's run
    int rt;
};

template <int NT, int EPI, bool F16SB>
__global__ void __launch_bounds__(kThreads, NT == 1 ? 3 : 2) qgemv_kernel(const QGemvParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int COLS = 8 * NT;
    __shared__ unsigned colmax[COLS];
    __shared__ float colscale[COLS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // k-range of this CTA group (blockIdx.y), in stages of 4 k-tiles (256 columns)
    const int g0 = (int)(((long long)blockIdx.y * p.kt4_total) / p.sk);
    const int g1 = (int)(((long long)(blockIdx.y + 1) * p.kt4_total) / p.sk);
    const int glen = g1 - g0;
    const int nk_cta = glen * 256;
    const int xs_stride = nk_cta + kXPad;
    const int rows_x = p.m < COLS ? p.m : COLS;

    unsigned char* my_ring = smem + warp * (kStages * kStageBytes);
    __nv_bfloat16* xsm = reinterpret_cast<__nv_bfloat16*>(smem + kRingBytes);
    float* xsum = reinterpret_cast<float*>(smem + kRingBytes + (size_t)rows_x * xs_stride * 2);

    // units of this group: u = rt * si + s, s-th slice of the group's k-range
    const int units = p.row_tiles * p.si;
    // dealt cyclically: CTA b takes units 8 b .. 8 b + 7, then those 8 gridDim.x further on, ... so that at any moment
    // the whole grid reads one contiguous window of the matrix (HBM streams a sweep much faster than hundreds of
    // separate streams: the same change took the single-sequence kernel's 28672 x 4096 product from 16.8 to 14.3 us)
    const int u_lo = (int)blockIdx.x * kWarps, u_hi = units;
    const int u_step = (int)gridDim.x * kWarps;
    auto open_unit = [&](UnitCursor& c) {
        if (c.u < c.u_end) {
            c.rt = c.u / p.si;
            const int s = c.u - c.rt * p.si;
            c.st = g0 + (s * glen) / p.si;
            c.st_end = g0 + ((s + 1) * glen) / p.si;
        }
    };
    UnitCursor ic{u_lo + warp, u_hi, 0, 0, 0};  // issue side, runs kStages-1 stages ahead
    open_unit(ic);
    auto issue = [&](int slot) {
        while (ic.u < ic.u_end && ic.st >= ic.st_end) { ic.u += u_step; open_unit(ic); }
        if (ic.u < ic.u_end) {
            unsigned char* dst = my_ring + slot * kStageBytes;
            const uint4* src = p.tiles + ((size_t)ic.rt * p.kt4_total + ic.st) * 128;
#pragma unroll
            for (int q = 0; q < 4; ++q) cp_async16(dst + (q * 32 + lane) * 16, src + q * 32 + lane);
            if (lane < 16) cp_async16(dst + 2048 + lane * 16, p.sb + ((size_t)ic.rt * p.kt4_total + ic.st) * 16 + lane);
            ic.st += 1;
        }
        cp_async_commit();
    };

    // Weights do not depend on the activations or on the preceding kernel: the ring starts filling at once.
    pdl_launch_dependents();
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) issue(i);
    pdl_wait();
    // ---- x: asynchronous copy in its natural order (the tile layout was chosen so that lane t's B
    // fragments of a group are the 16 consecutive elements 16t..16t+15)-------------------------------
    __shared__ float red[kWarps];
    const int tp_epoch = (p.push || p.in_tp) ? *p.tp.epoch + (p.push ? 1 : 0) : 0;
    if (p.norm_mode) {
        // fused norm (dimension <= 4096, one CTA group): thread tid owns run tid of every row
        for (int b = 0; b < rows_x; ++b) {
            unsigned w[8];
            const int k0 = tid * 16;
            fused_norm_run(p, b, k0, k0 < p.k, blockIdx.x == 0, red, w, tp_epoch);
            if (k0 < nk_cta) {
                uint4* dst = reinterpret_cast<uint4*>(xsm + (size_t)b * xs_stride + k0);
                dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
        }
        cp_async_commit();
    } else {
        const int chunks_per_row = nk_cta / 8;
        const int total = rows_x * chunks_per_row;
        for (int idx = tid; idx < total; idx += kThreads) {
            const int b = idx / chunks_per_row, cc = idx - b * chunks_per_row;
            const int kglob = g0 * 256 + cc * 8;
            __nv_bfloat16* dst = xsm + (size_t)b * xs_stride + cc * 8;
            if (kglob < p.k) cp_async16(dst, p.x + (size_t)b * p.x_stride + kglob);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        cp_async_commit();
    }

    // ---- x: bf16 -> fp16 times a power of two (exact unless an element is 2^-24 below the column's
    // largest), in place, and the per-group sums of the converted values (the zero-point term) -----------
    cp_async_wait<0>();
    if (tid < COLS) colmax[tid] = 0;
    __syncthreads();
    {
        const int words_per_row = nk_cta / 2;
        for (int b = 0; b < rows_x; ++b) {
            const unsigned* xw = reinterpret_cast<const unsigned*>(xsm + (size_t)b * xs_stride);
            unsigned mx = 0;
            for (int i = tid; i < words_per_row; i += kThreads) {
                const unsigned w = xw[i];
                mx = max(mx, max(w & 0x7FFFu, (w >> 16) & 0x7FFFu));
            }
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            if (lane == 0) atomicMax(&colmax[b], mx);
        }
    }
    __syncthreads();
    {
        const int tasks_per_row = nk_cta / 16;
        const int total = rows_x * tasks_per_row;
        for (int base = 0; base < total; base += kThreads) {
            const int idx = base + tid;
            const bool valid = idx < total;
            float s = 0.f;
            int b = 0, c = 0;
            if (valid) {
                b = idx / tasks_per_row; c = idx - b * tasks_per_row;
                // shift the column's largest exponent to 2^13: fp16 keeps every bf16 mantissa bit
                const int e = (int)(colmax[b] >> 7);
                const int sh = (e == 0 || e == 255) ? 0 : 140 - e;
                const float mul = __uint_as_float((unsigned)(127 + max(-120, min(120, sh))) << 23);
                unsigned* xp = reinterpret_cast<unsigned*>(xsm + (size_t)b * xs_stride + c * 16);
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    const unsigned v = xp[w];
                    const __half2 h = __floats2half2_rn(__uint_as_float(v << 16) * mul, __uint_as_float(v & 0xFFFF0000u) * mul);
                    xp[w] = *reinterpret_cast<const unsigned*>(&h);
                    const float2 f = __half22float2(h);
                    s += f.x + f.y;
                }
                if (c == 0) colscale[b] = 1.0f / mul;
            }
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            if (valid && (c & 3) == 0) xsum[(c >> 2) * COLS + b] = s;
        }
    }
    __syncthreads();

    const int s_total = p.sk * p.si;  // partial results per row tile
    // per-lane shared-memory bases (32-bit): the ring, this lane's 16 activations of a k-tile for each of its batch rows
    // (second half 16 bytes on), the per-group sums. A row beyond the batch points at a block of zeros with stride 0.
    __shared__ __align__(16) unsigned zero32[8];
    if (tid < 8) zero32[tid] = 0u;
    __syncthreads();
    const unsigned ring_sa = (unsigned)__cvta_generic_to_shared(my_ring);
    const unsigned xsum_sa = (unsigned)__cvta_generic_to_shared(xsum);
    unsigned x_lane_sa[NT], x_lane_step[NT], x_lane_second[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const bool has = 8 * nt + g < p.m;
        x_lane_sa[nt] = has ? (unsigned)__cvta_generic_to_shared(xsm + (size_t)(8 * nt + g) * xs_stride + t * 16)
                            : (unsigned)__cvta_generic_to_shared(zero32);
        x_lane_step[nt] = has ? 128u : 0u;      // bytes per k-tile (64 fp16)
        x_lane_second[nt] = has ? 16u : 0u;
    }
    int islot = (kStages - 1) % kStages, cslot = 0;
    UnitCursor cc{u_lo + warp, u_hi, 0, 0, 0};
    for (; cc.u < cc.u_end; cc.u += u_step) {
        open_unit(cc);
        const int rt = cc.rt;
        float tot[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.f;

        for (int stg = cc.st; stg < cc.st_end; ++stg) {
            issue(islot); islot = islot + 1 == kStages ? 0 : islot + 1;
            cp_async_wait<kStages - 1>();
            __syncwarp();
            // every address of the stage is a 32-bit shared-memory address built from per-lane bases set up once
            const unsigned st = ring_sa + cslot * kStageBytes;
            cslot = cslot + 1 == kStages ? 0 : cslot + 1;
            const uint4 sA = lds128b(st + 2048 + g * 16), sB = lds128b(st + 2048 + (g + 8) * 16);
            const unsigned sAw[4] = {sA.x, sA.y, sA.z, sA.w};
            const unsigned sBw[4] = {sB.x, sB.y, sB.z, sB.w};
            const int ktl0 = (stg - g0) * 4;
            const unsigned xs_sa = xsum_sa + ktl0 * (COLS * 4);
#pragma unroll
            for (int ti = 0; ti < 4; ++ti) {
                const uint4 wv = lds128b(st + lane * 16 + ti * 512);
                const unsigned wr[4] = {wv.x, wv.y, wv.z, wv.w};
                uint4 X0[NT], X1[NT];
                float acc[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
                    // rows beyond the batch read a block of zeros (stride 0), so the loop has no branch
                    const unsigned xa = x_lane_sa[nt] + (ktl0 + ti) * x_lane_step[nt];
                    X0[nt] = lds128b(xa);
                    X1[nt] = lds128b(xa + x_lane_second[nt]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // fp16 1024+q from the low nibble of each byte pair, 1024+16q from the high nibble:
                    // rows g (a0, a2) carry q, rows g+8 (a1, a3) carry 16q, undone through their scale
                    const unsigned r = wr[j], r8 = r >> 8;
                    const unsigned a0 = (r & 0x000F000Fu) | 0x64006400u;
                    const unsigned a1 = (r & 0x00F000F0u) | 0x64006400u;
                    const unsigned a2 = (r8 & 0x000F000Fu) | 0x64006400u;
                    const unsigned a3 = (r8 & 0x00F000F0u) | 0x64006400u;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const unsigned b0 = j == 0 ? X0[nt].x : j == 1 ? X0[nt].z : j == 2 ? X1[nt].x : X1[nt].z;
                        const unsigned b1 = j == 0 ? X0[nt].y : j == 1 ? X0[nt].w : j == 2 ? X1[nt].y : X1[nt].w;
                        mma_f16(acc[nt], a0, a1, a2, a3, b0, b1);
                    }
                }
                // group epilogue: sum_k (s*q + z)*x = s*(acc - 1024*xsum) + z*xsum, with s/16 for rows g+8
                const float s_lo = sb_scale<F16SB>(sAw[ti]), z_lo = sb_zero<F16SB>(sAw[ti]);
                const float s_hi = sb_scale<F16SB>(sBw[ti]) * 0.0625f, z_hi = sb_zero<F16SB>(sBw[ti]);
                const float zp_lo = fmaf(-1024.f, s_lo, z_lo);
                const float zp_hi = fmaf(-1024.f, s_hi, z_hi);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const float2 xs2 = lds64fb(xs_sa + (ti * COLS + 8 * nt + 2 * t) * 4);
                    tot[nt][0] = fmaf(s_lo, acc[nt][0], fmaf(zp_lo, xs2.x, tot[nt][0]));
                    tot[nt][1] = fmaf(s_lo, acc[nt][1], fmaf(zp_lo, xs2.y, tot[nt][1]));
                    tot[nt][2] = fmaf(s_hi, acc[nt][2], fmaf(zp_hi, xs2.x, tot[nt][2]));
                    tot[nt][3] = fmaf(s_hi, acc[nt][3], fmaf(zp_hi, xs2.y, tot[nt][3]));
                }
            }
            __syncwarp();
        }
        // undo the power-of-two scaling of x
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const float c0s = colscale[min(8 * nt + 2 * t, rows_x - 1)], c1s = colscale[min(8 * nt + 2 * t + 1, rows_x - 1)];
            tot[nt][0] *= c0s; tot[nt][1] *= c1s; tot[nt][2] *= c0s; tot[nt][3] *= c1s;
        }

        // ---- partial results of a row tile meet in global scratch; the last warp to arrive sums them in
        // slice order (so the result does not depend on arrival order) and runs the epilogue -----------
        if (s_total > 1) {
            const int s_glob = blockIdx.y * p.si + (cc.u - rt * p.si);
            float* dst = p.partial + (((size_t)rt * s_total + s_glob) * 16) * COLS;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                if (8 * nt + 2 * t < p.m) {
                    __stcg(reinterpret_cast<float2*>(dst + g * COLS + 8 * nt + 2 * t), make_float2(tot[nt][0], tot[nt][1]));
                    __stcg(reinterpret_cast<float2*>(dst + (g + 8) * COLS + 8 * nt + 2 * t), make_float2(tot[nt][2], tot[nt][3]));
                }
            __threadfence();
            __syncwarp();
            unsigned prev = 0;
            if (lane == 0) prev = atomicAdd(p.counters + rt, 1u);
            prev = __shfl_sync(0xffffffffu, prev, 0);
            if (prev != (unsigned)s_total - 1u) continue;
            __threadfence();
            if (lane == 0) p.counters[rt] = 0u;  // ready for the next launch
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.f;
            for (int s = 0; s < s_total; ++s) {
                const float* src = p.partial + (((size_t)rt * s_total + s) * 16) * COLS;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    if (8 * nt + 2 * t < p.m) {
                        const float2 lo = __ldcg(reinterpret_cast<const float2*>(src + g * COLS + 8 * nt + 2 * t));
                        const float2 hi = __ldcg(reinterpret_cast<const float2*>(src + (g + 8) * COLS + 8 * nt + 2 * t));
                        tot[nt][0] += lo.x; tot[nt][1] += lo.y; tot[nt][2] += hi.x; tot[nt][3] += hi.y;
                    }
            }
        }

        // ---- epilogue --------------------------------------------------------------------------------
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int col = 8 * nt + 2 * t + e;
                if (col >= p.m) continue;
                if (EPI == QGEMV_EPI_STORE && p.push) {
#pragma unroll
                    for (int hi = 0; hi < 2; ++hi) {
                        const int r = rt * 16 + g + 8 * hi;
                        if (r < p.seg_end[0]) tp_push_value(p, tp_epoch, r, col, tot[nt][2 * hi + e]);
                    }
                } else if (EPI == QGEMV_EPI_STORE) {
#pragma unroll
                    for (int hi = 0; hi < 2; ++hi) {
                        const int r = rt * 16 + g + 8 * hi;
                        const __nv_bfloat16 val = __float2bfloat16_rn(tot[nt][2 * hi + e]);
                        if (r < p.seg_end[0]) p.y[0][(size_t)col * p.y_stride[0] + r] = val;
                        else if (r < p.seg_end[1]) p.y[1][(size_t)col * p.y_stride[1] + (r - p.seg_end[0])] = val;
                        else if (r < p.seg_end[2]) p.y[2][(size_t)col * p.y_stride[2] + (r - p.seg_end[1])] = val;
                    }
                } else {
                    // rows 0-7 of the tile are gate rows, rows 8-15 the matching up rows; both are rounded to
                    // bf16 first because the reference stores them to bf16 scratch before `swiglu` reads them
                    // (Primitives/ElementwiseFragment.swift:49-54).
                    const int r = rt * 8 + g;
                    if (r < p.seg_end[0]) {
                        const float gate = __bfloat162float(__float2bfloat16_rn(tot[nt][e]));
                        const float up = __bfloat162float(__float2bfloat16_rn(tot[nt][2 + e]));
                        p.y[0][(size_t)col * p.y_stride[0] + r] = __float2bfloat16_rn(gated_activation(gate, up, p.gated_act));
                    }
                }
            }
        }
        if (EPI == QGEMV_EPI_STORE && p.push) tp_row_tile_done(p, tp_epoch, lane);
    }
    cp_async_wait<0>();
}

// =================================================================================================
// Single-sequence kernel (m == 1), the batch-1 decode path.
//
// The fp16 tensor-core path above spends one mma.m16n8k16 per 256 weights and, on this part, saturates the
// legacy mma.sync pipe near 3.5 TB/s of weight stream; the integer dot-product instruction (dp4a) turned
// out to issue on the quarter-rate conversion pipe. Batch 1 therefore uses the 8-bit integer tensor-core
// shape m16n8k32, twice the weights per instruction and almost no unpacking: a weight word gives four
// exact 8-bit weights of row g with one AND and four of row g+8 with a shift and an AND. The activations
// are held in shared memory in block floating point: every group of 64 carries a power-of-two exponent and
// 15-bit integers split into two signed bytes, exact for every element within 2^-7 of the group's largest
// and within 2^-14 of it otherwise. High and low digits ride in columns 0 and 1 of the B operand, so one
// instruction serves both; the integer sums are exact, and the group's scale and zero are applied once in
// fp32. Same tiles, ring and unit scheduling as above.
// =================================================================================================
__device__ __forceinline__ void imma_u8s8_zero(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    const int z = 0;
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
}
__device__ __forceinline__ void imma_u8s8(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 lds128(unsigned sa) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(sa));
    return v;
}
__device__ __forceinline__ unsigned lds32(unsigned sa) {
    unsigned v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(sa));
    return v;
}
__device__ __forceinline__ float2 lds64f(unsigned sa) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(sa));
    return v;
}

// The single-sequence product. (Running o_proj, gate/up, down and the next q/k/v as one launch with a software
// grid barrier between them was tried: on this part the barrier costs about 4.5 us, more than the 0.8 us a
// dependent launch needs to see its predecessor complete, so every product is its own launch.)
template <int EPI, bool F16SB>
__device__ __forceinline__ void qgemv1_body(const QGemvParams& p, unsigned char* smem) {
    const int tid = threadIdx.x, lane = tid & 31, cta_warp = tid >> 5;
    const int groups = blockDim.x / kThreads, grp = cta_warp / kWarps;
    const int warp = cta_warp % kWarps;   // warp within its group
    const int gtid = tid % kThreads;      // thread within its group
    const int vb = grp * gridDim.x + blockIdx.x, vgrid = gridDim.x * groups;  // the group as a virtual CTA
    const int g = lane >> 2, t = lane & 3;
    const int kt_total = p.kt4_total * 4;
    if (p.trace && tid == 0) p.trace[blockIdx.x * 4] = global_timer_ns();

    const int ring_bytes = groups * kRingBytes;
    unsigned char* my_ring = smem + cta_warp * (kStages * kStageBytes);
    uint4* xq = reinterpret_cast<uint4*>(smem + ring_bytes);                       // [kt][t][hi, lo]
    float2* xmeta = reinterpret_cast<float2*>(smem + ring_bytes + (size_t)kt_total * 128);  // [kt][t] {2^E, sum}

    // Two ways of dealing out the (row tile, k-slice) units. cta_mode (matrices with no more row tiles than
    // resident CTAs): a CTA takes eight consecutive units at a time, i.e. all slices of 8/si row tiles, and
    // adds the slices through shared memory. Otherwise every CTA owns an equal contiguous share, its warps
    // take units round-robin and the slices of a row tile meet in global scratch. si is a power of two.
    const int units = p.row_tiles << p.si_shift;
    // floor(a * b / c): 32-bit when the host has checked that every such product fits (a 64-bit division costs
    // over a hundred instructions, and this set-up sits between the predecessor's end and the first load)
    auto muldiv = [&](long long a, int b, int c) {
        return p.idx32 ? (int)(((unsigned)a * (unsigned)b) / (unsigned)c) : (int)(a * b / c);
    };
    const int u_lo = muldiv(units, vb, vgrid);
    const int u_hi = muldiv(units, vb + 1, vgrid);
    const int u_first = p.cta_mode ? vb * kWarps : u_lo;
    const int u_end = p.cta_mode ? units : u_hi;
    const int u_limit = p.cta_mode ? ((units + kWarps - 1) / kWarps) * kWarps : u_hi;  // uniform across the group
    const int u_stride = p.cta_mode ? vgrid * kWarps : kWarps;
    const int si_mask = (1 << p.si_shift) - 1;
    // stages are addressed by one absolute index a = rt * kt4_total + st: tiles at a * 128, pairs at a * 16
    auto unit_range = [&](int u, int& a0, int& a1) {
        const int rt = u >> p.si_shift, sl = u & si_mask;
        a0 = rt * p.kt4_total + ((sl * p.kt4_total) >> p.si_shift);
        a1 = rt * p.kt4_total + (((sl + 1) * p.kt4_total) >> p.si_shift);
    };
    // cp.async side: runs kStages-1 stages ahead of the math, across unit boundaries
    int iu = u_first + warp, ia = 0, ia_end = 0;
    const int iu_end = u_end;
    if (iu < u_end) unit_range(iu, ia, ia_end);
    const unsigned ring_sa = (unsigned)__cvta_generic_to_shared(my_ring) + lane * 16;
    const bool sb_lane = lane < 16;
    auto issue = [&](int slot) {
        if (ia == ia_end && iu < iu_end) {
            iu += u_stride;
            if (iu < iu_end) unit_range(iu, ia, ia_end);
        }
        if (iu < iu_end) {
            const unsigned dst = ring_sa + slot * kStageBytes;
            const uint4* src = p.tiles + (size_t)ia * 128 + lane;
            asm volatile(
                "cp.async.cg.shared.global [%0], [%1], 16;\n"
                "cp.async.cg.shared.global [%0+512], [%1+512], 16;\n"
                "cp.async.cg.shared.global [%0+1024], [%1+1024], 16;\n"
                "cp.async.cg.shared.global [%0+1536], [%1+1536], 16;\n" ::"r"(dst), "l"(src) : "memory");
            if (sb_lane) {
                const uint4* ssrc = p.sb + (size_t)ia * 16 + lane;
                asm volatile("cp.async.cg.shared.global [%0+2048], [%1], 16;\n" ::"r"(dst), "l"(ssrc) : "memory");
            }
            ++ia;
        }
        cp_async_commit();
    };
    // Weights do not depend on the preceding kernel: before anything else the CTA asks for its whole share (up
    // to a cap) to be moved from HBM into L2, a few instructions in total, so that HBM streams at full rate
    // while the preceding kernel drains and the activations are prepared; the ring then fills from L2.
    pdl_launch_dependents();
    prefetch_target_slice(p.prefetch, blockIdx.x, gridDim.x, tid, blockDim.x);  // a later launch's weights
    {
        const int pu0 = p.cta_mode ? u_first : u_lo;
        const int pu1 = p.cta_mode ? min(u_first + kWarps, units) : u_hi;
        if (pu0 < pu1) {
            int pa0, pa1, unused;
            unit_range(pu0, pa0, unused);
            unit_range(pu1 - 1, unused, pa1);
            pa1 = min(pa1, pa0 + p.bulk_stages);
            const int piece = gtid >> 1;  // even threads: tiles, odd threads: scale/zero pairs
            const int s0 = pa0 + piece * kBulkPiece;
            if (s0 < pa1) {
                const int ns = min(kBulkPiece, pa1 - s0);
                if (gtid & 1) prefetch_l2_bulk(p.sb + (size_t)s0 * 16, (unsigned)ns * 256u);
                else prefetch_l2_bulk(p.tiles + (size_t)s0 * 128, (unsigned)ns * 2048u);
            }
        }
    }
    int islot = 0, cslot = 0;  // ring slots of the next stage to issue / to consume
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i)
        if (i < p.pre_stages) { issue(islot); islot = islot + 1 == kStages ? 0 : islot + 1; }
    // the norm weights are constants of the model (and come from HBM): requested before the wait for the predecessor
    uint4 nw_early = make_uint4(0, 0, 0, 0);
    if (p.norm_mode && tid * 8 < p.k) nw_early = __ldg(reinterpret_cast<const uint4*>(p.norm_w + tid * 8));
    pdl_wait();
    if (p.trace && tid == 0) p.trace[blockIdx.x * 4 + 1] = global_timer_ns();
    // The activations of this thread's runs are requested now, all of them together (one trip to L2, not one per
    // run) and ahead of the remaining ring stages: a load issued after those would wait in the SM's memory pipeline
    // behind tens of kilobytes of weights, and the whole product waits for the activations.
    NormRunLoads pre_loads;
    pre_loads.x = pre_loads.res = pre_loads.nw = make_uint4(0, 0, 0, 0);
    uint4 x_more[2];
    x_more[0] = x_more[1] = make_uint4(0, 0, 0, 0);
    if (p.norm_mode) { pre_loads = fused_norm_load8(p, tid * 8, tid * 8 < p.k); pre_loads.nw = nw_early; }
    else {
        if (tid * 8 < p.k) pre_loads.x = __ldcg(reinterpret_cast<const uint4*>(p.x + tid * 8));
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int k0 = (tid + (i + 1) * (int)blockDim.x) * 8;
            if (k0 < p.k) x_more[i] = __ldcg(reinterpret_cast<const uint4*>(p.x + k0));
        }
    }
    // ring_late of the remaining stages are held back until the activations are in shared memory
    int held = 0;
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i)
        if (i >= p.pre_stages) {
            if (kStages - 1 - i <= p.ring_late) { ++held; continue; }
            issue(islot); islot = islot + 1 == kStages ? 0 : islot + 1;
        }

    // ---- activations -> block floating point, one run of 16 elements per thread ------------------------
    __shared__ float red[kMaxWarps1];
    __shared__ __align__(16) unsigned zero16[4];   // B operand of the lanes that carry no activations
    if (tid < 4) zero16[tid] = 0u;                 // visible after the barrier that ends this section
    const int tp_epoch = (p.push || p.in_tp) ? *p.tp.epoch + (p.push ? 1 : 0) : 0;
    const int nthreads = blockDim.x;
    const int nruns = kt_total * 8;  // runs of 8 elements: eight neighbouring threads share a group of 64
    const bool stamp0 = p.trace && blockIdx.x == 0 && tid == 0 && gridDim.x + 2 <= kTraceRows;  // finer stamps of the first CTA
    if (stamp0) p.trace[(gridDim.x + 1) * 4] = global_timer_ns();   // loads and ring stages issued
    for (int run = tid; run < nruns || (p.norm_mode && run < nthreads); run += nthreads) {
        const int k0 = run * 8;
        float xf[8];
        if (p.norm_mode) {
            // dimension <= 4096: exactly one pass, every thread takes part in the block-wide sum
            fused_norm_run8(p, k0, k0 < p.k, blockIdx.x == 0, red, xf, tp_epoch, nthreads >> 5, pre_loads);
            if (stamp0) p.trace[(gridDim.x + 1) * 4 + 1] = global_timer_ns();   // inputs arrived, norm formed
            if (run >= nruns) continue;
        } else {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (run == tid) v = pre_loads.x;
            else if (run == tid + nthreads) v = x_more[0];
            else if (run == tid + 2 * nthreads) v = x_more[1];
            else if (k0 < p.k) v = __ldcg(reinterpret_cast<const uint4*>(p.x + k0));
            const unsigned vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) { xf[2 * i] = __uint_as_float(vw[i] << 16); xf[2 * i + 1] = __uint_as_float(vw[i] & 0xFFFF0000u); }
        }
        // one exponent per group of 64
        const unsigned act = __activemask();
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(xf[i]));
        amax = fmaxf(amax, __shfl_xor_sync(act, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(act, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(act, amax, 4));
        const int e = (int)(__float_as_uint(amax) >> 23);  // biased exponent of the group's largest magnitude
        const bool live = e >= 16 && e < 255;               // not all-zero / denormal, not inf / nan
        // largest magnitude -> [2^13, 2^14): multiply by 2^(140 - e). Adding 1.5 * 2^23 leaves the rounded
        // (nearest-even) integer in the low mantissa bits in two's complement: its low byte is the low digit
        // as a signed byte, and (v + 128) >> 8 is the high digit, v = 256 * hi + lo.
        const float mul = __uint_as_float((unsigned)(267 - e) << 23);
        unsigned rb[8], rh[8];
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            rb[i] = live ? __float_as_uint(fmaf(xf[i], mul, 12582912.0f)) : 0x4B400000u;
            rh[i] = rb[i] + 128u;
            sum += (int)(rb[i] - 0x4B400000u);
        }
        sum += __shfl_xor_sync(act, sum, 1);
        sum += __shfl_xor_sync(act, sum, 2);
        sum += __shfl_xor_sync(act, sum, 4);
        // byte order inside a 4-element step matches the nibble order of a weight word: 0, 2, 1, 3
        uint2 hi, lo;
        lo.x = __byte_perm(__byte_perm(rb[0], rb[2], 0x0040), __byte_perm(rb[1], rb[3], 0x0040), 0x5410);
        lo.y = __byte_perm(__byte_perm(rb[4], rb[6], 0x0040), __byte_perm(rb[5], rb[7], 0x0040), 0x5410);
        hi.x = __byte_perm(__byte_perm(rh[0], rh[2], 0x0051), __byte_perm(rh[1], rh[3], 0x0051), 0x5410);
        hi.y = __byte_perm(__byte_perm(rh[4], rh[6], 0x0051), __byte_perm(rh[5], rh[7], 0x0051), 0x5410);
        // a quarter of a group (16 elements) is 16 high-digit bytes followed by 16 low-digit bytes
        unsigned char* qd = reinterpret_cast<unsigned char*>(xq) + (size_t)(run >> 1) * 32 + (run & 1) * 8;
        *reinterpret_cast<uint2*>(qd) = hi;
        *reinterpret_cast<uint2*>(qd + 16) = lo;
        const float scale = live ? __uint_as_float((unsigned)(e - 13) << 23) : 0.f;  // 2^(e - 140) = 1 / mul
        if ((run & 7) == 0) xmeta[run >> 3] = make_float2(scale, (float)sum * scale);
        if (stamp0 && run == tid) p.trace[(gridDim.x + 1) * 4 + 2] = global_timer_ns();   // this thread's first run quantised
    }
    if (stamp0) p.trace[(gridDim.x + 1) * 4 + 3] = global_timer_ns();   // all of this thread's runs
    for (; held > 0; --held) { issue(islot); islot = islot + 1 == kStages ? 0 : islot + 1; }
    __syncthreads();

    if (p.trace && tid == 0) p.trace[blockIdx.x * 4 + 2] = global_timer_ns();
    const int s_total = 1 << p.si_shift;
    __shared__ float cta_red_all[kMaxGroups][2][kWarps][16];
    float (*cta_red)[kWarps][16] = cta_red_all[grp];
    // B operand source. The four k-tiles of a stage (four groups of 64) share one set of accumulators: tile ti
    // carries its activations in columns 2 ti (high digits) and 2 ti + 1 (low digits) of the B operand and zeros
    // elsewhere, so after the stage's eight instructions lane (g, t) holds the integer sums of group t for rows g and
    // g + 8, and the scale / zero epilogue runs once per stage with all 32 lanes busy (one group each) instead of
    // once per tile with eight. Lane (g, t) therefore supplies data for tile g >> 1 only and reads zeros for the
    // other three. All shared-memory addresses below are 32-bit.
    const unsigned xq_sa = (unsigned)__cvta_generic_to_shared(xq);
    const unsigned xmeta_sa = (unsigned)__cvta_generic_to_shared(xmeta) + t * 8;
    const unsigned zero_sa = (unsigned)__cvta_generic_to_shared(zero16);
    const int my_ti = g >> 1;
    const unsigned my_xoff = xq_sa + my_ti * 128 + t * 32 + (g & 1) * 16;
    const unsigned ring_warp_sa = (unsigned)__cvta_generic_to_shared(my_ring);
    int round = 0;
    for (int base = u_first; base < u_limit; base += u_stride, ++round) {
        const int u = base + warp;
        const bool valid = u < u_end;
        const int rt = u >> p.si_shift;
        const int slice = u & si_mask;
        const int n_slices = s_total, pstride = s_total;
        float tot_lo = 0.f, tot_hi = 0.f, tot_hi16 = 0.f, tot_hiz = 0.f;
        int a0 = 0, a1 = 0;
        if (valid) unit_range(u, a0, a1);
        int stg = a0 - rt * p.kt4_total;
        for (int a = a0; a < a1; ++a, ++stg) {
            issue(islot); islot = islot + 1 == kStages ? 0 : islot + 1;
            cp_async_wait<kStages - 1>();
            __syncwarp();
            const unsigned st = ring_warp_sa + cslot * kStageBytes;
            cslot = cslot + 1 == kStages ? 0 : cslot + 1;
            const unsigned wsa = st + lane * 16;
            const unsigned xmine = my_xoff + stg * 512;
            int c[4];
#pragma unroll
            for (int ti = 0; ti < 4; ++ti) {
                const uint4 wv = lds128(wsa + ti * 512);
                const uint4 xd = lds128(ti == my_ti ? xmine : zero_sa);
                // A byte holds the nibble of row g (low) and of row g + 8 (high) for the same column. Rows g take
                // the masked low nibbles; rows g + 8 take the bytes as they are, lo + 16 * hi, against the same
                // activations: their sum is (row g's sum) + 16 * (row g + 8's sum), all exact integers, so the
                // high rows cost no unpacking at all and are recovered by one subtraction
                if (ti == 0) imma_u8s8_zero(c, wv.x & 0x0F0F0F0Fu, wv.x, wv.y & 0x0F0F0F0Fu, wv.y, xd.x, xd.y);
                else imma_u8s8(c, wv.x & 0x0F0F0F0Fu, wv.x, wv.y & 0x0F0F0F0Fu, wv.y, xd.x, xd.y);
                imma_u8s8(c, wv.z & 0x0F0F0F0Fu, wv.z, wv.w & 0x0F0F0F0Fu, wv.w, xd.z, xd.w);
            }
            // group t of the stage: (scale, zero) of rows g and g + 8, the group's 2^E and scaled activation sum
            const unsigned pa = lds32(st + 2048 + lane * 4), pb = lds32(st + 2048 + 128 + lane * 4);
            const float2 mt = lds64f(xmeta_sa + stg * 32);
            const float fa = (float)(c[0] * 256 + c[1]);                         // sum = 256 * hi + lo
            const float fb16 = (float)((c[2] - c[0]) * 256 + (c[3] - c[1]));     // 16 x the sum of row g + 8
            tot_lo = fmaf(sb_scale<F16SB>(pa) * mt.x, fa, fmaf(sb_zero<F16SB>(pa), mt.y, tot_lo));
            tot_hi16 = fmaf(sb_scale<F16SB>(pb) * mt.x, fb16, tot_hi16);
            tot_hiz = fmaf(sb_zero<F16SB>(pb), mt.y, tot_hiz);
            __syncwarp();
        }
        tot_hi = fmaf(tot_hi16, 0.0625f, tot_hiz);
        // lane (g, t) holds the part of groups t, t + 4, ... of rows g and g + 8: add the four lanes of a row
        tot_lo += __shfl_xor_sync(0xffffffffu, tot_lo, 1); tot_lo += __shfl_xor_sync(0xffffffffu, tot_lo, 2);
        tot_hi += __shfl_xor_sync(0xffffffffu, tot_hi, 1); tot_hi += __shfl_xor_sync(0xffffffffu, tot_hi, 2);

        bool finisher = valid;
        if (p.cta_mode) {
            if (s_total > 1) {
                // slices of a row tile sit in neighbouring warps: add them in slice order through shared memory
                if (valid && t == 0) { cta_red[round & 1][warp][g] = tot_lo; cta_red[round & 1][warp][g + 8] = tot_hi; }
                asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "n"(kThreads) : "memory");  // the group's own barrier
                finisher = valid && slice == 0;
                if (finisher) {
                    tot_lo = tot_hi = 0.f;
                    for (int s = 0; s < s_total; ++s) {
                        tot_lo += cta_red[round & 1][warp + s][g];
                        tot_hi += cta_red[round & 1][warp + s][g + 8];
                    }
                }
            }
        } else if (n_slices > 1 && valid) {
            float* dst = p.partial + ((size_t)rt * pstride + slice) * 16;
            if (t == 0) { __stcg(dst + g, tot_lo); __stcg(dst + g + 8, tot_hi); }
            __threadfence();
            __syncwarp();
            unsigned prev = 0;
            if (lane == 0) prev = atomicAdd(p.counters + rt, 1u);
            prev = __shfl_sync(0xffffffffu, prev, 0);
            finisher = prev == (unsigned)n_slices - 1u;
            if (finisher) {
                __threadfence();
                if (lane == 0) p.counters[rt] = 0u;
                tot_lo = tot_hi = 0.f;
                for (int s = 0; s < n_slices; ++s) {  // slice order: independent of arrival order
                    const float* src = p.partial + ((size_t)rt * pstride + s) * 16;
                    tot_lo += __ldcg(src + g);
                    tot_hi += __ldcg(src + g + 8);
                }
            }
        }
        if (!finisher) continue;
        if (EPI == QGEMV_EPI_STORE && p.push) {
            if (t == 0) {
                if (rt * 16 + g < p.seg_end[0]) tp_push_value(p, tp_epoch, rt * 16 + g, 0, tot_lo);
                if (rt * 16 + g + 8 < p.seg_end[0]) tp_push_value(p, tp_epoch, rt * 16 + g + 8, 0, tot_hi);
            }
            tp_row_tile_done(p, tp_epoch, lane);
            continue;
        }
        if (t != 0) continue;
        if (EPI == QGEMV_EPI_STORE) {
#pragma unroll
            for (int hi = 0; hi < 2; ++hi) {
                const int r = rt * 16 + g + 8 * hi;
                const __nv_bfloat16 val = __float2bfloat16_rn(hi ? tot_hi : tot_lo);
                if (r < p.seg_end[0]) p.y[0][r] = val;
                else if (r < p.seg_end[1]) p.y[1][r - p.seg_end[0]] = val;
                else if (r < p.seg_end[2]) p.y[2][r - p.seg_end[1]] = val;
            }
        } else {
            // gate rows 0-7, matching up rows 8-15; both rounded to bf16 first, as the reference stores them
            // to bf16 scratch before `swiglu` reads them (Primitives/ElementwiseFragment.swift:49-54)
            const int r = rt * 8 + g;
            if (r < p.seg_end[0]) {
                const float gate = __bfloat162float(__float2bfloat16_rn(tot_lo));
                const float up = __bfloat162float(__float2bfloat16_rn(tot_hi));
                p.y[0][r] = __float2bfloat16_rn(gated_activation(gate, up, p.gated_act));
            }
        }
    }
    cp_async_wait<0>();
    if (p.trace) {
        __syncthreads();
        if (tid == 0) p.trace[blockIdx.x * 4 + 3] = global_timer_ns();
    }
}

template <int EPI, bool F16SB>
__global__ void __launch_bounds__(kMaxGroups * kThreads, 1) qgemv1_kernel(const QGemvParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    qgemv1_body<EPI, F16SB>(p, smem);
}

struct QGemvConfig {
    int nt, si, sk, occ, cta_mode;
    dim3 grid;
    size_t smem;
};

constexpr int kSMs = 148;

size_t x_smem_bytes(int rows_x, int cols, int kt4, int sk) {
    const int nk = 256 * ((kt4 + sk - 1) / sk);
    return (size_t)rows_x * (nk + kXPad) * 2 + (size_t)(nk / 64) * cols * 4;
}

// Persistent grid: at most occ CTAs per SM, all resident at once; work is cut into (row tile, k-slice)
// units small enough that every SM streams the same number of bytes to within a few percent.
// one_k_group: the launch carries a fused norm, whose block-wide sum needs the whole activation row in one CTA group
QGemvConfig pick_config(const Q4Tiled& w, int m, bool one_k_group = false) {
    QGemvConfig c{};
    if (m == 1) {
        // integer dot-product kernel: the whole activation vector in block floating point (2 bytes + 1/8 byte
        // of metadata per element), one CTA group
        const int kt4 = w.kt_pad / 4;
        c.nt = 0; c.sk = 1;
        // one CTA per SM made of up to three eight-warp groups (c.occ = groups) that share the activations
        c.occ = kMaxGroups;
        const size_t x_bytes = (size_t)w.kt_pad * 160, budget = 214 * 1024;  // below every kernel's limit (opt-in maximum minus its static shared memory)
        while (c.occ > 1 && (size_t)c.occ * kRingBytes + x_bytes > budget) --c.occ;
        c.smem = (size_t)c.occ * kRingBytes + x_bytes;
        const int slots = kSMs * c.occ;  // groups resident on the GPU
        int vgrid;
        if (kt4 >= 2) {
            // One row tile per group and round, its eight warps split K and add their parts through shared memory (no
            // global scratch, no atomics); group v takes row tiles v, v + groups, ...: in every round the GPU reads one
            // contiguous window of the matrix, which is what HBM likes (measured on the 28672 x 4096 gate/up product:
            // 16.8 us when every warp streamed a private contiguous range of the matrix, 14.3 us this way; the
            // 128256 x 4096 output head 60 -> 50 us).
            c.cta_mode = 1;
            c.si = 1;
            while (c.si < kWarps && c.si * 2 <= kt4) c.si *= 2;
            const int chunks = (w.row_tiles * c.si + kWarps - 1) / kWarps;
            vgrid = std::min(slots, chunks);
        } else {
            c.si = 1;
            const int units = w.row_tiles * c.si;
            vgrid = std::min(slots, (units + kWarps - 1) / kWarps);
        }
        // groups are numbered group-major (group * CTAs + CTA): work spreads over the SMs before it stacks up
        c.grid = dim3((unsigned)std::min(kSMs, vgrid), 1, 1);
        return c;
    }
    c.nt = m <= 8 ? 1 : 2;
    const int cols = 8 * c.nt;
    const int rows_x = std::min(m, cols);
    const int kt4 = w.kt_pad / 4;
    const int max_occ = c.nt == 1 ? 3 : 2;
    const size_t sm_budget = 227 * 1024;
    // highest occupancy whose shared-memory share holds the ring plus this group's slice of x;
    // a second (or further) CTA group along K only when x does not fit otherwise
    c.occ = 1; c.sk = kt4;
    bool found = false;
    // Prefer the highest occupancy (more warps streaming per SM hide more latency) and split K across up to eight CTA
    // groups to make the activations fit, rather than the fewest K-splits: 36.4 -> 27.7 us for 14336 x 4096 at 16
    // sequences, 43.4 -> 32.3 us for 4096 x 14336. SWLM_BATCH_OCC_FIRST=0 restores the old preference.
    static const bool occ_first = [] { const char* v = getenv("SWLM_BATCH_OCC_FIRST"); return !(v && v[0] == '0'); }();
    if (occ_first) {
        for (int occ = max_occ; occ >= 1 && !found; --occ)
            for (int sk = 1; sk <= kt4 && sk <= (one_k_group ? 1 : 8) && !found; sk *= 2) {
                const size_t per_cta = sm_budget / occ - 1024;
                if ((size_t)kRingBytes + x_smem_bytes(rows_x, cols, kt4, sk) <= per_cta) { c.occ = occ; c.sk = sk; found = true; }
            }
    }
    for (int sk = 1; sk <= kt4 && !found; sk *= 2)
        for (int occ = max_occ; occ >= 1 && !found; --occ) {
            const size_t per_cta = sm_budget / occ - 1024;
            if ((size_t)kRingBytes + x_smem_bytes(rows_x, cols, kt4, sk) <= per_cta) { c.occ = occ; c.sk = sk; found = true; }
        }
    c.sk = std::min(c.sk, kt4);
    const int glen = std::max(1, kt4 / c.sk);
    // k-slices per group: aim at >= 16 units per SM, never shorter than two stages (4.6 KB)
    c.si = 1;
    while (c.si < 16 && c.si * 4 <= glen && (long long)w.row_tiles * c.si * c.sk < 16LL * kSMs) c.si *= 2;
    const int units = w.row_tiles * c.si;
    int gx = std::max(1, (kSMs * c.occ) / c.sk);
    gx = std::min(gx, (units + kWarps - 1) / kWarps);
    c.grid = dim3((unsigned)gx, (unsigned)c.sk, 1);
    c.smem = (size_t)kRingBytes + x_smem_bytes(rows_x, cols, kt4, c.sk);
    return c;
}

// ---- phase tracing of the batch-1 kernel (diagnostic, SWLM_TRACE=1) ---------------------------------------
// The first kTraceSlots launches get a slot each; a CUDA graph keeps the slots it was captured with, so after
// replays the buffer holds the timeline of the last replayed decode step. The report goes to stderr when a context is
// destroyed.
constexpr int kTraceSlots = 256, kTraceCtas = 512;
unsigned long long* g_trace_buf = nullptr;
int g_trace_next = 0;
struct TraceSlot { int ctas, row_tiles, kt4, epi, norm; };
TraceSlot g_trace_slot[kTraceSlots];

template <int EPI>
int launch_1(const QGemvParams& p_in, const QGemvConfig& c, cudaStream_t s) {
    QGemvParams p = p_in;
    p.trace = qgemv_trace_slot((int)c.grid.x, p.row_tiles, p.kt4_total, EPI, p.norm_mode);
    cudaError_t e;
    e = p.sb_f16 ? launch_k(qgemv1_kernel<EPI, true>, c.grid, dim3(c.occ * kThreads), c.smem, s, p)
                 : launch_k(qgemv1_kernel<EPI, false>, c.grid, dim3(c.occ * kThreads), c.smem, s, p);
    if (e != cudaSuccess) return cuda_fail(e, "qgemv1 launch");
    return SWLM_OK;
}

template <int NT, int EPI>
int launch_t(const QGemvParams& p, const QGemvConfig& c, cudaStream_t s) {
    cudaError_t e = p.sb_f16 ? launch_k(qgemv_kernel<NT, EPI, true>, c.grid, dim3(kThreads), c.smem, s, p)
                             : launch_k(qgemv_kernel<NT, EPI, false>, c.grid, dim3(kThreads), c.smem, s, p);
    if (e != cudaSuccess) return cuda_fail(e, "qgemv launch");
    return SWLM_OK;
}

}  // namespace

static int g_max_dyn_smem = 0;

template <typename K>
static int opt_in_smem(K kernel) {
    int dev = 0, optin = 0;
    SWLM_CUDA(cudaGetDevice(&dev));
    SWLM_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cudaFuncAttributes fa;
    SWLM_CUDA(cudaFuncGetAttributes(&fa, kernel));
    const int dyn = optin - (int)fa.sharedSizeBytes;  // static shared memory counts against the same limit
    SWLM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    if (g_max_dyn_smem == 0 || dyn < g_max_dyn_smem) g_max_dyn_smem = dyn;
    return SWLM_OK;
}

unsigned long long* qgemv_trace_slot(int ctas, int row_tiles, int kt4, int epi, int norm) {
    if (!g_trace_buf || ctas > kTraceCtas || g_trace_next >= kTraceSlots) return nullptr;
    const int slot = g_trace_next++;
    g_trace_slot[slot] = {ctas, row_tiles, kt4, epi, norm};
    return g_trace_buf + (size_t)slot * kTraceCtas * 4;
}

void qgemv_trace_report() {
    if (!g_trace_buf) return;
    cudaDeviceSynchronize();
    std::vector<unsigned long long> h((size_t)kTraceSlots * kTraceCtas * 4);
    if (cudaMemcpy(h.data(), g_trace_buf, h.size() * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return;
    const int used = std::min(g_trace_next, kTraceSlots);
    unsigned long long origin = 0;
    fprintf(stderr, "times in us from the first traced kernel's first CTA entry; dur = means over CTAs\n");
    fprintf(stderr, "slot ctas rowtiles kt4 epi norm | first-entry first-deps last-deps last-xready first-done last-done | dur: wait prologue stream\n");
    for (int sl = 0; sl < used; ++sl) {
        const TraceSlot& t = g_trace_slot[sl];
        const unsigned long long* r = h.data() + (size_t)sl * kTraceCtas * 4;
        unsigned long long e0 = ~0ull, d0 = ~0ull, d1 = 0, x1 = 0, f0 = ~0ull, f1 = 0;
        double a = 0, b = 0, c = 0;
        int n = 0;
        for (int i = 0; i < t.ctas; ++i) {
            if (!r[i * 4] || !r[i * 4 + 3]) continue;
            e0 = std::min(e0, r[i * 4]);
            d0 = std::min(d0, r[i * 4 + 1]); d1 = std::max(d1, r[i * 4 + 1]);
            x1 = std::max(x1, r[i * 4 + 2]);
            f0 = std::min(f0, r[i * 4 + 3]); f1 = std::max(f1, r[i * 4 + 3]);
            a += (double)(r[i * 4 + 1] - r[i * 4]); b += (double)(r[i * 4 + 2] - r[i * 4 + 1]); c += (double)(r[i * 4 + 3] - r[i * 4 + 2]);
            ++n;
        }
        if (!n) continue;
        if (!origin || e0 < origin) origin = e0;
        if (t.epi == 9) {
            // attention: [1] predecessor complete, [2] main loop done, [3] partials published; merged stamps follow
            auto rel9 = [&](unsigned long long v) { return ((double)v - (double)origin) / 1e3; };
            unsigned long long m0 = ~0ull, m1 = 0;
            const int nm = -t.row_tiles;
            for (int i = 0; i < nm; ++i) { const unsigned long long v = r[(t.ctas + i) * 4]; if (v) { m0 = std::min(m0, v); m1 = std::max(m1, v); } }
            fprintf(stderr, "%3d attention %d CTAs | first-entry %9.2f deps %9.2f..%9.2f loop-done(last) %9.2f published %9.2f..%9.2f merged %9.2f..%9.2f | dur: wait %.2f prologue+loop %.2f publish %.2f\n",
                    sl, t.ctas, rel9(e0), rel9(d0), rel9(d1), rel9(x1), rel9(f0), rel9(f1), rel9(m0), rel9(m1), a / n / 1e3, b / n / 1e3, c / n / 1e3);
            if (r[t.ctas * 4 + 1])  // finer stamps of CTA 0, relative to the completion of its predecessor
                fprintf(stderr, "    CTA 0 after deps (us): q/k/v in shared memory %.2f, rotated %.2f, self score %.2f, q fragments %.2f, first 64 tokens %.2f, loop done %.2f, published %.2f\n",
                        ((double)r[t.ctas * 4 + 1] - (double)r[1]) / 1e3, ((double)r[(t.ctas + 1) * 4 + 1] - (double)r[1]) / 1e3,
                        ((double)r[(t.ctas + 1) * 4 + 2] - (double)r[1]) / 1e3, ((double)r[t.ctas * 4 + 2] - (double)r[1]) / 1e3,
                        ((double)r[t.ctas * 4 + 3] - (double)r[1]) / 1e3, ((double)r[2] - (double)r[1]) / 1e3, ((double)r[3] - (double)r[1]) / 1e3);
            continue;
        }
        auto rel = [&](unsigned long long v) { return ((double)v - (double)origin) / 1e3; };
        fprintf(stderr, "%3d %4d %6d %4d %d %d | %9.2f %9.2f %9.2f %9.2f %9.2f %9.2f | %6.2f %6.2f %6.2f", sl, t.ctas, t.row_tiles, t.kt4, t.epi,
                t.norm, rel(e0), rel(d0), rel(d1), rel(x1), rel(f0), rel(f1), a / n / 1e3, b / n / 1e3, c / n / 1e3);
        if (t.ctas + 2 <= kTraceCtas && !r[t.ctas * 4] && r[(t.ctas + 1) * 4 + 3]) {
            // finer stamps of CTA 0, relative to the completion of its predecessor
            auto d0 = [&](unsigned long long v) { return v ? ((double)v - (double)r[1]) / 1e3 : 0.0; };
            fprintf(stderr, " | CTA 0 after deps (us): requests issued %.2f, norm formed %.2f, first run quantised %.2f, all runs %.2f, x ready %.2f, done %.2f",
                    d0(r[(t.ctas + 1) * 4]), d0(r[(t.ctas + 1) * 4 + 1]), d0(r[(t.ctas + 1) * 4 + 2]), d0(r[(t.ctas + 1) * 4 + 3]), d0(r[2]), d0(r[3]));
        }
        // the tensor-core kernel also stamps the end of its set-up and the release of its TMEM, in the rows after
        // its CTAs'
        if (2 * t.ctas <= kTraceCtas && r[t.ctas * 4]) {
            unsigned long long s1 = 0, r1 = 0;
            double dd = 0, tw = 0, tl = 0, gap = 0, gapmax = 0, setup = 0;
            for (int i = 0; i < t.ctas; ++i) {
                const unsigned long long* q = r + (size_t)(t.ctas + i) * 4;
                s1 = std::max(s1, q[0]); r1 = std::max(r1, q[1]);
                dd += (double)(q[1] - q[2]); tw += (double)(q[3] >> 32); tl += (double)(q[3] & 0xFFFFFFFFull);
                gap += (double)q[2] - (double)r[i * 4 + 3]; gapmax = std::max(gapmax, (double)q[2] - (double)r[i * 4 + 3]);
                setup += (double)q[0] - (double)r[i * 4];
            }
            if (3 * t.ctas <= kTraceCtas) {
                double m0 = 0, m1 = 0, m2 = 0, m3 = 0;
                for (int i = 0; i < t.ctas; ++i) {
                    const unsigned long long* q2 = r + (size_t)(2 * t.ctas + i) * 4;
                    const double done = (double)r[i * 4 + 3];
                    m0 += (double)q2[0] - done; m1 += (double)q2[1] - done; m2 += (double)q2[2] - done; m3 += (double)q2[3] - done;
                }
                fprintf(stderr, " | rel. to done (us): mma loop exit %.2f, warp1 after last barrier %.2f, epilogue exit %.2f, mask exit %.2f",
                        m0 / t.ctas / 1e3, m1 / t.ctas / 1e3, m2 / t.ctas / 1e3, m3 / t.ctas / 1e3);
            }
            fprintf(stderr, " | set-up mean %.2f us, last done %9.2f; done -> release mean %.2f max %.2f us, release %.2f us; epilogue clocks per CTA: waiting for MMAs %.0f, reading TMEM %.0f",
                    setup / t.ctas / 1e3, rel(s1), gap / t.ctas / 1e3, gapmax / 1e3, dd / t.ctas / 1e3, tw / t.ctas, tl / t.ctas);
        }
        fprintf(stderr, "\n");
    }
}

int qgemv_init() {
    int rc;
    const char* tr = getenv("SWLM_TRACE");
    if (tr && tr[0] == '1' && !g_trace_buf) {
        SWLM_CUDA(cudaMalloc((void**)&g_trace_buf, (size_t)kTraceSlots * kTraceCtas * 4 * 8));
        SWLM_CUDA(cudaMemset(g_trace_buf, 0, (size_t)kTraceSlots * kTraceCtas * 4 * 8));
    }
    if ((rc = opt_in_smem(qgemv_kernel<1, 0, false>))) return rc;
    if ((rc = opt_in_smem(qgemv_kernel<1, 1, false>))) return rc;
    if ((rc = opt_in_smem(qgemv_kernel<2, 0, false>))) return rc;
    if ((rc = opt_in_smem(qgemv_kernel<2, 1, false>))) return rc;
    if ((rc = opt_in_smem(qgemv_kernel<1, 0, true>))) return rc;
    if ((rc = opt_in_smem(qgemv_kernel<1, 1, true>))) return rc;
    if ((rc = opt_in_smem(qgemv_kernel<2, 0, true>))) return rc;
    if ((rc = opt_in_smem(qgemv_kernel<2, 1, true>))) return rc;
    if ((rc = opt_in_smem(qgemv1_kernel<0, false>))) return rc;
    if ((rc = opt_in_smem(qgemv1_kernel<1, false>))) return rc;
    if ((rc = opt_in_smem(qgemv1_kernel<0, true>))) return rc;
    if ((rc = opt_in_smem(qgemv1_kernel<1, true>))) return rc;
    return SWLM_OK;
}

size_t qgemv_scratch_floats(const Q4Tiled& w, int m) {
    size_t need = 0;
    for (int one = 0; one < 2; ++one) {   // with and without a fused norm (different K splits)
        QGemvConfig c = pick_config(w, m, one != 0);
        if (c.sk * c.si <= 1 || c.cta_mode) continue;
        need = std::max(need, (size_t)w.row_tiles * c.sk * c.si * 16 * (c.nt ? 8 * c.nt : 1));
    }
    return need;
}
int qgemv_counter_count(const Q4Tiled& w) { return w.row_tiles; }

static int build_params(const QGemvLaunch& a, QGemvParams& p, QGemvConfig& c);

int launch_qgemv(const QGemvLaunch& a, cudaStream_t s) {
    QGemvParams p{};
    QGemvConfig c{};
    int rc = build_params(a, p, c);
    if (rc) return rc;
    if (c.nt == 0) return a.epilogue == QGEMV_EPI_SWIGLU ? launch_1<1>(p, c, s) : launch_1<0>(p, c, s);
    if (a.epilogue == QGEMV_EPI_SWIGLU) return c.nt == 1 ? launch_t<1, 1>(p, c, s) : launch_t<2, 1>(p, c, s);
    return c.nt == 1 ? launch_t<1, 0>(p, c, s) : launch_t<2, 0>(p, c, s);
}

static int build_params(const QGemvLaunch& a, QGemvParams& p, QGemvConfig& c) {
    const Q4Tiled& w = *a.w;
    if (a.m < 1 || a.m > 16) { set_error("qgemv: m=%d outside 1..16", a.m); return SWLM_ERR_INVALID; }
    if ((a.x_stride & 7) || (reinterpret_cast<uintptr_t>(a.x) & 15)) {
        set_error("qgemv: x must be 16-byte aligned with a stride that is a multiple of 8 elements");
        return SWLM_ERR_INVALID;
    }
    c = pick_config(w, a.m, a.norm.mode != 0);
    if (g_max_dyn_smem == 0 || c.smem > (size_t)g_max_dyn_smem) { set_error("qgemv: shared memory %zu exceeds the limit %d", c.smem, g_max_dyn_smem); return SWLM_ERR_INVALID; }
    if (c.sk * c.si > 1 && !c.cta_mode && (!a.partial || !a.counters)) { set_error("qgemv: split launch without scratch"); return SWLM_ERR_INVALID; }
    p = QGemvParams{};
    p.tiles = w.tiles; p.sb = w.sb; p.row_tiles = w.row_tiles; p.kt4_total = w.kt_pad / 4; p.sb_f16 = w.sb_f16 ? 1 : 0;
    p.x = a.x; p.x_stride = a.x_stride; p.k = w.k;
    for (int i = 0; i < 3; ++i) {
        p.y[i] = a.y[i]; p.y_stride[i] = a.y_stride[i];
        p.seg_end[i] = a.seg_end[i] > 0 ? a.seg_end[i] : (i ? p.seg_end[i - 1] : 0);
    }
    p.m = a.m;
    p.gated_act = a.gated_act;
    p.si = c.si; p.sk = c.sk; p.cta_mode = c.cta_mode;
    {
        // Ring stages requested before the wait for the preceding kernel, and stages asked into L2 up front. Both
        // put weight traffic ahead of the activation loads in the SM's memory pipeline, and the product cannot
        // start before its activations: measured best on the Llama-3-8B shape is no stage before the wait
        // (563 / 570 / 575 tok/s for 2 / 1 / 0) and 8 stages into L2.
        static const int pre = [] { const char* v = getenv("SWLM_PRE_STAGES"); return v ? atoi(v) : 0; }();
        p.pre_stages = pre < 0 ? 0 : pre;
        static const int bulk = [] { const char* v = getenv("SWLM_BULK_STAGES"); return v ? atoi(v) : kBulkMaxStages; }();
        p.bulk_stages = bulk;
        // measured on the Llama-3-8B shape: 630 / 634 / 616 tok/s for 0 / 1 / 2 stages held back
        static const int late = [] { const char* v = getenv("SWLM_RING_LATE"); return v ? atoi(v) : 1; }();
        p.ring_late = late;
    }
    p.si_shift = 0;
    while ((1 << p.si_shift) < c.si) ++p.si_shift; p.partial = a.partial; p.counters = a.counters;
    {
        const unsigned long long vgrid = (unsigned long long)c.grid.x * (unsigned long long)std::max(1, c.occ);
        const unsigned long long stages = (unsigned long long)p.row_tiles * (unsigned long long)p.kt4_total;
        const unsigned long long units = (unsigned long long)p.row_tiles << p.si_shift;
        p.idx32 = (stages + 1) * (vgrid * kWarps + 1) < (1ull << 32) && (units + 1) * (vgrid + 1) < (1ull << 32);
    }
    p.push = a.push; p.in_tp = a.in_tp; p.tp = a.tp;
    p.prefetch = a.prefetch;
    if ((a.push || a.in_tp) && (a.tp.tp < 2 || !a.tp.epoch || !a.tp.done || !a.tp.status)) { set_error("qgemv: tensor-parallel exchange not attached"); return SWLM_ERR_STATE; }
    if (a.in_tp && !a.norm.mode) { set_error("qgemv: a pushed partial sum must be consumed by a fused norm"); return SWLM_ERR_INVALID; }
    p.norm_mode = a.norm.mode;
    if (a.norm.mode) {
        if (w.k > 4096 || (w.k & 15) || c.sk != 1 || !a.norm.weight || a.norm.res_in == a.norm.res_out) {
            set_error("qgemv: fused norm needs k <= 4096, k %% 16 == 0 and distinct residual buffers");
            return SWLM_ERR_INVALID;
        }
        p.res_in = a.norm.res_in; p.res_out = a.norm.res_out; p.res_stride = a.norm.res_stride;
        p.norm_w = a.norm.weight; p.eps = a.norm.eps; p.weight_bias = a.norm.weight_bias;
    }
    return SWLM_OK;
}

// =================================================================================================
// Re-tiling: MLX source layout -> streaming layout, on the device.
// =================================================================================================
namespace {

struct RepackParams {
    RepackSrc src[3];
    int n_src, mode, k, row_tiles, kt_pad;
    uint4* tiles;
    uint4* sb;
};

__device__ __forceinline__ bool repack_source_row(const RepackParams& p, int dest_row, int& which, int& row) {
    if (p.mode == 1) {  // two sources interleaved in runs of 8 rows
        const int tile = dest_row >> 4, r = dest_row & 15;
        which = r >> 3;
        row = tile * 8 + (r & 7);
        return row < p.src[which].n;
    }
    int r = dest_row;
    for (int i = 0; i < p.n_src; ++i) {
        if (r < p.src[i].n) { which = i; row = r; return true; }
        r -= p.src[i].n;
    }
    return false;
}

// one thread per destination 32-bit word
__global__ void repack_tiles_kernel(const RepackParams p) {
    const size_t total = (size_t)p.row_tiles * p.kt_pad * 128;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int j = idx & 3, lane = (idx >> 2) & 31;
    const size_t tile = idx >> 7;
    const int kt = (int)(tile % p.kt_pad), rt = (int)(tile / p.kt_pad);
    const int g = lane >> 2, t = lane & 3;
    unsigned out = 0;
    if (kt * 64 < p.k) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int dest_row = rt * 16 + g + 8 * (e & 1);
            const int col = kt * 64 + 16 * t + 4 * j + (e >> 2) + 2 * ((e >> 1) & 1);
            int which, row;
            if (repack_source_row(p, dest_row, which, row)) {
                const unsigned word = p.src[which].w[(size_t)row * (p.k / 8) + (col >> 3)];
                out |= ((word >> (4 * (col & 7))) & 0xFu) << (4 * e);
            }
        }
    }
    reinterpret_cast<unsigned*>(p.tiles)[idx] = out;
}

// one thread per (row tile, kt4, row, group-in-4) scale/zero pair
__global__ void repack_sb_kernel(const RepackParams p) {
    const size_t total = (size_t)p.row_tiles * (p.kt_pad / 4) * 64;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int i = idx & 3, r = (idx >> 2) & 15;
    const size_t blk = idx >> 6;
    const int kt4 = (int)(blk % (p.kt_pad / 4)), rt = (int)(blk / (p.kt_pad / 4));
    const int kt = kt4 * 4 + i;
    unsigned out = 0;
    int which, row;
    if (kt * 64 < p.k && repack_source_row(p, rt * 16 + r, which, row)) {
        const size_t gi = (size_t)row * (p.k / 64) + kt;
        out = (unsigned)p.src[which].scales[gi] | ((unsigned)p.src[which].biases[gi] << 16);
    }
    reinterpret_cast<unsigned*>(p.sb)[idx] = out;
}

__global__ void untile_bf16_kernel(const uint4* tiles, const uint4* sb, int n, int k, int kt_pad, int sb_f16,
                                   int interleaved, __nv_bfloat16* out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * k) return;
    const int row = (int)(idx / k), col = (int)(idx % k);
    (void)interleaved;
    const int rt = row >> 4, r = row & 15, kt = col >> 6, kk = col & 63;
    const int t = kk >> 4, j = (kk & 15) >> 2, sl = kk & 3;
    const int e = ((sl & 1) << 2) | ((sl >> 1) << 1) | (r >> 3), g = r & 7;
    const unsigned word = reinterpret_cast<const unsigned*>(tiles)[(((size_t)rt * kt_pad + kt) * 32 + (g * 4 + t)) * 4 + j];
    const unsigned q = (word >> (4 * e)) & 0xFu;
    const unsigned pair = reinterpret_cast<const unsigned*>(sb)[(((size_t)rt * (kt_pad / 4) + (kt >> 2)) * 16 + r) * 4 + (kt & 3)];
    const float s = half_bits_to_float(pair & 0xFFFFu, sb_f16), z = half_bits_to_float(pair >> 16, sb_f16);
    out[idx] = __float2bfloat16_rn(s * (float)q + z);
}

}  // namespace

int launch_repack(const RepackSrc* src, int n_src, int mode, int k, const Q4Tiled& dst, cudaStream_t s) {
    if (n_src < 1 || n_src > 3 || (mode == 1 && n_src != 2)) { set_error("repack: bad source count"); return SWLM_ERR_INVALID; }
    {   // an error left behind by an earlier, unrelated runtime call must not be blamed on this launch
        cudaError_t stale = cudaGetLastError();
        if (stale != cudaSuccess) { set_error("stale CUDA error %d (%s) found before the repack launch", (int)stale, cudaGetErrorString(stale)); return SWLM_ERR_CUDA; }
    }
    RepackParams p{};
    for (int i = 0; i < n_src; ++i) p.src[i] = src[i];
    p.n_src = n_src; p.mode = mode; p.k = k; p.row_tiles = dst.row_tiles; p.kt_pad = dst.kt_pad;
    p.tiles = dst.tiles; p.sb = dst.sb;
    const size_t words = (size_t)dst.row_tiles * dst.kt_pad * 128;
    repack_tiles_kernel<<<(unsigned)((words + 255) / 256), 256, 0, s>>>(p);
    const size_t pairs = (size_t)dst.row_tiles * (dst.kt_pad / 4) * 64;
    repack_sb_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, s>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "repack launch");
    return SWLM_OK;
}

int launch_untile_bf16(const Q4Tiled& t, __nv_bfloat16* out, cudaStream_t s) {
    const size_t total = (size_t)t.n * t.k;
    untile_bf16_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(t.tiles, t.sb, t.n, t.k, t.kt_pad, t.sb_f16 ? 1 : 0,
                                                                      t.interleaved ? 1 : 0, out);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "untile launch");
    return SWLM_OK;
}

}  // namespace swlm
