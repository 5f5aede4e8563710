// Declarations shared by the quantised GEMV kernels: the launch parameters and the fused
// residual-add / copy / RMSNorm prologue of the single-sequence kernels.
#pragma once

#include "swlm_internal.h"
#include "tp_device.cuh"

namespace swlm {
namespace {

struct QGemvParams {
    const uint4* tiles;
    const uint4* sb;
    int row_tiles, kt4_total, sb_f16;
    const __nv_bfloat16* x;
    int x_stride, k;
    __nv_bfloat16* y[3];
    int y_stride[3], seg_end[3];
    int m;
    int si, sk;   // k-slices per CTA group, CTA groups along K
    int si_shift; // log2(si) for the batch-1 kernel
    int cta_mode; // batch-1 kernel: slices of a row tile live in one CTA and meet in shared memory
    int pre_stages;               // batch-1 kernel: ring stages requested before the wait for the preceding kernel
    int bulk_stages;              // batch-1 kernel: stages per CTA asked into L2 up front
    int ring_late;                // batch-1 kernel: ring stages held back until the activations are in shared memory
    int idx32;                    // batch-1 kernel: the share arithmetic (stages x warps, units x CTAs) fits 32 bits
    float* partial;
    unsigned* counters;
    // optional fused residual-add / copy / RMSNorm in front of the product (norm_mode = step kind, 0 = none)
    int gated_act;   // activation of the gated epilogue (GATED_ACT_*)
    int norm_mode;
    const __nv_bfloat16* res_in;
    __nv_bfloat16* res_out;
    int res_stride;
    const __nv_bfloat16* norm_w;
    float eps, weight_bias;
    // tensor parallel: push = this product's rows are partial sums that go to every rank's exchange buffer;
    // in_tp = the fused norm's input is the sum of the partials the preceding product pushed
    int push, in_tp;
    TpParams tp;
    // phase timestamps (SWLM_TRACE=1): [cta][4] = kernel entry, predecessor complete, activations ready, done
    unsigned long long* trace;
    PrefetchTarget prefetch;
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Fused fused_copy_rms_norm / fused_residual_add_copy_rms_norm / fused_residual_add_rms_norm
// (Primitives/Reduction.swift:74-115 with CopyFragment / ResidualAddFragment,
// Compiler/MetalEntryCollector.swift:143-218) as the prologue of a single-sequence product: every thread owns
// the run of 8 elements k0..k0+7 (dimension <= 4096): h = in (+ residual) in fp32, residual_out = bf16(h)
// (written by one CTA only), then bf16(h * rsqrt(mean(h^2)+eps) * (w+bias)) returned as floats holding
// bf16-rounded numbers. The norm sees the unrounded sum, as the reference's fused kernel does. res_in and
// res_out are different buffers: other CTAs read res_in while one writes res_out.
// The global loads of a run, issued ahead of their use (the caller puts other memory traffic between the two).
struct NormRunLoads { uint4 x, res, nw; };
__device__ __forceinline__ NormRunLoads fused_norm_load8(const QGemvParams& p, int k0, bool in_range) {
    NormRunLoads l;
    l.x = l.res = l.nw = make_uint4(0, 0, 0, 0);
    if (in_range) {   // (the caller fills in the norm weights, which it requested earlier)
        if (!p.in_tp) l.x = __ldcg(reinterpret_cast<const uint4*>(p.x + k0));
        if (p.norm_mode != SWLM_STEP_COPY_RMSNORM) l.res = __ldcg(reinterpret_cast<const uint4*>(p.res_in + k0));
    }
    return l;
}
__device__ __forceinline__ void fused_norm_run8(const QGemvParams& p, int k0, bool in_range, bool writer,
                                                float* red, float (&xf)[8], int tp_epoch, int nwarps, const NormRunLoads& pre) {
    float h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = 0.f;
    uint4 nw4 = make_uint4(0, 0, 0, 0);
    if (in_range) {
        nw4 = pre.nw;
        if (p.in_tp) {
            const int par = tp_epoch & 1;
            tp_add_tagged_all<4>(p.tp, p.tp.lay.recv_ar(par, 0, 0) + (size_t)k0 * 8, p.tp.lay.recv_ar(par, 1, 0) - p.tp.lay.recv_ar(par, 0, 0), tp_epoch, h);
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = __bfloat162float(__float2bfloat16_rn(h[i]));
        } else {
            const uint4 v = pre.x;
            const unsigned vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) { h[2 * i] = __uint_as_float(vw[i] << 16); h[2 * i + 1] = __uint_as_float(vw[i] & 0xFFFF0000u); }
        }
        if (p.norm_mode != SWLM_STEP_COPY_RMSNORM) {
            const uint4 r = pre.res;
            const unsigned rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) { h[2 * i] += __uint_as_float(rw[i] << 16); h[2 * i + 1] += __uint_as_float(rw[i] & 0xFFFF0000u); }
        }
        if (writer && p.norm_mode != SWLM_STEP_RESADD_RMSNORM) {
            unsigned o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 v = __floats2bfloat162_rn(h[2 * i], h[2 * i + 1]);
                o[i] = *reinterpret_cast<const unsigned*>(&v);
            }
            *reinterpret_cast<uint4*>(p.res_out + k0) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(h[i], h[i], ss);
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < nwarps; ++i) total += red[i];
    const float rs = rsqrtf(total / (float)p.k + p.eps);
    const unsigned nw[4] = {nw4.x, nw4.y, nw4.z, nw4.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(h[2 * i] * rs * (__uint_as_float(nw[i] << 16) + p.weight_bias),
                                                       h[2 * i + 1] * rs * (__uint_as_float(nw[i] & 0xFFFF0000u) + p.weight_bias));
        const unsigned bits = *reinterpret_cast<const unsigned*>(&v);
        xf[2 * i] = __uint_as_float(bits << 16);
        xf[2 * i + 1] = __uint_as_float(bits & 0xFFFF0000u);
    }
}


}  // namespace
}  // namespace swlm
