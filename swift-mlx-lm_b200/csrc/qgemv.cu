// Q4 group-64 affine GEMV / small-M GEMM for sm_100a.
//
// Replaces the reference's `gemv_q4_g64` (Generator/MetalSourceGenerator+Quantized.swift:496-575,
// one SIMD-group per output row, one byte load per weight) and, for 1 < M <= 16, its
// `gemm_q4_g64` (:88-156, which re-reads the weights once per sequence position).
//
// Design: the kernel is HBM-bound on the 0.5625 bytes/weight stream, and on B200 the
// per-weight instruction budget is the second limit, so
//   * weights are re-tiled at upload into 512-byte tiles (16 rows x 64 columns) laid out in
//     mma.m16n8k16 A-fragment order: one 16-byte load per lane per tile, no shuffles;
//   * every warp streams its tiles through a private cp.async ring in shared memory
//     (kStages deep), so loads stay in flight independent of register pressure;
//   * a nibble pair becomes two bf16 values 128+q with one LOP3 ((w>>s) & 0x000F000F | 0x43004300);
//     the tensor core forms sum((128+q)*x) per group in fp32, and the group epilogue applies
//     scale*(acc - 128*sum(x)) + zero*sum(x) in fp32 — algebraically the reference's
//     sum((scale*q+zero)*x), with q and x exact in bf16 and products exact in fp32;
//   * the B operand holds up to 16 sequences (columns), so batch <= 16 costs the same weight traffic.
#include <algorithm>

#include "swlm_internal.h"

namespace swlm {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 4;                 // ring depth per warp; one stage = 4 k-tiles + their scales
constexpr int kStageBytes = 4 * 512 + 256;
constexpr int kRingBytes = kWarps * kStages * kStageBytes;
constexpr int kXPad = 8;                   // bf16 elements of padding per x row (bank skew)
constexpr int kMaxXBytes = 96 * 1024;

struct QGemvParams {
    const uint4* tiles;
    const uint4* sb;
    int row_tiles, kt4_total, sb_f16;
    const __nv_bfloat16* x;
    int x_stride, k;
    __nv_bfloat16* y[3];
    int y_stride[3], seg_end[3];
    int m;
    int rw, sw, sk;
    float* partial;
    unsigned* counters;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem) : "memory");
}
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

__device__ __forceinline__ float half_bits_to_float(unsigned bits16, int is_f16) {
    return is_f16 ? __half2float(__ushort_as_half((unsigned short)bits16)) : __uint_as_float(bits16 << 16);
}

template <int NT, int EPI>
__global__ void __launch_bounds__(kThreads, 2) qgemv_kernel(const QGemvParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int COLS = 8 * NT;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // k-range of this CTA and of this warp, in units of 4 k-tiles (256 columns)
    const int c0 = (int)(((long long)blockIdx.y * p.kt4_total) / p.sk);
    const int c1 = (int)(((long long)(blockIdx.y + 1) * p.kt4_total) / p.sk);
    const int nk_cta = (c1 - c0) * 256;
    const int xs_stride = nk_cta + kXPad;
    const int rows_x = p.m < COLS ? p.m : COLS;

    unsigned char* ring = smem;
    __nv_bfloat16* xperm = reinterpret_cast<__nv_bfloat16*>(smem + kRingBytes);
    float* xsum = reinterpret_cast<float*>(smem + kRingBytes + (size_t)rows_x * xs_stride * 2);

    const int rt = blockIdx.x * p.rw + warp / p.sw;
    const int ks = warp % p.sw;
    const bool active = rt < p.row_tiles;
    const int w0 = c0 + (ks * (c1 - c0)) / p.sw;
    const int w1 = c0 + ((ks + 1) * (c1 - c0)) / p.sw;
    const int nst = active ? (w1 - w0) : 0;

    unsigned char* my_ring = ring + warp * (kStages * kStageBytes);
    const uint4* tile_src = p.tiles + ((size_t)rt * p.kt4_total * 4) * 32;
    const uint4* sb_src = p.sb + (size_t)rt * p.kt4_total * 16;

    auto issue = [&](int i) {
        if (i < nst) {
            const int kt4 = w0 + i;
            unsigned char* dst = my_ring + (i % kStages) * kStageBytes;
            const uint4* src = tile_src + (size_t)kt4 * 128;
#pragma unroll
            for (int q = 0; q < 4; ++q) cp_async16(dst + (q * 32 + lane) * 16, src + q * 32 + lane);
            if (lane < 16) cp_async16(dst + 2048 + lane * 16, sb_src + (size_t)kt4 * 16 + lane);
        }
        cp_async_commit();
    };

    // Weights do not depend on the activations: start streaming before x is staged.
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) issue(i);

    // ---- stage x: permute each 64-element group into B-fragment order and sum it -------------
    {
        const int chunks_per_row = nk_cta / 8;
        const int total = rows_x * chunks_per_row;
        for (int idx = tid; idx < total; idx += kThreads) {
            const int b = idx / chunks_per_row, cc = idx - b * chunks_per_row;
            const int kglob = c0 * 256 + cc * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (kglob < p.k) v = *reinterpret_cast<const uint4*>(p.x + (size_t)b * p.x_stride + kglob);
            const int ktl = cc >> 3, c = cc & 7, j = c >> 1, half = c & 1;
            unsigned* dst = reinterpret_cast<unsigned*>(xperm + (size_t)b * xs_stride + ktl * 64 + j * 4 + half * 2);
            dst[0] = v.x;   // t = 0 : elements 2t, 2t+1 of this half
            dst[8] = v.y;   // t = 1 (16 bf16 = 8 words apart)
            dst[16] = v.z;
            dst[24] = v.w;
            float s = __uint_as_float(v.x << 16) + __uint_as_float(v.x & 0xFFFF0000u) +
                      __uint_as_float(v.y << 16) + __uint_as_float(v.y & 0xFFFF0000u) +
                      __uint_as_float(v.z << 16) + __uint_as_float(v.z & 0xFFFF0000u) +
                      __uint_as_float(v.w << 16) + __uint_as_float(v.w & 0xFFFF0000u);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (c == 0) xsum[ktl * COLS + b] = s;
        }
    }
    __syncthreads();

    float tot[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.f;

    for (int i = 0; i < nst; ++i) {
        issue(i + kStages - 1);
        cp_async_wait<kStages - 1>();
        __syncwarp();
        const unsigned char* st = my_ring + (i % kStages) * kStageBytes;
        const uint4* wsm = reinterpret_cast<const uint4*>(st);
        const uint4 sA = reinterpret_cast<const uint4*>(st + 2048)[g];
        const uint4 sB = reinterpret_cast<const uint4*>(st + 2048)[g + 8];
        const unsigned sAw[4] = {sA.x, sA.y, sA.z, sA.w};
        const unsigned sBw[4] = {sB.x, sB.y, sB.z, sB.w};
        const int ktl0 = (w0 + i - c0) * 4;
#pragma unroll
        for (int ti = 0; ti < 4; ++ti) {
            const uint4 wv = wsm[ti * 32 + lane];
            const unsigned wr[4] = {wv.x, wv.y, wv.z, wv.w};
            const int ktl = ktl0 + ti;
            uint4 X0[NT], X1[NT];
            float acc[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
                const int col = 8 * nt + g;
                if (col < p.m) {
                    const uint4* xp = reinterpret_cast<const uint4*>(xperm + (size_t)col * xs_stride + ktl * 64 + t * 16);
                    X0[nt] = xp[0];
                    X1[nt] = xp[1];
                } else {
                    X0[nt] = make_uint4(0, 0, 0, 0);
                    X1[nt] = make_uint4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const unsigned r = wr[j];
                const unsigned a0 = (r & 0x000F000Fu) | 0x43004300u;
                const unsigned a1 = ((r >> 4) & 0x000F000Fu) | 0x43004300u;
                const unsigned a2 = ((r >> 8) & 0x000F000Fu) | 0x43004300u;
                const unsigned a3 = ((r >> 12) & 0x000F000Fu) | 0x43004300u;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const unsigned b0 = j == 0 ? X0[nt].x : j == 1 ? X0[nt].z : j == 2 ? X1[nt].x : X1[nt].z;
                    const unsigned b1 = j == 0 ? X0[nt].y : j == 1 ? X0[nt].w : j == 2 ? X1[nt].y : X1[nt].w;
                    mma_bf16(acc[nt], a0, a1, a2, a3, b0, b1);
                }
            }
            // group epilogue: sum_k (s*q + z)*x = s*(acc - 128*xsum) + z*xsum
            const float s_lo = half_bits_to_float(sAw[ti] & 0xFFFFu, p.sb_f16);
            const float z_lo = half_bits_to_float(sAw[ti] >> 16, p.sb_f16);
            const float s_hi = half_bits_to_float(sBw[ti] & 0xFFFFu, p.sb_f16);
            const float z_hi = half_bits_to_float(sBw[ti] >> 16, p.sb_f16);
            const float zp_lo = fmaf(-128.f, s_lo, z_lo);
            const float zp_hi = fmaf(-128.f, s_hi, z_hi);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float2 xs2 = *reinterpret_cast<const float2*>(xsum + ktl * COLS + 8 * nt + 2 * t);
                tot[nt][0] = fmaf(s_lo, acc[nt][0], fmaf(zp_lo, xs2.x, tot[nt][0]));
                tot[nt][1] = fmaf(s_lo, acc[nt][1], fmaf(zp_lo, xs2.y, tot[nt][1]));
                tot[nt][2] = fmaf(s_hi, acc[nt][2], fmaf(zp_hi, xs2.x, tot[nt][2]));
                tot[nt][3] = fmaf(s_hi, acc[nt][3], fmaf(zp_hi, xs2.y, tot[nt][3]));
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();

    // ---- reduce the in-CTA k-splits through shared memory ---------------------------------------
    if (p.sw > 1) {
        __syncthreads();  // every warp is done with its ring
        float* red = reinterpret_cast<float*>(smem);
        float* mine = red + warp * (16 * COLS);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            *reinterpret_cast<float2*>(mine + g * COLS + 8 * nt + 2 * t) = make_float2(tot[nt][0], tot[nt][1]);
            *reinterpret_cast<float2*>(mine + (g + 8) * COLS + 8 * nt + 2 * t) = make_float2(tot[nt][2], tot[nt][3]);
        }
        __syncthreads();
        if (ks == 0) {
            for (int o = 1; o < p.sw; ++o) {
                const float* other = red + (warp + o) * (16 * COLS);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const float2 lo = *reinterpret_cast<const float2*>(other + g * COLS + 8 * nt + 2 * t);
                    const float2 hi = *reinterpret_cast<const float2*>(other + (g + 8) * COLS + 8 * nt + 2 * t);
                    tot[nt][0] += lo.x; tot[nt][1] += lo.y; tot[nt][2] += hi.x; tot[nt][3] += hi.y;
                }
            }
        }
    }

    // ---- reduce the cross-CTA k-splits through global scratch; the last CTA to arrive finishes ----
    if (p.sk > 1) {
        __shared__ int is_last;
        if (ks == 0 && active) {
            float* dst = p.partial + (((size_t)rt * p.sk + blockIdx.y) * 16) * COLS;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                *reinterpret_cast<float2*>(dst + g * COLS + 8 * nt + 2 * t) = make_float2(tot[nt][0], tot[nt][1]);
                *reinterpret_cast<float2*>(dst + (g + 8) * COLS + 8 * nt + 2 * t) = make_float2(tot[nt][2], tot[nt][3]);
            }
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned prev = atomicAdd(p.counters + blockIdx.x, 1u);
            is_last = (prev == (unsigned)p.sk - 1u);
            if (is_last) p.counters[blockIdx.x] = 0u;  // ready for the next launch
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        if (ks == 0 && active) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.f;
            for (int s = 0; s < p.sk; ++s) {  // fixed order: results do not depend on arrival order
                const float* src = p.partial + (((size_t)rt * p.sk + s) * 16) * COLS;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const float2 lo = __ldcg(reinterpret_cast<const float2*>(src + g * COLS + 8 * nt + 2 * t));
                    const float2 hi = __ldcg(reinterpret_cast<const float2*>(src + (g + 8) * COLS + 8 * nt + 2 * t));
                    tot[nt][0] += lo.x; tot[nt][1] += lo.y; tot[nt][2] += hi.x; tot[nt][3] += hi.y;
                }
            }
        }
    }

    if (ks != 0 || !active) return;

    // ---- epilogue ----------------------------------------------------------------------------------
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = 8 * nt + 2 * t + e;
            if (col >= p.m) continue;
            if (EPI == QGEMV_EPI_STORE) {
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
                    const float act = gate * (1.0f / (1.0f + expf(-gate))) * up;
                    p.y[0][(size_t)col * p.y_stride[0] + r] = __float2bfloat16_rn(act);
                }
            }
        }
    }
}

struct QGemvConfig {
    int nt, rw, sw, sk;
    dim3 grid;
    size_t smem;
};

QGemvConfig pick_config(const Q4Tiled& w, int m) {
    QGemvConfig c{};
    c.nt = m <= 8 ? 1 : 2;
    const int cols = 8 * c.nt;
    const int rows_x = std::min(m, cols);
    const int kt4 = w.kt_pad / 4;
    // cross-CTA split until the x slice fits in shared memory
    c.sk = 1;
    while ((size_t)rows_x * ((size_t)256 * ((kt4 + c.sk - 1) / c.sk) + kXPad) * 2 > (size_t)kMaxXBytes && c.sk < kt4) ++c.sk;
    const int kt4_cta = std::max(1, kt4 / c.sk);
    // in-CTA split: enough warps to cover two resident CTAs on each of the 148 SMs
    c.sw = 1;
    while (c.sw < kWarps && (long long)w.row_tiles * c.sw * c.sk < 8LL * 296 && kt4_cta / (c.sw * 2) >= 1) c.sw *= 2;
    c.rw = kWarps / c.sw;
    c.grid = dim3((unsigned)((w.row_tiles + c.rw - 1) / c.rw), (unsigned)c.sk, 1);
    const int nk_cta_max = 256 * ((kt4 + c.sk - 1) / c.sk);
    c.smem = (size_t)kRingBytes + (size_t)rows_x * (nk_cta_max + kXPad) * 2 + (size_t)(nk_cta_max / 64) * cols * 4;
    return c;
}

template <int NT, int EPI>
int launch_t(const QGemvParams& p, const QGemvConfig& c, cudaStream_t s) {
    qgemv_kernel<NT, EPI><<<c.grid, kThreads, c.smem, s>>>(p);
    cudaError_t e = cudaGetLastError();
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

int qgemv_init() {
    int rc;
    if ((rc = opt_in_smem(qgemv_kernel<1, 0>))) return rc;
    if ((rc = opt_in_smem(qgemv_kernel<1, 1>))) return rc;
    if ((rc = opt_in_smem(qgemv_kernel<2, 0>))) return rc;
    if ((rc = opt_in_smem(qgemv_kernel<2, 1>))) return rc;
    return SWLM_OK;
}

size_t qgemv_scratch_floats(const Q4Tiled& w, int m) {
    QGemvConfig c = pick_config(w, m);
    if (c.sk <= 1) return 0;
    return (size_t)w.row_tiles * c.sk * 16 * (8 * c.nt);
}
int qgemv_counter_count(const Q4Tiled& w) { return w.row_tiles; }

int launch_qgemv(const QGemvLaunch& a, cudaStream_t s) {
    const Q4Tiled& w = *a.w;
    if (a.m < 1 || a.m > 16) { set_error("qgemv: m=%d outside 1..16", a.m); return SWLM_ERR_INVALID; }
    if ((a.x_stride & 7) || (reinterpret_cast<uintptr_t>(a.x) & 15)) {
        set_error("qgemv: x must be 16-byte aligned with a stride that is a multiple of 8 elements");
        return SWLM_ERR_INVALID;
    }
    QGemvConfig c = pick_config(w, a.m);
    if (g_max_dyn_smem == 0 || c.smem > (size_t)g_max_dyn_smem) { set_error("qgemv: shared memory %zu exceeds the limit %d", c.smem, g_max_dyn_smem); return SWLM_ERR_INVALID; }
    if (c.sk > 1 && (!a.partial || !a.counters)) { set_error("qgemv: split-K launch without scratch"); return SWLM_ERR_INVALID; }
    QGemvParams p{};
    p.tiles = w.tiles; p.sb = w.sb; p.row_tiles = w.row_tiles; p.kt4_total = w.kt_pad / 4; p.sb_f16 = w.sb_f16 ? 1 : 0;
    p.x = a.x; p.x_stride = a.x_stride; p.k = w.k;
    for (int i = 0; i < 3; ++i) {
        p.y[i] = a.y[i]; p.y_stride[i] = a.y_stride[i];
        p.seg_end[i] = a.seg_end[i] > 0 ? a.seg_end[i] : (i ? p.seg_end[i - 1] : 0);
    }
    p.m = a.m;
    p.rw = c.rw; p.sw = c.sw; p.sk = c.sk; p.partial = a.partial; p.counters = a.counters;
    if (a.epilogue == QGEMV_EPI_SWIGLU) return c.nt == 1 ? launch_t<1, 1>(p, c, s) : launch_t<2, 1>(p, c, s);
    return c.nt == 1 ? launch_t<1, 0>(p, c, s) : launch_t<2, 0>(p, c, s);
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
            const int col = kt * 64 + 16 * j + 2 * t + (e >> 2) + 8 * ((e >> 1) & 1);
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
    const int j = kk >> 4, w16 = kk & 15;
    const int t = (w16 & 7) >> 1, e = ((w16 & 1) << 2) | ((w16 >> 3) << 1) | (r >> 3), g = r & 7;
    const unsigned word = reinterpret_cast<const unsigned*>(tiles)[(((size_t)rt * kt_pad + kt) * 32 + (g * 4 + t)) * 4 + j];
    const unsigned q = (word >> (4 * e)) & 0xFu;
    const unsigned pair = reinterpret_cast<const unsigned*>(sb)[(((size_t)rt * (kt_pad / 4) + (kt >> 2)) * 16 + r) * 4 + (kt & 3)];
    const float s = half_bits_to_float(pair & 0xFFFFu, sb_f16), z = half_bits_to_float(pair >> 16, sb_f16);
    out[idx] = __float2bfloat16_rn(s * (float)q + z);
}

}  // namespace

int launch_repack(const RepackSrc* src, int n_src, int mode, int k, const Q4Tiled& dst, cudaStream_t s) {
    if (n_src < 1 || n_src > 3 || (mode == 1 && n_src != 2)) { set_error("repack: bad source count"); return SWLM_ERR_INVALID; }
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
