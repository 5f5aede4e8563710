// Single-sequence Q4 group-64 GEMV on the 5th-generation tensor cores (tcgen05 / TMEM) for sm_100a.
//
// Same contract as gemv_q4_g64 (Generator/MetalSourceGenerator+Quantized.swift:496-575): y[N] = W_deq[N,K] . x[K],
// W = scale * q + zero per group of 64, fp32 accumulation. The legacy mma.sync path spends about 70 issue slots per
// 512 bytes of weights (nibble unpacking, per-lane post-processing of which 3/4 is wasted, address arithmetic)
// and is bound by instruction issue near 6 TB/s of weight stream, whether the weights come from HBM or from L2.
// Here a warp never touches individual weights:
//   * Weights are stored as shared-memory images (Q4Umma): a tile is 256 rows x 128 columns; byte (i, k) holds
//     the nibble of row i (low) and of row i + 128 (high) for column k, laid out K-major with the 128-byte
//     swizzle tcgen05.mma reads. One cp.async.bulk brings a tile (16 KB + 2 KB of scale/zero pairs) into a stage.
//   * The tensor core multiplies the bytes AS THEY ARE (u8 = lo + 16 * hi) and a copy with the high nibbles masked
//     off (one AND per 4 bytes, the only per-weight work left on the CUDA cores) by the activations, which are
//     held in block floating point (per group of 64: a power-of-two exponent, 15-bit integers as two signed-byte
//     digits = two columns of the B operand). Integer sums are exact: rows i come from the masked product, rows
//     i + 128 from (raw - masked) / 16.
//   * One accumulator set per quantisation group lives in TMEM; 128 threads (one per TMEM lane = byte row) read
//     their sums with tcgen05.ld and apply the group's scale and zero once, in fp32.
//   * Warp roles: bulk-copy producer, MMA issuer, 4 masking warps, 4 epilogue warps, coupled by mbarriers; all
//     waits are bounded (error word + orderly exit instead of a hang).
// Tiles are dealt to the CTAs (one per SM) as equal contiguous ranges of the [row block][k chunk] order; a row
// block cut by a range boundary is summed through global scratch by the last CTA to arrive, in range order.
#include "qgemv_common.cuh"

namespace swlm {
namespace {

constexpr int kTcgThreads = 512;       // warp 0 producer, warp 1 MMA, warps 2-5 masking, warps 6-9 epilogue; the rest
                                       // only help to prepare the activations (512 threads x 8 = one pass over 4096)
constexpr int kTileA = 16384;          // 128 byte-rows x 128 bytes
constexpr int kTileSb = 2048;          // uint2[2 groups][128 byte-rows]
constexpr int kTileBytes = kTileA + kTileSb;
constexpr int kTileB = 2048;           // activations: 16 rows (two digits, the rest zero) x 128 bytes; with M = 128
                                       // the smallest N tcgen05.mma accepts is 16
constexpr int kStageBytes2 = kTileBytes + kTileA + kTileB;  // raw + pairs + masked + B
constexpr int kAccSlots = 4;           // accumulator sets in TMEM: 4 accumulators of 16 columns each
constexpr int kTmemCols = 256;
constexpr int kSpin = 1 << 22;

__device__ __forceinline__ unsigned s_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(unsigned long long* b, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_addr(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(unsigned long long* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_addr(b)) : "memory");
}
__device__ __forceinline__ bool bar_wait(unsigned long long* b, unsigned parity) {
    const unsigned a = s_addr(b);
    for (int spin = 0; spin < kSpin; ++spin) {
        unsigned done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(a), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart, descriptor version 1
__device__ __forceinline__ unsigned long long umma_desc128(unsigned smem_addr) {
    return (unsigned long long)((smem_addr & 0x3FFFFu) >> 4) | ((unsigned long long)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::i8: D = s32, A = u8, B = s8, both K-major, M = 128, N = 16
constexpr unsigned kIdescI8 = (2u << 4) | (0u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
__device__ __forceinline__ void umma_i8(unsigned d_tmem, unsigned long long a, unsigned long long b, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a), "l"(b), "r"(kIdescI8), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_to(unsigned long long* b) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_addr(b)) : "memory");
}
__device__ __forceinline__ void tmem_ld2(unsigned taddr, int& a, int& b) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0,%1}, [%2];" : "=r"(a), "=r"(b) : "r"(taddr) : "memory");
}

template <bool F16SB>
__device__ __forceinline__ float pair_scale(unsigned pair) {
    return F16SB ? __half2float(__ushort_as_half((unsigned short)(pair & 0xFFFFu))) : __uint_as_float(pair << 16);
}
template <bool F16SB>
__device__ __forceinline__ float pair_zero(unsigned pair) {
    return F16SB ? __half2float(__ushort_as_half((unsigned short)(pair >> 16))) : __uint_as_float(pair & 0xFFFF0000u);
}

// owner of tile t when `total` tiles are dealt to `parts` CTAs as [c * total / parts, (c + 1) * total / parts)
__device__ __forceinline__ int tile_owner(long long t, int total, int parts) {
    int c = (int)(((t + 1) * parts - 1) / total);
    while (c > 0 && (long long)c * total / parts > t) --c;
    while (c + 1 < parts && (long long)(c + 1) * total / parts <= t) ++c;
    return c;
}

template <int EPI, bool F16SB>
__global__ void __launch_bounds__(kTcgThreads, 1) qgemv_tc_kernel(const QGemvParams p, int stages) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024 - (s_addr(smem_raw) & 1023)) & 1023);
    __shared__ __align__(8) unsigned long long full_bar[8], masked_bar[8], free_bar[8], acc_full[kAccSlots], acc_free[kAccSlots];
    __shared__ unsigned tmem_base_s;
    __shared__ volatile int failed;
    __shared__ float red[kTcgThreads / 32];
    __shared__ int fin_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunks = p.chunks, total = p.row_blocks * chunks, parts = gridDim.x;
    const int t0 = (int)((long long)blockIdx.x * total / parts), t1 = (int)((long long)(blockIdx.x + 1) * total / parts);
    const int ntiles = t1 - t0;
    const int kt_total = chunks * 2;  // groups of 64
    if (p.trace && tid == 0) p.trace[blockIdx.x * 4] = global_timer_ns();

    unsigned char* xd_hi = smem + (size_t)stages * kStageBytes2;     // high digits of x, one byte per element
    unsigned char* xd_lo = xd_hi + (size_t)chunks * 128;             // low digits
    float2* xmeta = reinterpret_cast<float2*>(xd_lo + (size_t)chunks * 128);  // per group {2^E, sum * 2^E}

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) { bar_init(&full_bar[s], 1); bar_init(&masked_bar[s], 128); bar_init(&free_bar[s], 129); }
        for (int a = 0; a < kAccSlots; ++a) { bar_init(&acc_full[a], 1); bar_init(&acc_free[a], 128); }
        failed = 0;
        fin_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(&tmem_base_s)), "r"((unsigned)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // rows 2..15 of every stage's B tile stay zero for the whole kernel (rows 0 and 1 carry the two digits)
    for (int i = tid; i < stages * (kTileB / 16); i += kTcgThreads) {
        const int s = i / (kTileB / 16), c = i % (kTileB / 16);
        *reinterpret_cast<uint4*>(smem + (size_t)s * kStageBytes2 + kTileBytes + kTileA + c * 16) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads these rows
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = tmem_base_s;
    if (p.trace && tid == 0) p.trace[(blockIdx.x + gridDim.x) * 4] = global_timer_ns();  // set-up done
    // A wait that gives up after its limit marks the CTA as failed; from then on nobody waits or issues any more,
    // but every thread still walks through all its tiles, so that barriers are met and the kernel ends.
    auto wait_or_fail = [&](unsigned long long* b, unsigned parity, int code) {
        if (failed) return;
        if (!bar_wait(b, parity)) { failed = 1; atomicExch(p.status, code); }
    };

    pdl_launch_dependents();
    // the weights do not depend on the preceding kernel: the first stages are requested before its results are awaited
    int issued = 0;
    auto issue_tile = [&](int n) {
        const int s = n % stages;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s_addr(&full_bar[s])), "r"((unsigned)kTileBytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(s_addr(smem + (size_t)s * kStageBytes2)), "l"(p.tc_tiles + (size_t)(t0 + n) * kTileBytes), "r"((unsigned)kTileBytes),
                       "r"(s_addr(&full_bar[s])) : "memory");
    };
    if (tid == 0) {
        for (; issued < stages && issued < ntiles; ++issued) issue_tile(issued);
    }
    pdl_wait();
    if (p.trace && tid == 0) p.trace[blockIdx.x * 4 + 1] = global_timer_ns();

    // ---- activations -> block floating point: per group of 64 a power-of-two exponent and 15-bit integers ----
    {
        const int nruns = kt_total * 8;
        for (int run = tid; run < nruns || (p.norm_mode && run < kTcgThreads); run += kTcgThreads) {
            const int k0 = run * 8;
            float xf[8];
            if (p.norm_mode) {
                fused_norm_run8(p, k0, k0 < p.k, blockIdx.x == 0, red, xf, 0, kTcgThreads >> 5, fused_norm_load8(p, k0, k0 < p.k));
                if (run >= nruns) continue;
            } else {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (k0 < p.k) v = __ldg(reinterpret_cast<const uint4*>(p.x + k0));
                const unsigned vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) { xf[2 * i] = __uint_as_float(vw[i] << 16); xf[2 * i + 1] = __uint_as_float(vw[i] & 0xFFFF0000u); }
            }
            const unsigned act = __activemask();
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(xf[i]));
            amax = fmaxf(amax, __shfl_xor_sync(act, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(act, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(act, amax, 4));
            const int e = (int)(__float_as_uint(amax) >> 23);
            const bool live = e >= 16 && e < 255;
            // largest magnitude -> [2^13, 2^14); adding 1.5 * 2^23 leaves the rounded integer v in the low mantissa
            // bits (two's complement): low byte = low digit, (v + 128) >> 8 = high digit, v = 256 * hi + lo
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
            uint2 hi, lo;
            lo.x = __byte_perm(__byte_perm(rb[0], rb[1], 0x0040), __byte_perm(rb[2], rb[3], 0x0040), 0x5410);
            lo.y = __byte_perm(__byte_perm(rb[4], rb[5], 0x0040), __byte_perm(rb[6], rb[7], 0x0040), 0x5410);
            hi.x = __byte_perm(__byte_perm(rh[0], rh[1], 0x0051), __byte_perm(rh[2], rh[3], 0x0051), 0x5410);
            hi.y = __byte_perm(__byte_perm(rh[4], rh[5], 0x0051), __byte_perm(rh[6], rh[7], 0x0051), 0x5410);
            *reinterpret_cast<uint2*>(xd_hi + k0) = hi;
            *reinterpret_cast<uint2*>(xd_lo + k0) = lo;
            const float scale = live ? __uint_as_float((unsigned)(e - 13) << 23) : 0.f;  // 2^(e - 140) = 1 / mul
            if ((run & 7) == 0) xmeta[run >> 3] = make_float2(scale, (float)sum * scale);
        }
    }
    __syncthreads();
    if (p.trace && tid == 0) p.trace[blockIdx.x * 4 + 2] = global_timer_ns();

    if (warp == 0) {
        // ---- producer: refill a stage as soon as its MMAs and its epilogue readers are done with it ----------
        if (lane == 0) {
            for (int n = issued; n < ntiles; ++n) {
                const int s = n % stages, u = n / stages;
                wait_or_fail(&free_bar[s], (unsigned)((u - 1) & 1), 1);
                if (failed) break;  // single thread, no barrier inside: nothing more is requested
                issue_tile(n);
                issued = n + 1;
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: per tile 2 groups x {masked, raw} x 2 k-steps of 32 -------------------------------
        if (lane == 0) {
            for (int n = 0; n < ntiles; ++n) {
                const int s = n % stages, u = n / stages, a = n % kAccSlots, ua = n / kAccSlots;
                wait_or_fail(&masked_bar[s], (unsigned)(u & 1), 2);
                if (ua > 0) wait_or_fail(&acc_free[a], (unsigned)((ua - 1) & 1), 3);
                if (failed) break;  // single thread, no barrier inside
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned st = s_addr(smem + (size_t)s * kStageBytes2);
                const unsigned a_raw = st, a_msk = st + kTileBytes, b_x = st + kTileBytes + kTileA;
                const unsigned d = tmem + (unsigned)a * 64u;
#pragma unroll
                for (int g = 0; g < 2; ++g) {
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks) {
                        const unsigned off = (unsigned)(g * 2 + ks) * 32u;  // 32 bytes along K inside the 128-byte row
                        umma_i8(d + (unsigned)g * 32u, umma_desc128(a_msk + off), umma_desc128(b_x + off), (unsigned)ks);
                        umma_i8(d + (unsigned)g * 32u + 16u, umma_desc128(a_raw + off), umma_desc128(b_x + off), (unsigned)ks);
                    }
                }
                umma_commit_to(&free_bar[s]);
                umma_commit_to(&acc_full[a]);
            }
            if (p.trace) p.trace[(blockIdx.x + 2 * gridDim.x) * 4] = global_timer_ns();
        }
    } else if (warp < 6) {
        // ---- masking warps: low-nibble copy of the tile and the two digit rows of the activations ----------
        const int mt = tid - 64;
        for (int n = 0; n < ntiles; ++n) {
            const int s = n % stages, u = n / stages;
            wait_or_fail(&full_bar[s], (unsigned)(u & 1), 4);
            if (failed) break;  // no barrier inside this loop
            unsigned char* st = smem + (size_t)s * kStageBytes2;
            const uint4* raw = reinterpret_cast<const uint4*>(st);
            uint4* msk = reinterpret_cast<uint4*>(st + kTileBytes);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                uint4 v = raw[mt + 128 * q];
                v.x &= 0x0F0F0F0Fu; v.y &= 0x0F0F0F0Fu; v.z &= 0x0F0F0F0Fu; v.w &= 0x0F0F0F0Fu;
                msk[mt + 128 * q] = v;
            }
            if (mt < 16) {
                const int c = (t0 + n) % chunks, row = mt >> 3, c16 = mt & 7;
                const uint4 v = *reinterpret_cast<const uint4*>((row ? xd_lo : xd_hi) + (size_t)c * 128 + c16 * 16);
                *reinterpret_cast<uint4*>(st + kTileBytes + kTileA + row * 128 + ((c16 ^ row) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            bar_arrive(&masked_bar[s]);
        }
        if (p.trace && mt == 0) p.trace[(blockIdx.x + 2 * gridDim.x) * 4 + 3] = global_timer_ns();
    } else if (warp < 10) {
        // ---- epilogue warps: thread = TMEM lane = byte row i, i.e. weight rows i (low nibbles) and i + 128 ---
        const int quarter = warp & 3, i = quarter * 32 + lane;
        float acc_lo = 0.f, acc_hi16 = 0.f, acc_hiz = 0.f;
        long long t_wait = 0, t_ld = 0;  // tracing only: clocks spent waiting for the MMAs / reading TMEM
        for (int n = 0; n < ntiles; ++n) {  // all 128 threads walk every tile: the loop contains named barriers
            const int s = n % stages, u = n / stages, a = n % kAccSlots, ua = n / kAccSlots;
            const int t = t0 + n, rbk = t / chunks, c = t - rbk * chunks;
            wait_or_fail(&full_bar[s], (unsigned)(u & 1), 5);
            const uint2* sbp = reinterpret_cast<const uint2*>(smem + (size_t)s * kStageBytes2 + kTileA);
            const uint2 sb0 = sbp[i], sb1 = sbp[128 + i];
            bar_arrive(&free_bar[s]);  // the pairs are in registers: the stage may be refilled once its MMAs are done
            const long long c0 = clock64();
            wait_or_fail(&acc_full[a], (unsigned)(ua & 1), 6);
            const long long c1 = clock64();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned ta = tmem + ((unsigned)(quarter * 32) << 16) + (unsigned)a * 64u;
            int m0h, m0l, r0h, r0l, m1h, m1l, r1h, r1l;
            tmem_ld2(ta, m0h, m0l); tmem_ld2(ta + 16u, r0h, r0l); tmem_ld2(ta + 32u, m1h, m1l); tmem_ld2(ta + 48u, r1h, r1l);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            t_wait += c1 - c0; t_ld += clock64() - c1;
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            bar_arrive(&acc_free[a]);
            const float2 x0 = xmeta[2 * c], x1 = xmeta[2 * c + 1];
            // columns 0 / 1 carry the high / low activation digits: sum = 256 * hi + lo, exact in s32
            const float v0 = (float)(m0h * 256 + m0l), w0 = (float)((r0h - m0h) * 256 + (r0l - m0l));
            const float v1 = (float)(m1h * 256 + m1l), w1 = (float)((r1h - m1h) * 256 + (r1l - m1l));
            acc_lo = fmaf(pair_scale<F16SB>(sb0.x) * x0.x, v0, fmaf(pair_zero<F16SB>(sb0.x), x0.y, acc_lo));
            acc_lo = fmaf(pair_scale<F16SB>(sb1.x) * x1.x, v1, fmaf(pair_zero<F16SB>(sb1.x), x1.y, acc_lo));
            acc_hi16 = fmaf(pair_scale<F16SB>(sb0.y) * x0.x, w0, acc_hi16);
            acc_hi16 = fmaf(pair_scale<F16SB>(sb1.y) * x1.x, w1, acc_hi16);
            acc_hiz = fmaf(pair_zero<F16SB>(sb0.y), x0.y, fmaf(pair_zero<F16SB>(sb1.y), x1.y, acc_hiz));

            // ---- end of this CTA's part of the row block? ------------------------------------------------
            const bool seg_end = c == chunks - 1 || n == ntiles - 1;
            if (!seg_end) continue;
            float r_lo = acc_lo, r_hi = fmaf(acc_hi16, 0.0625f, acc_hiz);
            acc_lo = acc_hi16 = acc_hiz = 0.f;
            const int c_begin = max(rbk * chunks, t0) - rbk * chunks;
            bool finisher = true;
            if (c_begin > 0 || c < chunks - 1) {
                // the row block is shared with other CTAs: partial sums meet in global scratch, the last to arrive
                // adds them in range order (independent of arrival order)
                const int slot = rbk == t0 / chunks ? 0 : 1;
                float* dst = p.partial + ((size_t)(blockIdx.x * 2 + slot) * 256);
                __stcg(dst + i, r_lo);
                __stcg(dst + 128 + i, r_hi);
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (i == 0) {
                    const int c_first = tile_owner((long long)rbk * chunks, total, parts);
                    const int c_last = tile_owner((long long)(rbk + 1) * chunks - 1, total, parts);
                    unsigned prev;
                    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(p.counters + rbk) : "memory");
                    const int last = prev == (unsigned)(c_last - c_first);
                    if (last) p.counters[rbk] = 0u;
                    fin_flag = last ? (c_first + 1) | ((c_last + 1) << 16) : 0;
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
                const int ff = fin_flag;
                finisher = ff != 0;
                if (finisher) {
                    const int c_first = (ff & 0xFFFF) - 1, c_last = (ff >> 16) - 1;
                    r_lo = r_hi = 0.f;
                    for (int cc = c_first; cc <= c_last; ++cc) {
                        const int cslot = rbk == (int)((long long)cc * total / parts) / chunks ? 0 : 1;
                        const float* src = p.partial + ((size_t)(cc * 2 + cslot) * 256);
                        r_lo += __ldcg(src + i);
                        r_hi += __ldcg(src + 128 + i);
                    }
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");  // fin_flag may be rewritten
            }
            if (!finisher) continue;
            if (EPI == QGEMV_EPI_STORE) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int r = rbk * 256 + i + 128 * h;
                    const __nv_bfloat16 val = __float2bfloat16_rn(h ? r_hi : r_lo);
                    if (r < p.seg_end[0]) p.y[0][r] = val;
                    else if (r < p.seg_end[1]) p.y[1][r - p.seg_end[0]] = val;
                    else if (r < p.seg_end[2]) p.y[2][r - p.seg_end[1]] = val;
                }
            } else {
                // low nibbles: gate row, high nibbles: the matching up row; both rounded to bf16 first, as the
                // reference stores them to bf16 scratch before `swiglu` reads them
                // (Primitives/ElementwiseFragment.swift:49-54)
                const int r = rbk * 128 + i;
                if (r < p.seg_end[0]) {
                    const float gate = __bfloat162float(__float2bfloat16_rn(r_lo));
                    const float up = __bfloat162float(__float2bfloat16_rn(r_hi));
                    p.y[0][r] = __float2bfloat16_rn(gate * (1.0f / (1.0f + expf(-gate))) * up);
                }
            }
        }
        if (p.trace && i == 0) {
            p.trace[(blockIdx.x + 2 * gridDim.x) * 4 + 2] = global_timer_ns();
            p.trace[(blockIdx.x + gridDim.x) * 4 + 3] = ((unsigned long long)t_wait << 32) | (unsigned long long)(t_ld & 0xFFFFFFFFll);
        }
    }

    // The single-thread roles leave their warps diverged; a diverged warp would arrive at the block-wide barrier
    // below twice (once per group of lanes) and release it before the last warps are there.
    __syncwarp();
    // ---- orderly exit: no bulk copy may still be in flight, TMEM goes back -------------------------------------
    if (failed && tid == 0) {
        for (int n = max(0, issued - stages); n < issued; ++n) bar_wait(&full_bar[n % stages], (unsigned)((n / stages) & 1));
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (p.trace && tid == 0) p.trace[blockIdx.x * 4 + 3] = global_timer_ns();
    if (p.trace && tid == 32) p.trace[(blockIdx.x + 2 * gridDim.x) * 4 + 1] = global_timer_ns();
    if (warp == 1) {
        const unsigned long long tb = p.trace ? global_timer_ns() : 0ull;
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((unsigned)kTmemCols) : "memory");
        if (p.trace && lane == 0) {
            p.trace[(blockIdx.x + gridDim.x) * 4 + 1] = global_timer_ns();  // TMEM released
            p.trace[(blockIdx.x + gridDim.x) * 4 + 2] = tb;                 // just before the release
        }
    }
}

// ---- re-tiling: MLX source layout -> shared-memory images -----------------------------------------------------
struct UmmaRepackParams {
    RepackSrc src[3];
    int n_src, mode, k, n_total, row_blocks, chunks;
    unsigned char* tiles;
};

// source row for destination row r of the concatenated sources; false: padding
__device__ __forceinline__ bool umma_src_row(const UmmaRepackParams& p, int r, int& which, int& row) {
    int base = 0;
    for (int s = 0; s < p.n_src; ++s) {
        if (r < base + p.src[s].n) { which = s; row = r - base; return true; }
        base += p.src[s].n;
    }
    return false;
}

// one thread per 16-byte chunk of a tile image (1024 per tile) plus 256 threads for the scale/zero pairs
__global__ void umma_repack_kernel(const UmmaRepackParams p) {
    const int tile = blockIdx.x, rbk = tile / p.chunks, c = tile - rbk * p.chunks;
    unsigned char* out = p.tiles + (size_t)tile * kTileBytes;
    const int words_per_row = p.k / 8, groups_per_row = p.k / 64;
    for (int idx = threadIdx.x; idx < 1024 + 256; idx += blockDim.x) {
        if (idx < 1024) {
            const int i = idx >> 3, c16 = idx & 7;  // byte row, logical 16-byte chunk (16 columns)
            const int k0 = c * 128 + c16 * 16;
            unsigned lo_w[2] = {0, 0}, hi_w[2] = {0, 0};
            for (int h = 0; h < 2; ++h) {
                int which = 0, row = 0;
                bool ok;
                if (p.mode == 1) { which = h; row = rbk * 128 + i; ok = row < p.src[h].n; }
                else ok = umma_src_row(p, rbk * 256 + i + 128 * h, which, row);
                if (ok && k0 < p.k) {
                    const uint32_t* w = p.src[which].w + (size_t)row * words_per_row + k0 / 8;
                    (h ? hi_w : lo_w)[0] = w[0];
                    (h ? hi_w : lo_w)[1] = w[1];
                }
            }
            unsigned o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // output word j = columns 4j..4j+3, one byte each
                unsigned word = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int col = 4 * j + e;
                    const unsigned lo = (lo_w[col >> 3] >> (4 * (col & 7))) & 0xFu, hi = (hi_w[col >> 3] >> (4 * (col & 7))) & 0xFu;
                    word |= (lo | (hi << 4)) << (8 * e);
                }
                o[j] = word;
            }
            *reinterpret_cast<uint4*>(out + i * 128 + ((c16 ^ (i & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
        } else {
            const int j = idx - 1024, g = j >> 7, i = j & 127;
            unsigned pr[2] = {0, 0};
            for (int h = 0; h < 2; ++h) {
                int which = 0, row = 0;
                bool ok;
                if (p.mode == 1) { which = h; row = rbk * 128 + i; ok = row < p.src[h].n; }
                else ok = umma_src_row(p, rbk * 256 + i + 128 * h, which, row);
                const int grp = c * 2 + g;
                if (ok && grp < groups_per_row)
                    pr[h] = (unsigned)p.src[which].scales[(size_t)row * groups_per_row + grp] | ((unsigned)p.src[which].biases[(size_t)row * groups_per_row + grp] << 16);
            }
            reinterpret_cast<uint2*>(out + kTileA)[g * 128 + i] = make_uint2(pr[0], pr[1]);
        }
    }
}

int g_tc_max_dyn = 0;

}  // namespace

size_t Q4Umma::bytes() const { return (size_t)row_blocks * chunks * kTileBytes; }

int launch_umma_repack(const RepackSrc* src, int n_src, int mode, int k, const Q4Umma& dst, cudaStream_t s) {
    if (n_src < 1 || n_src > 3 || (mode == 1 && n_src != 2) || (k & 63)) { set_error("umma repack: bad sources"); return SWLM_ERR_INVALID; }
    cudaError_t stale = cudaGetLastError();
    if (stale != cudaSuccess) { set_error("stale CUDA error %d (%s) found before the repack launch", (int)stale, cudaGetErrorString(stale)); return SWLM_ERR_CUDA; }
    UmmaRepackParams p{};
    for (int i = 0; i < n_src; ++i) p.src[i] = src[i];
    p.n_src = n_src; p.mode = mode; p.k = k; p.n_total = dst.n; p.row_blocks = dst.row_blocks; p.chunks = dst.chunks; p.tiles = dst.tiles;
    umma_repack_kernel<<<dst.row_blocks * dst.chunks, 256, 0, s>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "umma repack launch");
    return SWLM_OK;
}

int qgemv_tc_init() {
    int dev = 0, optin = 0;
    SWLM_CUDA(cudaGetDevice(&dev));
    SWLM_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cudaFuncAttributes fa;
    SWLM_CUDA(cudaFuncGetAttributes(&fa, qgemv_tc_kernel<0, false>));
    g_tc_max_dyn = optin - (int)fa.sharedSizeBytes - 64;
    SWLM_CUDA(cudaFuncSetAttribute(qgemv_tc_kernel<0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, g_tc_max_dyn));
    SWLM_CUDA(cudaFuncSetAttribute(qgemv_tc_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, g_tc_max_dyn));
    SWLM_CUDA(cudaFuncSetAttribute(qgemv_tc_kernel<0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, g_tc_max_dyn));
    SWLM_CUDA(cudaFuncSetAttribute(qgemv_tc_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, g_tc_max_dyn));
    return SWLM_OK;
}

size_t qgemv_tc_scratch_floats() { return (size_t)148 * 2 * 256; }
int qgemv_tc_counter_count(const Q4Umma& w) { return w.row_blocks; }

// Shared memory: `stages` stages (raw + pairs + masked + activations) + the digit store + group metadata.
static int tc_stages_for(const Q4Umma& w, size_t* smem_out) {
    const size_t x_bytes = (size_t)w.chunks * 256 + (size_t)w.chunks * 2 * sizeof(float2);
    int stages = 5;
    while (stages > 2 && (size_t)stages * kStageBytes2 + x_bytes + 1024 > (size_t)g_tc_max_dyn) --stages;
    *smem_out = (size_t)stages * kStageBytes2 + x_bytes + 1024;
    return stages;
}

bool qgemv_tc_supports(const Q4Umma& w, const QGemvLaunch& a) {
    if (a.m != 1 || a.push || a.in_tp || !w.tiles) return false;
    if (a.norm.mode && (w.k > 4096 || (w.k & 15))) return false;
    size_t smem;
    tc_stages_for(w, &smem);
    return smem <= (size_t)g_tc_max_dyn;
}

int launch_qgemv_tc(const Q4Umma& w, const QGemvLaunch& a, int* status, cudaStream_t s) {
    if (!qgemv_tc_supports(w, a)) { set_error("qgemv (tcgen05): launch not supported on this path"); return SWLM_ERR_UNSUPPORTED; }
    if ((a.x_stride & 7) || (reinterpret_cast<uintptr_t>(a.x) & 15)) { set_error("qgemv: x must be 16-byte aligned"); return SWLM_ERR_INVALID; }
    if (!a.partial || !a.counters || !status) { set_error("qgemv (tcgen05): scratch missing"); return SWLM_ERR_INVALID; }
    QGemvParams p{};
    p.tc_tiles = w.tiles; p.row_blocks = w.row_blocks; p.chunks = w.chunks; p.tc_interleaved = w.interleaved ? 1 : 0; p.sb_f16 = w.sb_f16 ? 1 : 0;
    p.x = a.x; p.x_stride = a.x_stride; p.k = w.k; p.m = 1;
    for (int i = 0; i < 3; ++i) {
        p.y[i] = a.y[i]; p.y_stride[i] = a.y_stride[i];
        p.seg_end[i] = a.seg_end[i] > 0 ? a.seg_end[i] : (i ? p.seg_end[i - 1] : 0);
    }
    p.partial = a.partial; p.counters = a.counters; p.status = status;
    p.norm_mode = a.norm.mode;
    if (a.norm.mode) {
        if (!a.norm.weight || a.norm.res_in == a.norm.res_out) { set_error("qgemv: fused norm needs distinct residual buffers"); return SWLM_ERR_INVALID; }
        p.res_in = a.norm.res_in; p.res_out = a.norm.res_out; p.res_stride = a.norm.res_stride;
        p.norm_w = a.norm.weight; p.eps = a.norm.eps; p.weight_bias = a.norm.weight_bias;
    }
    p.trace = qgemv_trace_slot(std::min(148, w.row_blocks * w.chunks), w.row_blocks * 16, w.chunks * 2, a.epilogue, a.norm.mode);
    size_t smem;
    const int stages = tc_stages_for(w, &smem);
    const dim3 grid((unsigned)std::min(148, w.row_blocks * w.chunks));
    cudaError_t e;
    if (a.epilogue == QGEMV_EPI_SWIGLU)
        e = w.sb_f16 ? launch_k(qgemv_tc_kernel<1, true>, grid, dim3(kTcgThreads), smem, s, p, stages)
                     : launch_k(qgemv_tc_kernel<1, false>, grid, dim3(kTcgThreads), smem, s, p, stages);
    else
        e = w.sb_f16 ? launch_k(qgemv_tc_kernel<0, true>, grid, dim3(kTcgThreads), smem, s, p, stages)
                     : launch_k(qgemv_tc_kernel<0, false>, grid, dim3(kTcgThreads), smem, s, p, stages);
    if (e != cudaSuccess) return cuda_fail(e, "qgemv_tc launch");
    return SWLM_OK;
}

}  // namespace swlm
