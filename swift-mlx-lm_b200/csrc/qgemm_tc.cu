// Q4 group-64 prefill GEMM for sm_100a on the 5th-generation tensor cores (tcgen05 / TMEM).
//
// Replaces the reference's `gemm_q4_g64` for M >= 64 (Generator/MetalSourceGenerator+Quantized.swift:88-156,
// which repeats the per-row dot product for every sequence position and so re-reads the weights M times)
// with a real contraction whose result equals the fp32-weight product up to the order of the fp32 sums. The weight
// is split as scale*q + zero = scale*(q - 8) + (zero + 8*scale): |q - 8| <= 8 has at most three significant bits (or
// is a power of two) and a bf16 or fp16 scale at most eleven, so scale*(q - 8) is EXACT in fp16 and is the A operand;
// the second term is constant over a group of 64 and multiplies the group's sum of activations, which becomes three
// extra K-columns per group appended after the real ones (c_hi x sum_hi, c_lo x sum_hi, c_hi x sum_lo, fp16 pairs
// that carry 22 bits). tcgen05.mma kind::f16 wants both operands in one format (fp16 weights against bf16 activations
// is an illegal instruction on this part), so a small kernel first copies the activations to fp16, every token row
// times a power of two that puts its largest magnitude at 2^14 (exact for every element within 2^-28 of the row's
// largest, immune to fp16's range, undone per token in the epilogue), and appends the per-group sums. (A dequantised
// weight rounded to 16 bits, the reference's dequantise-then-matmul route of +Quantized.swift:361-416, does not hold
// 1e-2 per output against `gemm_q4_g64`: bf16 weights leave outputs a tenth of the typical magnitude 1-5 % off,
// fp16 weights 1 %.)
//
// One CTA (18 warps) computes a 128 (weight rows) x BN (tokens) tile of Y^T:
//   * a TMA warp (one thread) keeps a ring of stages full, two cp.async.bulk.tensor.2d per 64-column group
//     (every CTA fetches its own copy): the packed weights of the group (128 rows x 32 bytes) and the activation tile (BN tokens
//     x 64 columns of fp16, 128-byte swizzle, rows past the last token filled with zeros); an mbarrier per
//     stage counts the bytes;
//   * 16 warps dequantise: four threads own one weight row, per group each reads 8 packed bytes from shared
//     memory, takes the row's (scale, zero) from registers (fetched eight groups at a time), turns nibble
//     pairs into fp16 with LOP3 (1024+q), subtracts 1032 and multiplies by the scale with one f16x2 instruction
//     each — scale*(q - 8), exact — and stores its 16 values into the row's lane of tensor memory
//     (tcgen05.st): the A operand of the MMA is read from TMEM, so the dequantised weights never cross shared
//     memory and four such tiles (32 columns each) fit beside the accumulator;
//   * an MMA warp (one thread) issues four tcgen05.mma (M=128, N=BN, K=16, kind::f16, A from TMEM, B through
//     a shared-memory descriptor, fp32 accumulator in TMEM) per group as soon as the group's weights and
//     activations are in place; tcgen05.commit signals an mbarrier when the stage and the weight tile may
//     be overwritten;
//   * the epilogue reads the accumulator with tcgen05.ld, rounds to bf16 and stores Y[token][row].
// Every mbarrier wait is bounded: on expiry an error word is set, the CTA stops issuing, waits (bounded) for
// the copies it has in flight, frees its TMEM and returns.
#include <cstdlib>
#include <cuda.h>
#include "swlm_internal.h"

namespace swlm {
namespace {

constexpr int kTcThreads = 512;          // dequantising threads
constexpr int kTcAllThreads = kTcThreads + 64;  // + the MMA warp and the activation (TMA) warp
constexpr int kTcRows = 128;            // weight rows per CTA = UMMA M
constexpr int kTcBK = 64;               // one quantisation group per pipeline stage
constexpr int kTcSpinLimit = 1 << 22;

struct QGemmTcParams {
    const uint32_t* w;        // [n][k/8] MLX words
    const uint16_t* scales;   // [n][k/64] bf16
    const uint16_t* biases;
    int n, k;
    const __half* x;          // [m][x_stride]: the activations as fp16, every token row scaled by a power of two
    const float* rscale;      // [m]: the inverse of each row's scale
    int x_stride, m;
    int ext_steps;            // 64-column steps of appended group-sum columns (three planes of ceil(k/64/64) steps)
    TcSegments out;           // weight rows [end[q-1], end[q]) go to out.y[q][token][row - end[q-1]]
    int* status;              // set non-zero when a bounded wait expired
    // launches of at most 64 token rows over few weight rows: K is cut into gridDim.z ranges of `split_steps` groups
    // (a multiple of 8) so that more SMs take part; every range writes its fp32 sums to part[z][m][n] and a second
    // launch adds the ranges in order. The last range also takes the appended group-sum steps.
    float* part;
    int split_steps;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// Bounded wait on phase parity; returns false when the limit was reached. The loop is two instructions per
// attempt (try_wait suspends the warp for a while by itself): waiting warps share their scheduler with warps
// that still dequantise.
__device__ __forceinline__ bool mbar_wait_addr(unsigned addr, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .u32 n;\n\t"
        "mov.u32 n, 0;\n\t"
        "SWLM_TRY:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "@p bra SWLM_DONE;\n\t"
        "add.u32 n, n, 1;\n\t"
        "setp.lt.u32 q, n, %3;\n\t"
        "@q bra SWLM_TRY;\n\t"
        "SWLM_DONE:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done) : "r"(addr), "r"(parity), "r"((unsigned)kTcSpinLimit) : "memory");
    return done != 0;
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) { return mbar_wait_addr(smem_u32(bar), parity); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024
// bytes apart (stride byte offset); leading byte offset unused for this layout; descriptor version 1.
__device__ __forceinline__ unsigned long long umma_desc(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)(1024u >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Instruction descriptor for kind::f16: D = fp32, A = B = fp16 (format 0), both K-major, M = 128, N = BN.
__host__ __device__ constexpr unsigned umma_idesc(int bn) {
    return (1u << 4) | (0u << 7) | (0u << 10) | ((unsigned)(bn >> 3) << 17) | ((unsigned)(kTcRows >> 4) << 24);
}

// D[tmem] (+)= A[tmem] x B[shared memory]: the A operand (128 rows x 16 bf16 = 8 columns of 32 bits) is read from
// tensor memory, where the dequantising threads put it, so it never crosses shared memory
__device__ __forceinline__ void umma_f16_ta(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// One result, rounded once to bf16, to the output its weight row belongs to.
__device__ __forceinline__ void tc_store(const TcSegments& o, int token, int row, float val) {
    const int q = row < o.end[0] ? 0 : row < o.end[1] ? 1 : 2;
    const int first = q == 0 ? 0 : o.end[q - 1];
    o.y[q][(size_t)token * o.stride[q] + (row - first)] = __float2bfloat16_rn(val);
}

// F16SB: scale and zero are fp16 (tensors uploaded as STAF blocks) instead of bf16 (MLX tensors).
//
// Dequantising thread (warp w, lane l): weight row 32 (w & 3) + l (= its TMEM lane), columns 16 (w >> 2) ..
// + 15 of every group. ready_bar[kt % SA] collects the 512 arrivals of group kt; full_bar[kt % SB] completes
// when the group's stage has landed; empty_bar[kt % SB] when its MMAs are done. With SA = 2 the dequantisation
// of group kt had to wait for the MMAs of group kt - 2 (measured: 200 clocks per group); SA = 4 removes that.
template <int BN, int STAGES, bool F16SB>
__global__ void __launch_bounds__(kTcAllThreads) qgemm_tc_kernel(const QGemmTcParams p, const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap) {
    constexpr int SA = BN == 64 ? 2 : 4, SB = STAGES;   // dequantised weight tiles in flight
    constexpr unsigned kTmemCols = BN == 256 ? 512 : BN == 128 ? 256 : 128;   // accumulator (BN) + SA weight tiles of 32, power of two
    constexpr unsigned kACol0 = BN;                                            // first column of the weight tiles
    static_assert(SB >= 3, "the activation ring must be deeper than the weight ring");
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment for the swizzle atoms
    unsigned char* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
    constexpr int B_BYTES = BN * 128;
    constexpr int W_BYTES = kTcRows * 32;        // packed weights of one group
    constexpr int STAGE_BYTES = B_BYTES + W_BYTES;
    __shared__ __align__(8) unsigned long long empty_bar[STAGES];
    __shared__ __align__(8) unsigned long long full_bar[STAGES];    // the activation tile of a stage has landed
    __shared__ __align__(8) unsigned long long ready_bar[4];   // a weight tile and its activation tile are in place
    __shared__ __align__(8) unsigned long long done_bar;
    __shared__ unsigned tmem_base_smem;
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = (warp & 3) * 32 + lane, part = (warp >> 2) & 3;   // TMEM lane = weight row; part: which 16 of the group's 64 columns
    const int row0 = blockIdx.x * kTcRows, tok0 = blockIdx.y * BN;
    const int kt_total = p.k / kTcBK;
    // this CTA's range of groups [kt_lo, kt_lo + real_steps) and, for the last range, the appended group-sum columns
    const int kt_lo = gridDim.z > 1 ? (int)blockIdx.z * p.split_steps : 0;
    const int real_steps = gridDim.z > 1 ? min(p.split_steps, kt_total - kt_lo) : kt_total;
    const int ext_steps = blockIdx.z == gridDim.z - 1 ? p.ext_steps : 0;
    const int steps_total = real_steps + ext_steps;
    unsigned char* const b_ring = smem;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) { mbar_init(&empty_bar[s], 1); mbar_init(&full_bar[s], 1); }
        for (int i = 0; i < 4; ++i) mbar_init(&ready_bar[i], kTcThreads);
        mbar_init(&done_bar, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();  // the allocation is a warp-wide instruction: re-converge after the single-thread block
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_smem)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_d = tmem_base_smem;

    const int row = row0 + r;
    const bool row_ok = row < p.n;
    const uint16_t* srow = p.scales + (size_t)(row_ok ? row : 0) * kt_total;
    const uint16_t* zrow = p.biases + (size_t)(row_ok ? row : 0) * kt_total;
    constexpr unsigned idesc = umma_idesc(BN);

    // scales and zeros of groups kt0..kt0+7 of this thread's row (16-bit each), one 16-byte load each when the
    // rows are 16-byte aligned; they do not depend on the preceding kernel
    const bool sz_vec = (kt_total & 7) == 0;
    auto load8 = [&](const uint16_t* rowp, int kt0) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (!row_ok || kt0 >= kt_total) return v;
        if (sz_vec) return __ldg(reinterpret_cast<const uint4*>(rowp + kt0));
        unsigned h[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = kt0 + j < kt_total ? (unsigned)__ldg(rowp + kt0 + j) : 0u;
        return make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
    };
    auto pick16 = [](const uint4& v, int j) {  // 16-bit element j (0..7)
        const unsigned lo = (j & 2) ? v.y : v.x, hi = (j & 2) ? v.w : v.z;
        const unsigned w = (j & 4) ? hi : lo;
        return (j & 1) ? w >> 16 : w & 0xFFFFu;
    };
    if (warp == kTcThreads / 32) {
        // ---- MMA warp: one thread issues the four MMAs of a group as soon as its tiles are in place; the
        // dequantising warps are already busy with the next group by then -----------------------------------
        if (lane == 0) {
            for (int kt = 0; kt < steps_total; ++kt) {
                if (!mbar_wait(&ready_bar[kt % SA], (unsigned)((kt / SA) & 1)) || !mbar_wait(&full_bar[kt % SB], (unsigned)((kt / SB) & 1))) {
                    // giving up: let done_bar complete behind the MMAs already issued, so that tensor memory is not
                    // freed under them
                    atomicExch(p.status, 2); failed = 1; umma_commit(&done_bar); break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned a_addr = tmem_d + kACol0 + (unsigned)(kt % SA) * 32u, b_addr = smem_u32(b_ring + (kt % SB) * STAGE_BYTES);
#pragma unroll
                for (int j = 0; j < kTcBK / 16; ++j)  // 16 bf16 = 8 columns of A, 32 bytes along K inside B's 128-byte row
                    umma_f16_ta(tmem_d, a_addr + 8u * j, umma_desc(b_addr + 32 * j), idesc, (kt > 0 || j > 0) ? 1u : 0u);
                umma_commit(&empty_bar[kt % SB]);
                if (kt == steps_total - 1) umma_commit(&done_bar);
            }
        }
        __syncwarp();
    } else if (warp == kTcThreads / 32 + 1) {
        // ---- activation warp: one thread keeps the ring of activation tiles full ----------------------------
        if (lane == 0) {
            pdl_wait();                         // the activations may come from the kernel just before this one
            int issued = 0;
            for (int kt = 0; kt < steps_total; ++kt) {
                const int s = kt % SB;
                // the MMAs that read this stage SB groups ago are done
                if (kt >= SB && !mbar_wait(&empty_bar[s], (unsigned)((kt / SB - 1) & 1))) { atomicExch(p.status, 3); failed = 1; break; }
                if (failed) break;
                const unsigned bar = smem_u32(&full_bar[s]);
                const bool real = kt < real_steps;   // an appended step has activations (the group sums) but no packed weights
                const int kg = real ? kt_lo + kt : kt_total + (kt - real_steps);   // 64-column step within the activation rows
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((unsigned)(real ? STAGE_BYTES : B_BYTES)) : "memory");
                if (real)
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                 ::"r"(smem_u32(b_ring + s * STAGE_BYTES + B_BYTES)), "l"(reinterpret_cast<unsigned long long>(&wmap)), "r"(kg * 32), "r"(row0), "r"(bar) : "memory");
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                             ::"r"(smem_u32(b_ring + s * STAGE_BYTES)), "l"(reinterpret_cast<unsigned long long>(&xmap)), "r"(kg * kTcBK), "r"(tok0), "r"(bar) : "memory");
                issued = kt + 1;
            }
            if (failed) {
                // stopping early: the copies already requested still write shared memory; wait for them (bounded)
                for (int kt = issued > SB ? issued - SB : 0; kt < issued; ++kt) mbar_wait(&full_bar[kt % SB], (unsigned)((kt / SB) & 1));
            }
        }
        __syncwarp();
    } else {
    uint4 s_cur = load8(srow, kt_lo), z_cur = load8(zrow, kt_lo), s_nxt = load8(srow, kt_lo + 8), z_nxt = load8(zrow, kt_lo + 8);

    // ring bookkeeping without divisions: stage and parity of this group's activations/packed weights, and of
    // the group SA back whose MMAs free this group's weight tile
    int fs = 0, es = 0, as = 0;
    unsigned fpar = 0, epar = 0;
    const unsigned char* const w_src = b_ring + B_BYTES + r * 32 + part * 8;
    const unsigned a_dst = tmem_d + ((unsigned)((warp & 3) * 32) << 16) + kACol0 + (unsigned)part * 8u;
    const unsigned full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]), ready0 = smem_u32(&ready_bar[0]);
    // one group; j = kt & 7 is a compile-time constant in the unrolled loop below, so picking the group's scale and
    // zero out of the 16-byte vectors costs one instruction each
    auto group = [&](int kt, int j) {
        // ---- the MMAs of group kt - SA are done: its weight tile (this group's) may be overwritten -----------
        if (kt >= SA) {
            if (!mbar_wait_addr(empty0 + 8u * es, epar)) { atomicExch(p.status, 1); failed = 1; }
            if (++es == SB) { es = 0; epar ^= 1u; }
        }
        // ---- this group's packed weights have landed (with its activations) ---------------------------------
        if (!mbar_wait_addr(full0 + 8u * fs, fpar)) { atomicExch(p.status, 1); failed = 1; }
        // ---- weights: 16 nibbles of this thread's row -> 16 bf16 = bf16(scale * q + zero) -----------------
        const uint2 wq = *reinterpret_cast<const uint2*>(w_src + fs * STAGE_BYTES);
        if (++fs == SB) { fs = 0; fpar ^= 1u; }
        const unsigned vs = pick16(s_cur, j), vz = pick16(z_cur, j);
        // the scale as an fp16 pair: STAF tensors carry fp16 already; a bf16 (MLX) scale converts exactly (8 mantissa
        // bits into 11) unless it lies below fp16's normal range, where the weights it scales are nil anyway
        const __half s16 = F16SB ? __ushort_as_half((unsigned short)vs) : __float2half_rn(__uint_as_float(vs << 16));
        const __half2 sc = __half2half2(s16);
        (void)vz;
        const unsigned c1032 = 0x64086408u;   // fp16 1032 = 1024 + 8
        const __half2 off = *reinterpret_cast<const __half2*>(&c1032);
        const unsigned words[2] = {wq.x, wq.y};
        unsigned a_regs[8];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            // a word holds 8 consecutive columns, nibble i = column i; pairs (i, i+4) come out of one LOP3
            const unsigned wv = words[c];
            unsigned o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const unsigned pr = ((wv >> (4 * i)) & 0x000F000Fu) | 0x64006400u;         // fp16 (1024+q_i, 1024+q_{i+4})
                __half2 q2 = __hsub2(*reinterpret_cast<const __half2*>(&pr), off);        // (q_i - 8, q_{i+4} - 8), exact
                q2 = __hmul2(q2, sc);                                                      // scale * (q - 8): exact in fp16
                o[i] = *reinterpret_cast<const unsigned*>(&q2);                            // lo = column i, hi = column i+4
            }
            // reorder the pairs (i, i+4) into consecutive columns 0..7
            a_regs[4 * c + 0] = __byte_perm(o[0], o[1], 0x5410); a_regs[4 * c + 1] = __byte_perm(o[2], o[3], 0x5410);
            a_regs[4 * c + 2] = __byte_perm(o[0], o[1], 0x7632); a_regs[4 * c + 3] = __byte_perm(o[2], o[3], 0x7632);
        }
        // 16 bf16 of this row -> 8 columns of the row's TMEM lane (a warp owns the 32 lanes of its quarter)
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                     ::"r"(a_dst + (unsigned)as * 32u), "r"(a_regs[0]), "r"(a_regs[1]), "r"(a_regs[2]), "r"(a_regs[3]), "r"(a_regs[4]), "r"(a_regs[5]), "r"(a_regs[6]), "r"(a_regs[7]) : "memory");
        // the stores to tensor memory are complete and ordered before the MMA warp's reads, then tell the MMA warp
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ready0 + 8u * as) : "memory");
        if (++as == SA) as = 0;
    };
    // (group indices are local to this CTA's range: they only drive the rings; the scales come from kt_lo on)
    for (int kt0 = 0; kt0 < real_steps && !failed; kt0 += 8) {
        if (kt0 > 0) { s_cur = s_nxt; z_cur = z_nxt; s_nxt = load8(srow, kt_lo + kt0 + 8); z_nxt = load8(zrow, kt_lo + kt0 + 8); }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (kt0 + j < real_steps) group(kt0 + j, j);
    }
    // ---- appended steps: the A operand is the groups' constant term c = 64 (zero + 8 scale) as an fp16 pair (hi, lo);
    // plane 0 carries c_hi (against sum_hi), plane 1 c_lo (against sum_hi), plane 2 c_hi (against sum_lo); the
    // activation side holds sum / 64 so that neither factor leaves fp16's range -----------------------------------
    const int plane_steps = p.ext_steps / 3;
    for (int e = 0; e < ext_steps && !failed; ++e) {
        const int kt = real_steps + e;
        if (kt >= SA) {
            if (!mbar_wait_addr(empty0 + 8u * es, epar)) { atomicExch(p.status, 1); failed = 1; }
            if (++es == SB) { es = 0; epar ^= 1u; }
        }
        if (!mbar_wait_addr(full0 + 8u * fs, fpar)) { atomicExch(p.status, 1); failed = 1; }
        if (++fs == SB) { fs = 0; fpar ^= 1u; }
        const int plane = e / plane_steps, g0 = (e - plane * plane_steps) * 64 + part * 16;
        unsigned a_regs[8];
#pragma unroll
        for (int h8 = 0; h8 < 2; ++h8) {
            const uint4 sv = load8(srow, g0 + 8 * h8), zv = load8(zrow, g0 + 8 * h8);   // zero beyond the last group
            float c[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const unsigned bs = pick16(sv, i), bz = pick16(zv, i);
                const float sf = F16SB ? __half2float(__ushort_as_half((unsigned short)bs)) : __uint_as_float(bs << 16);
                const float zf = F16SB ? __half2float(__ushort_as_half((unsigned short)bz)) : __uint_as_float(bz << 16);
                const float cf = 64.0f * fmaf(8.0f, sf, zf);
                const float hi = __half2float(__float2half_rn(cf));
                c[i] = plane == 1 ? cf - hi : hi;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __half2 pr = __floats2half2_rn(c[2 * i], c[2 * i + 1]);
                a_regs[4 * h8 + i] = *reinterpret_cast<const unsigned*>(&pr);
            }
        }
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                     ::"r"(a_dst + (unsigned)as * 32u), "r"(a_regs[0]), "r"(a_regs[1]), "r"(a_regs[2]), "r"(a_regs[3]), "r"(a_regs[4]), "r"(a_regs[5]), "r"(a_regs[6]), "r"(a_regs[7]) : "memory");
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ready0 + 8u * as) : "memory");
        if (++as == SA) as = 0;
    }
    }  // dequantising warps

    // ---- epilogue: TMEM -> registers -> bf16 -> Y[token][row] --------------------------------------------
    // a warp reads the 32 accumulator lanes of its quarter (warp & 3); warps 4i..4i+3 take the i-th quarter of
    // the token columns
    bool ok = !failed && warp < kTcThreads / 32;
    if (ok && !mbar_wait(&done_bar, 0u)) { atomicExch(p.status, 1); ok = false; }
    if (failed && tid == 0) mbar_wait(&done_bar, 0u);   // (bounded) the MMAs issued before the failure have drained
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
        const int erow = row0 + (warp & 3) * 32 + lane;
        const int cbase = (warp >> 2) * (BN / 4);
#pragma unroll 1
        for (int c0 = cbase; c0 < cbase + BN / 4; c0 += 16) {
            if (tok0 + c0 >= p.m) break;  // uniform across the warp
            unsigned v[16];
            const unsigned taddr = tmem_d + ((unsigned)((warp & 3) * 32) << 16) + (unsigned)c0;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                  "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                : "r"(taddr) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (erow < p.n) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int tkn = tok0 + c0 + i;
                    // undo the token row's power-of-two scaling (exact), round once to bf16 (or leave this K range's
                    // sum for the launch that adds the ranges up)
                    if (tkn < p.m) {
                        const float val = __uint_as_float(v[i]) * __ldg(p.rscale + tkn);
                        if (gridDim.z > 1) p.part[((size_t)blockIdx.z * p.m + tkn) * p.n + erow] = val;
                        else tc_store(p.out, tkn, erow, val);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kTmemCols) : "memory");
}

// Y[t][n] = bf16(sum over the K ranges, in order) for a launch whose K was cut in `splits` ranges.
__global__ void __launch_bounds__(256) tc_sum_splits_kernel(const float* part, int splits, int m, int n, const TcSegments out) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)m * n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int z = 0; z < splits; ++z) acc += __ldcg(part + (size_t)z * total + i);
        const int t = (int)(i / n), r = (int)(i - (size_t)t * n);
        tc_store(out, t, r, acc);
    }
}

// Activations bf16 -> fp16, one CTA per token row: the row's largest magnitude goes to [2^14, 2^15), so that nothing
// overflows fp16 and every element within 2^-28 of the largest converts exactly (bf16 carries 8 significant bits,
// fp16 11). rscale[row] = the inverse factor, applied to the accumulators in the product's epilogue. Behind the k
// converted values the row gets three planes of g_pad columns: sum / 64 of every group of 64 converted values as an
// fp16 pair, laid out (hi, hi, lo) to meet the (c_hi, c_lo, c_hi) planes of the weight side; columns past the last
// group are zero.
__global__ void __launch_bounds__(256) x_to_f16_kernel(const __nv_bfloat16* x, int x_stride, int k, int g_pad, __half* xh, int xh_stride, float* rscale) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ unsigned red[8];
    const int row = blockIdx.x, tid = threadIdx.x;
    const unsigned* src = reinterpret_cast<const unsigned*>(x + (size_t)row * x_stride);
    unsigned mx = 0;
    for (int i = tid; i < k / 2; i += 256) {
        const unsigned w = src[i];
        mx = max(mx, max(w & 0x7FFFu, (w >> 16) & 0x7FFFu));   // bf16 magnitudes order like their bit patterns
    }
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = 0;
    for (int i = 0; i < 8; ++i) mx = max(mx, red[i]);
    const int e = (int)(mx >> 7);                                   // biased exponent of the largest magnitude
    const int sh = (e == 0 || e == 255) ? 0 : max(-100, min(100, 141 - e));
    const float mul = __uint_as_float((unsigned)(127 + sh) << 23);  // 2^sh
    __half* out = xh + (size_t)row * xh_stride;
    // a warp converts one group of 64 at a time (one 32-bit word of two values per lane) and sums it
    const int lane = tid & 31, warp = tid >> 5, groups = k / 64;
    for (int g = warp; g < g_pad; g += 8) {
        float sum = 0.f;
        if (g < groups) {
            const unsigned w = src[g * 32 + lane];
            const __half2 h = __floats2half2_rn(__uint_as_float(w << 16) * mul, __uint_as_float(w & 0xFFFF0000u) * mul);
            reinterpret_cast<unsigned*>(out)[g * 32 + lane] = *reinterpret_cast<const unsigned*>(&h);
            const float2 f = __half22float2(h);
            sum = f.x + f.y;
        }
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) {
            const float sc = sum * 0.015625f;
            const __half hi = __float2half_rn(sc), lo = __float2half_rn(sc - __half2float(hi));
            out[k + g] = hi; out[k + g_pad + g] = hi; out[k + 2 * g_pad + g] = lo;
        }
    }
    if (tid == 0) rscale[row] = __uint_as_float((unsigned)(127 - sh) << 23);
}

template <int BN, int STAGES>
constexpr size_t tc_smem_bytes() { return (size_t)STAGES * (BN * 128 + kTcRows * 32) + 1024; }

// cuTensorMapEncodeTiled, looked up through the runtime so that the library does not link against the driver
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                      const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TensorMapEncodeFn tensor_map_encode_fn() {
    static TensorMapEncodeFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
        return reinterpret_cast<TensorMapEncodeFn>(f);
    }();
    return fn;
}

// fp16 activations X[m][x_stride] as a 2-D tensor (k innermost); box = 64 columns x bn tokens, 128-byte swizzle
int make_x_map(const __half* x, int x_stride, int m, int k, int bn, CUtensorMap* map) {
    TensorMapEncodeFn fn = tensor_map_encode_fn();
    if (!fn) { set_error("qgemm (tcgen05): cuTensorMapEncodeTiled is not available"); return SWLM_ERR_CUDA; }
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)m};
    const cuuint64_t strides[1] = {(cuuint64_t)x_stride * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTcBK, (cuuint32_t)bn};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(x), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("qgemm (tcgen05): cuTensorMapEncodeTiled failed (%d)", (int)r); return SWLM_ERR_CUDA; }
    return SWLM_OK;
}

template <int BN, int STAGES>
int tc_init_one() {
    SWLM_CUDA(cudaFuncSetAttribute(qgemm_tc_kernel<BN, STAGES, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem_bytes<BN, STAGES>()));
    SWLM_CUDA(cudaFuncSetAttribute(qgemm_tc_kernel<BN, STAGES, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem_bytes<BN, STAGES>()));
    return SWLM_OK;
}
// packed weights W[n][k/2 bytes] as a 2-D byte tensor; box = 32 bytes (one group) x 128 rows, no swizzle
int make_w_map(const uint32_t* w, int n, int k, CUtensorMap* map) {
    TensorMapEncodeFn fn = tensor_map_encode_fn();
    if (!fn) { set_error("qgemm (tcgen05): cuTensorMapEncodeTiled is not available"); return SWLM_ERR_CUDA; }
    const cuuint64_t dims[2] = {(cuuint64_t)k / 2, (cuuint64_t)n};
    const cuuint64_t strides[1] = {(cuuint64_t)k / 2};
    const cuuint32_t box[2] = {32, (cuuint32_t)kTcRows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint32_t*>(w), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("qgemm (tcgen05): cuTensorMapEncodeTiled failed for the weights (%d)", (int)r); return SWLM_ERR_CUDA; }
    return SWLM_OK;
}

template <int BN, int STAGES>
int tc_launch_one(const QGemmTcParams& p, bool f16, cudaStream_t s) {
    CUtensorMap xmap, wmap;
    int rc = make_x_map(p.x, p.x_stride, p.m, p.x_stride, BN, &xmap);   // the appended columns are part of the tensor
    if (rc) return rc;
    if ((rc = make_w_map(p.w, p.n, p.k, &wmap))) return rc;
    const int splits = p.split_steps > 0 ? (p.k / kTcBK + p.split_steps - 1) / p.split_steps : 1;
    const dim3 grid((unsigned)((p.n + kTcRows - 1) / kTcRows), (unsigned)((p.m + BN - 1) / BN), (unsigned)splits);
    const cudaError_t e = f16 ? launch_k(qgemm_tc_kernel<BN, STAGES, true>, grid, dim3(kTcAllThreads), tc_smem_bytes<BN, STAGES>(), s, p, xmap, wmap)
                              : launch_k(qgemm_tc_kernel<BN, STAGES, false>, grid, dim3(kTcAllThreads), tc_smem_bytes<BN, STAGES>(), s, p, xmap, wmap);
    if (e != cudaSuccess) return cuda_fail(e, "qgemm_tc launch");
    if (splits > 1) {
        const size_t total = (size_t)p.m * p.n;
        const cudaError_t e2 = launch_k(tc_sum_splits_kernel, dim3((unsigned)std::min<size_t>(296, (total + 1023) / 1024)), dim3(256), 0, s,
                                        (const float*)p.part, splits, p.m, p.n, p.out);
        if (e2 != cudaSuccess) return cuda_fail(e2, "qgemm_tc split sum launch");
    }
    return SWLM_OK;
}

// K ranges for a launch of at most 64 token rows: as many as keep all CTAs resident at once (two per SM for the
// 64-token tile: 576 threads x 42 registers, 74 KB of shared memory, 128 columns of tensor memory each), each a whole
// number of 8-group blocks (the scale/zero vectors are read 8 groups at a time) and all of equal length. 0 = no split.
constexpr int kTcSplitMaxRows = 64;
constexpr int kTcSplitMaxCtas = 296;
constexpr size_t kTcSplitBytes = (size_t)kTcSplitMaxRows * kTcSplitMaxCtas * kTcRows * 4;   // fp32 partial sums of all CTAs
int tc_pick_split_steps(int m, int n, int k) {
    static const bool off = [] { const char* v = getenv("SWLM_TC_KSPLIT"); return v && v[0] == '0'; }();
    if (off || m > kTcSplitMaxRows) return 0;
    static const int cap = [] { const char* v = getenv("SWLM_TC_KSPLIT_CTAS"); const int c = v ? atoi(v) : 0; return c >= 1 && c <= kTcSplitMaxCtas ? c : kTcSplitMaxCtas; }();
    const int n_tiles = (n + kTcRows - 1) / kTcRows, kt_total = k / kTcBK;
    int best = 0;
    for (int per = kt_total - 8; per >= 8; per -= 8) {
        if (kt_total % per) continue;
        if (n_tiles * (kt_total / per) > cap) break;
        best = per;
    }
    return best;
}

}  // namespace

int qgemm_tc_init() {
    int rc;
    if ((rc = tc_init_one<64, 6>())) return rc;
    if ((rc = tc_init_one<128, 6>())) return rc;
    if ((rc = tc_init_one<256, 6>())) return rc;
    return SWLM_OK;
}

// Y[m][n] = bf16(X[m][k] . fp16(W)^T) on the tcgen05 path. xh (m * k fp16 values) and rscale (m floats) are scratch
// for the fp16 copy of the activations. `status` is a device word the kernel sets when a
// bounded wait expires. Token tile: 256 when there are that many tokens (each dequantised weight then feeds
// 256 columns of the MMA), else 128 or 64.
// columns of one plane of appended group sums: the groups of a row, padded to whole 64-column steps
static int ext_plane_cols(int k) { return (k / 64 + 63) / 64 * 64; }
// [partial sums of a K-split launch][fp16 activations + group sums][one float per token row]
size_t qgemm_tc_scratch_bytes(int m, int k) { return kTcSplitBytes + ((size_t)m * (k + 3 * ext_plane_cols(k)) * 2 + 255) / 256 * 256 + (size_t)m * 4; }

int qgemm_tc_launch_count(const Q4Raw& w, int m, bool reuse_x) {
    return (reuse_x ? 0 : 1) + 1 + (tc_pick_split_steps(m, w.n, w.k) > 0 ? 1 : 0);
}

int launch_qgemm_tc(const Q4Raw& w, int m, const __nv_bfloat16* x, int x_stride, __nv_bfloat16* y, int y_stride,
                    void* scratch, int* status, cudaStream_t s, bool reuse_x, const TcSegments* segments) {
    float* part = static_cast<float*>(scratch);
    __half* xh = scratch ? reinterpret_cast<__half*>(static_cast<unsigned char*>(scratch) + kTcSplitBytes) : nullptr;
    const int g_pad = ext_plane_cols(w.k), xh_stride = w.k + 3 * g_pad;
    float* rscale = scratch ? reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + kTcSplitBytes + ((size_t)m * xh_stride * 2 + 255) / 256 * 256) : nullptr;
    if (w.k % kTcBK || (x_stride & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(xh) & 15) || !xh || !rscale) {
        set_error("qgemm (tcgen05): bad shape, alignment or scratch");
        return SWLM_ERR_INVALID;
    }
    // xh: m rows of w.k fp16 values followed by three planes of g_pad group sums
    // (reuse_x: the scratch still holds the copy of these very rows, made for the product before this one)
    if (!reuse_x) {
        cudaError_t e = launch_k(x_to_f16_kernel, dim3((unsigned)m), dim3(256), 0, s, x, x_stride, w.k, g_pad, xh, xh_stride, rscale);
        if (e != cudaSuccess) return cuda_fail(e, "x_to_f16 launch");
    }
    QGemmTcParams p{};
    p.w = w.w; p.scales = w.scales; p.biases = w.biases; p.n = w.n; p.k = w.k;
    p.x = xh; p.rscale = rscale; p.x_stride = xh_stride; p.m = m; p.status = status;
    if (segments) {
        p.out = *segments;
        if (p.out.count < 1 || p.out.count > 3 || p.out.end[p.out.count - 1] != w.n) { set_error("qgemm (tcgen05): output segments do not cover the %d weight rows", w.n); return SWLM_ERR_INVALID; }
        for (int q = p.out.count; q < 3; ++q) p.out.end[q] = p.out.end[p.out.count - 1];   // never selected
    } else {
        p.out.count = 1; p.out.y[0] = y; p.out.stride[0] = y_stride; p.out.end[0] = p.out.end[1] = p.out.end[2] = w.n;
    }
    p.ext_steps = 3 * g_pad / 64;
    p.part = part;
    p.split_steps = tc_pick_split_steps(m, w.n, w.k);
    int rc;
    int bn = m > 128 ? 256 : m > 64 ? 128 : 64;
    static const int forced_bn = [] { const char* v = getenv("SWLM_TC_BN"); return v ? atoi(v) : 0; }();
    if (forced_bn == 64 || forced_bn == 128 || forced_bn == 256) bn = forced_bn;
    if (bn == 256) rc = tc_launch_one<256, 6>(p, w.sb_f16, s);
    else if (bn == 128) rc = tc_launch_one<128, 6>(p, w.sb_f16, s);
    else rc = tc_launch_one<64, 6>(p, w.sb_f16, s);
    return rc;
}

}  // namespace swlm
