// Device side of the tensor-parallel exchange: a one-shot push all-reduce fused into the row-parallel
// product that produces the partial sums and the product that consumes them.
//
// The reference has no multi-device code; this is the sm_100a design for "one all-reduce per attention
// and MLP block". Every rank owns one exchange buffer, mapped into every other rank's address space
// (cudaIpc handles). The producing kernel stores its fp32 partial row straight into every rank's
// buffer over NVLink (plain peer stores: the data lands in the consumer's own memory). Every element
// travels as one 64-bit scalar store {value, number of the exchange}: a reader that sees the number sees the
// value (single-copy atomicity of an aligned 64-bit access), so the exchange needs no fence, no completion count and no separate flag, and its latency is
// one NVLink store. The consuming kernel polls the elements it needs in its own memory, adds the partials
// in rank order (the same order on every rank, so all ranks continue with bit-identical activations) and
// goes on with the residual add and the norm. Two parities of buffers suffice: a rank can only be one
// exchange ahead of the slowest rank. Every wait is bounded; on expiry an error word is set and the
// kernel carries on with whatever it has, so a missing rank surfaces as a status, not as a hung GPU.
// (The arg-max exchange of a vocabulary-sharded head, once per token, still uses a flag per source.)
#pragma once

#include <cstddef>
#include <cstdint>

namespace swlm {

constexpr int kTpMax = 8;

struct TpLayout {
    int tp, batch, hidden;
    int rows = 0;  // prompt chunks: token rows one exchange can carry (0: none)
    __host__ __device__ size_t flags_am(int par, int src) const { return 64 + ((size_t)par * kTpMax + src) * 4; }
    __host__ __device__ size_t flags_rows(int par, int src) const { return 128 + ((size_t)par * kTpMax + src) * 4; }
    // partial sums: 8 bytes per element {fp32 bits, exchange number}
    __host__ __device__ size_t recv_ar(int par, int src, int b) const { return 256 + ((((size_t)par * tp + src) * batch + b) * hidden) * 8; }
    __host__ __device__ size_t recv_am(int par, int src, int b) const { return 256 + (size_t)2 * tp * batch * hidden * 8 + (((size_t)par * tp + src) * batch + b) * 8; }
    __host__ __device__ size_t decode_total() const { return (256 + (size_t)2 * tp * batch * hidden * 8 + (size_t)2 * tp * batch * 8 + 255) / 256 * 256; }
    // prompt chunks: bf16 partial rows [rows][hidden] per source, two parities, completion signalled by flags_rows
    __host__ __device__ size_t recv_rows(int par, int src) const { return decode_total() + ((size_t)par * tp + src) * rows * hidden * 2; }
    __host__ __device__ size_t total() const { return decode_total() + (size_t)2 * tp * rows * hidden * 2; }
};

// What a kernel needs to take part in an exchange. tp == 1: unused.
struct TpParams {
    int tp, rank;
    TpLayout lay;
    unsigned char* peer[kTpMax];  // exchange buffers of all ranks; peer[rank] is this rank's own
    int* epoch;                   // local: number of all-reduces completed so far
    unsigned* done;               // local: row tiles of the current product already pushed (the last one advances epoch)
    int* status;                  // local: set to non-zero when a bounded wait expired
    int* host_status;             // the same news for the host: a word in mapped pinned memory, read after a sync (may be null)
};

#ifdef __CUDACC__
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

constexpr int kTpSpinLimit = 1 << 21;  // polls of ~128 ns each: about a quarter of a second

// A bounded wait gave up: say so on the device (later exchanges then stop waiting) and to the host.
__device__ __forceinline__ void tp_wait_expired(const TpParams& tp) {
    atomicExch(tp.status, 1);
    if (tp.host_status) *reinterpret_cast<volatile int*>(tp.host_status) = 21;
}

// Wait (bounded) until every source has raised flag `epoch` on this rank. One lane per source.
__device__ __forceinline__ void tp_wait_flags(const TpParams& tp, const unsigned char* own, size_t flag_off0, int epoch, int lane_src) {
    if (lane_src < tp.tp) {
        const unsigned* f = reinterpret_cast<const unsigned*>(own + flag_off0 + (size_t)lane_src * 4);
        int spins = 0;
        while ((int)ld_acquire_sys(f) < epoch) {
            if (++spins > kTpSpinLimit) { tp_wait_expired(tp); break; }
            __nanosleep(128);
        }
    }
}

// One element of a partial-sum buffer: value in the low half, number of the exchange in the high half of ONE naturally
// aligned 64-bit scalar, written with one 64-bit store. PTX guarantees single-copy atomicity for such an access (a
// vector store would count as two independent 32-bit accesses), so a reader can never see the number without the value.
__device__ __forceinline__ void tp_store_tagged(unsigned char* dst, float v, int epoch) {
    const unsigned long long packed = ((unsigned long long)(unsigned)epoch << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(packed) : "memory");
}

// 2 * N2 consecutive elements of a partial-sum buffer in this rank's own memory: one attempt, ... (the elements are
// read as 64-bit scalars, two per instruction: each element is atomic on its own, which is all the protocol needs)
template <int N2>
__device__ __forceinline__ void tp_load_tagged(const unsigned char* src, uint4 (&v)[N2]) {
#pragma unroll
    for (int i = 0; i < N2; ++i) {
        unsigned long long a, b;
        asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(src + 16 * i) : "memory");
        v[i].x = (unsigned)a; v[i].y = (unsigned)(a >> 32); v[i].z = (unsigned)b; v[i].w = (unsigned)(b >> 32);
    }
}
// ... the check that all of them carry the number of this exchange, ...
template <int N2>
__device__ __forceinline__ bool tp_all_tagged(const uint4 (&v)[N2], int epoch) {
    bool ok = true;
#pragma unroll
    for (int i = 0; i < N2; ++i) ok = ok && v[i].y == (unsigned)epoch && v[i].w == (unsigned)epoch;
    return ok;
}
// ... and the bounded polling for those that did not on the first attempt. After a wait has expired once, later
// exchanges do not wait again: the status word says so.
template <int N2>
__device__ __forceinline__ void tp_poll_tagged(const TpParams& tp, const unsigned char* src, int epoch, uint4 (&v)[N2]) {
    int spins = 0;
    while (!tp_all_tagged(v, epoch)) {
        if (spins == 0 && *reinterpret_cast<volatile int*>(tp.status) != 0) break;
        if (++spins > kTpSpinLimit) { tp_wait_expired(tp); break; }
        __nanosleep(64);
        tp_load_tagged(src, v);
    }
}
template <int N2>
__device__ __forceinline__ void tp_accumulate(const uint4 (&v)[N2], float* acc) {
#pragma unroll
    for (int i = 0; i < N2; ++i) { acc[2 * i] += __uint_as_float(v[i].x); acc[2 * i + 1] += __uint_as_float(v[i].z); }
}
// One source after the other.
template <int N2>
__device__ __forceinline__ void tp_add_tagged(const TpParams& tp, const unsigned char* src, int epoch, float* acc) {
    uint4 v[N2];
    tp_load_tagged(src, v);
    tp_poll_tagged(tp, src, epoch, v);
    tp_accumulate(v, acc);
}
// All sources of an exchange, two at a time: their loads travel together (one L2 round trip per two ranks
// instead of one per rank; more at a time would spill the product kernels' registers); the sums are still
// taken in rank order.
template <int N2>
__device__ __forceinline__ void tp_add_tagged_all(const TpParams& tp, size_t off0, size_t src_stride, int epoch, float* acc) {
    const unsigned char* own = tp.peer[tp.rank];
#pragma unroll 1
    for (int s0 = 0; s0 < tp.tp; s0 += 2) {
        uint4 v[2][N2];
        const bool two = s0 + 1 < tp.tp;
        tp_load_tagged(own + off0 + (size_t)s0 * src_stride, v[0]);
        if (two) tp_load_tagged(own + off0 + (size_t)(s0 + 1) * src_stride, v[1]);
        tp_poll_tagged(tp, own + off0 + (size_t)s0 * src_stride, epoch, v[0]);
        tp_accumulate(v[0], acc);
        if (two) {
            tp_poll_tagged(tp, own + off0 + (size_t)(s0 + 1) * src_stride, epoch, v[1]);
            tp_accumulate(v[1], acc);
        }
    }
}
#endif

}  // namespace swlm
