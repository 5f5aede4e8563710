// Host runtime of libswlm_cuda.so: weight store, plan compiler (step list -> fused launch list),
// per-context runtime state, CUDA-graph decode executor, and the C ABI declared in include/swlm.h.
//
// Reference counterparts: STAFWeightStore (Sources/MetalCompiler/STAF/STAFLoader.swift:213-299),
// MetalDispatchStepBuilder.buildDecodePlan (Compiler/MetalDispatchStepBuilder.swift:4-105),
// MetalInferenceModel / MetalDecodeExecutor (Execution/MetalInferenceModel.swift,
// Execution/MetalDecodeExecutor.swift:7-43), MetalPromptStateStore (Execution/MetalPromptStateStore.swift:5-137).
// Where the reference encodes and commits a command buffer per token and blocks on it, this runtime
// captures the whole step into one CUDA graph and keeps position, input token and output token on
// the device, so consecutive greedy steps need no host round trip.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <cmath>

#include "swlm_internal.h"

namespace swlm {

// ---- errors ---------------------------------------------------------------------------------------
static thread_local char g_error[512] = "";
void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}
bool pdl_enabled() {
    static const bool on = [] { const char* v = getenv("SWLM_NO_PDL"); return !(v && v[0] == '1'); }();
    return on;
}
int cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return SWLM_ERR_CUDA;
}

}  // namespace swlm

using namespace swlm;

// =====================================================================================================
// Context + weight store
// =====================================================================================================
struct swlm_ctx {
    int device = 0, tp_rank = 0, tp_size = 1;
    cudaStream_t stream = nullptr;
    std::map<std::string, Q4Raw> raw;
    std::map<std::string, Q4Tiled> tiled;  // plain and fused tensors, keyed by name ("a|b|c" for fused)
    std::map<std::string, Q4Raw> raw_cat;  // source-layout tensors with the rows of several raw tensors one after the other ("a|b|c")
    std::map<std::string, DenseTensor> dense;
    std::map<std::string, DenseF32> densef;   // fp32 tensors (recurrent layers' norm weight and A_log)
    int64_t bytes = 0;
    float* op_partial = nullptr; size_t op_partial_floats = 0;
    unsigned char* op_xh = nullptr; size_t op_xh_bytes = 0;   // scratch of the op-level tensor-core product
    unsigned* op_attn_counters = nullptr; size_t op_attn_counter_count = 0;
    unsigned* op_counters = nullptr; size_t op_counter_count = 0;
    int* tc_status = nullptr;  // device word the tcgen05 GEMM sets when one of its bounded waits expired
    // Lifetime: plans keep their context alive, states their plan. A destroy call on an object that still has
    // users only marks it; the memory goes when the last user is destroyed (hosts with garbage-collected
    // wrappers release objects in no particular order).
    int users = 0;
    bool destroy_requested = false;
};

namespace {

int ensure_device(const swlm_ctx* ctx) {
    SWLM_CUDA(cudaSetDevice(ctx->device));
    return SWLM_OK;
}

template <typename T>
int dev_alloc(T** p, size_t count, swlm_ctx* ctx = nullptr) {
    *p = nullptr;
    if (count == 0) return SWLM_OK;
    SWLM_CUDA(cudaMalloc((void**)p, count * sizeof(T)));
    if (ctx) ctx->bytes += (int64_t)(count * sizeof(T));
    return SWLM_OK;
}

int alloc_tiled(swlm_ctx* ctx, int n, int k, bool sb_f16, Q4Tiled* t) {
    t->n = n; t->k = k; t->sb_f16 = sb_f16;
    t->row_tiles = (n + 15) / 16;
    t->kt_pad = ((k / 64 + 3) / 4) * 4;
    int rc = dev_alloc(&t->tiles, (size_t)t->row_tiles * t->kt_pad * 32, ctx);
    if (rc) return rc;
    return dev_alloc(&t->sb, (size_t)t->row_tiles * (t->kt_pad / 4) * 16, ctx);
}

// Rank-local slice of a [rows][cols] matrix given in `unit`-sized column units.
// `parts` > 1: the rows are `parts` equal sections of `part_stride` source rows and the slice takes rows
// [row0, row0 + rows) of every section, laid one after the other.
struct Slice { int row0, rows, col0, cols; int parts = 1; int part_stride = 0; };
int shard_slice(const swlm_ctx* ctx, int shard_kind, int n, int k, Slice* s) {
    *s = Slice{0, n, 0, k};
    if (ctx->tp_size == 1 || shard_kind == SWLM_SHARD_REPLICATE) return SWLM_OK;
    if (shard_kind == SWLM_SHARD_COLUMN) {
        if (n % ctx->tp_size) { set_error("column shard: n=%d not divisible by tp=%d", n, ctx->tp_size); return SWLM_ERR_INVALID; }
        s->rows = n / ctx->tp_size; s->row0 = ctx->tp_rank * s->rows;
        return SWLM_OK;
    }
    if (shard_kind == SWLM_SHARD_ROW) {
        if (k % (64 * ctx->tp_size)) { set_error("row shard: k=%d not divisible by 64*tp", k); return SWLM_ERR_INVALID; }
        s->cols = k / ctx->tp_size; s->col0 = ctx->tp_rank * s->cols;
        return SWLM_OK;
    }
    if (shard_kind == SWLM_SHARD_COLUMN3) {
        if (n % (3 * ctx->tp_size)) { set_error("three-section column shard: n=%d not divisible by 3*tp=%d", n, 3 * ctx->tp_size); return SWLM_ERR_INVALID; }
        s->parts = 3; s->part_stride = n / 3;
        s->rows = n / 3 / ctx->tp_size; s->row0 = ctx->tp_rank * s->rows;
        return SWLM_OK;
    }
    set_error("unsupported shard kind %d", shard_kind);
    return SWLM_ERR_UNSUPPORTED;
}

const Q4Tiled* find_tiled(swlm_ctx* ctx, const std::string& name) {
    auto it = ctx->tiled.find(name);
    return it == ctx->tiled.end() ? nullptr : &it->second;
}

// Build (or fetch) the streaming-layout tensor for one raw tensor or a fusion of several.
int get_tiled(swlm_ctx* ctx, const std::vector<std::string>& names, int mode, const Q4Tiled** out) {
    std::string key = names[0];
    for (size_t i = 1; i < names.size(); ++i) key += (mode == 1 ? "^" : "|") + names[i];
    if (const Q4Tiled* t = find_tiled(ctx, key)) { *out = t; return SWLM_OK; }
    RepackSrc src[3];
    int n_total = 0, k = 0;
    bool f16 = false;
    for (size_t i = 0; i < names.size(); ++i) {
        auto it = ctx->raw.find(names[i]);
        if (it == ctx->raw.end()) { set_error("tensor '%s' not in the weight store", names[i].c_str()); return SWLM_ERR_NOT_FOUND; }
        const Q4Raw& r = it->second;
        if (i == 0) { k = r.k; f16 = r.sb_f16; }
        else if (r.k != k || r.sb_f16 != f16) { set_error("fused tensors must share K and header type"); return SWLM_ERR_INVALID; }
        src[i] = RepackSrc{r.w, r.scales, r.biases, r.n};
        n_total += r.n;
    }
    if (mode == 1) {
        if (names.size() != 2 || src[0].n != src[1].n) { set_error("interleave needs two tensors with equal N"); return SWLM_ERR_INVALID; }
        n_total = ((src[0].n + 7) / 8) * 16;
    }
    Q4Tiled t;
    int rc = alloc_tiled(ctx, n_total, k, f16, &t);
    if (rc) return rc;
    t.interleaved = mode == 1;
    rc = launch_repack(src, (int)names.size(), mode, k, t, ctx->stream);
    if (rc) return rc;
    SWLM_CUDA(cudaStreamSynchronize(ctx->stream));
    ctx->tiled[key] = t;
    *out = &ctx->tiled[key];
    return SWLM_OK;
}

int add_q4_raw(swlm_ctx* ctx, const char* name, int n, int k, const uint32_t* w, const uint16_t* s,
               const uint16_t* b, bool f16, int shard_kind) {
    if (!ctx || !name || !w || !s || !b) { set_error("null argument"); return SWLM_ERR_INVALID; }
    if (n <= 0 || k <= 0 || k % 64) { set_error("q4g64 tensor '%s': k=%d must be a positive multiple of 64", name, k); return SWLM_ERR_INVALID; }
    int rc = ensure_device(ctx);
    if (rc) return rc;
    Slice sl;
    rc = shard_slice(ctx, shard_kind, n, k, &sl);
    if (rc) return rc;
    // Re-adding a name replaces the tensor and every fused layout built from it; plans compiled against
    // the old tensor must be rebuilt.
    auto old = ctx->raw.find(name);
    if (old != ctx->raw.end()) {
        SWLM_CUDA(cudaDeviceSynchronize());
        cudaFree(old->second.w); cudaFree(old->second.scales); cudaFree(old->second.biases);
        ctx->raw.erase(old);
        const std::string needle = name;
        for (auto it = ctx->tiled.begin(); it != ctx->tiled.end();) {
            bool uses = false;
            size_t start = 0;
            const std::string& key = it->first;
            while (start <= key.size()) {
                size_t end = key.find_first_of("|^", start);
                if (end == std::string::npos) end = key.size();
                uses |= key.compare(start, end - start, needle) == 0;
                start = end + 1;
            }
            if (uses) { cudaFree(it->second.tiles); cudaFree(it->second.sb); it = ctx->tiled.erase(it); }
            else ++it;
        }
        for (auto it = ctx->raw_cat.begin(); it != ctx->raw_cat.end();) {
            bool uses = false;
            size_t start = 0;
            const std::string& key = it->first;
            while (start <= key.size()) {
                size_t end = key.find('|', start);
                if (end == std::string::npos) end = key.size();
                uses |= key.compare(start, end - start, needle) == 0;
                start = end + 1;
            }
            if (uses) { cudaFree(it->second.w); cudaFree(it->second.scales); cudaFree(it->second.biases); it = ctx->raw_cat.erase(it); }
            else ++it;
        }
    }
    Q4Raw r;
    r.n = sl.rows * sl.parts; r.k = sl.cols; r.sb_f16 = f16; r.shard_kind = shard_kind;
    const int wpr = k / 8, gpr = k / 64, lw = sl.cols / 8, lg = sl.cols / 64;
    if ((rc = dev_alloc(&r.w, (size_t)r.n * lw, ctx))) return rc;
    if ((rc = dev_alloc(&r.scales, (size_t)r.n * lg, ctx))) return rc;
    if ((rc = dev_alloc(&r.biases, (size_t)r.n * lg, ctx))) return rc;
    for (int part = 0; part < sl.parts; ++part) {
        const size_t src_row = (size_t)part * sl.part_stride + sl.row0, dst_row = (size_t)part * sl.rows;
        SWLM_CUDA(cudaMemcpy2D(r.w + dst_row * lw, (size_t)lw * 4, w + src_row * wpr + sl.col0 / 8, (size_t)wpr * 4, (size_t)lw * 4, sl.rows, cudaMemcpyHostToDevice));
        SWLM_CUDA(cudaMemcpy2D(r.scales + dst_row * lg, (size_t)lg * 2, s + src_row * gpr + sl.col0 / 64, (size_t)gpr * 2, (size_t)lg * 2, sl.rows, cudaMemcpyHostToDevice));
        SWLM_CUDA(cudaMemcpy2D(r.biases + dst_row * lg, (size_t)lg * 2, b + src_row * gpr + sl.col0 / 64, (size_t)gpr * 2, (size_t)lg * 2, sl.rows, cudaMemcpyHostToDevice));
    }
    ctx->raw[name] = r;
    return SWLM_OK;
}

}  // namespace

// =====================================================================================================
// Plan
// =====================================================================================================
namespace {

enum LaunchKind { L_EMBED, L_RMSNORM, L_QGEMV, L_QK_NORM, L_ATTN, L_SWIGLU, L_CONV, L_ARGMAX, L_SSM };

struct Launch {
    int kind = 0;
    swlm_step st{};            // the (first) step this launch came from
    const Q4Tiled* w = nullptr;
    std::vector<std::string> w_names;
    int w_mode = 0;
    int epilogue = QGEMV_EPI_STORE;
    int gated_act = GATED_ACT_SILU;
    int n_seg = 1;
    int seg_buf[3] = {-1, -1, -1};
    int seg_end[3] = {0, 0, 0};
    const DenseTensor* d1 = nullptr;
    const DenseTensor* d2 = nullptr;
    const Q4Raw* q_embed = nullptr;  // embedding step over a quantized table
    const DenseF32* f1 = nullptr;    // recurrent step: norm weight, A_log (d1 = conv taps, d2 = dt_bias)
    const DenseF32* f2 = nullptr;
    int rope_table = -1;       // index into plan->rope_tables
    std::string label;
    int steps_covered = 1;
    // residual add / copy / RMSNorm folded into this product's prologue (norm.kind == 0: none)
    swlm_step norm{};
    const DenseTensor* norm_w = nullptr;
    int x_buf = -1;            // buffer the product reads (the norm's input when fused)
    int push = 0, in_tp = 0;   // tensor parallel: partial rows pushed to all ranks / pushed partials consumed
    int res_in = 0, res_out = 0;  // physical residual buffers (0 or 1) this launch reads / writes
    int prefetch_launch = -1;     // index of the later product whose weights this launch pulls into L2
    int kv_prefetch_attn = -1;    // index of the attention launch whose K/V rows this product pulls into L2
};

struct RopeTable { int rope_dim; float base; float* inv_freq; };

}  // namespace

struct swlm_plan {
    swlm_ctx* ctx = nullptr;
    swlm_buffers_desc desc{};
    std::vector<swlm_step> steps;
    std::vector<Launch> launches;
    std::vector<RopeTable> rope_tables;
    int attn_splits = 1;
    size_t attn_scratch = 0, qgemv_partial = 0, qgemv_counters = 0;
    int final_res = 0;  // physical residual buffer that holds the residual stream after a step
    // Row-wise execution (prompt chunks, more than 16 sequences): consecutive products of one input run as one product
    // over their concatenated rows. Per step: how many steps the product starting there covers (0: covered by an
    // earlier one) and the tensor it multiplies.
    struct RowsGroup { int count = 1; const Q4Raw* raw = nullptr; };
    std::vector<RowsGroup> rows_groups;
    bool rows_groups_ready = false;
    int users = 0;
    bool destroy_requested = false;
};

namespace {

int buf_width(const swlm_buffers_desc& d, int buf) {
    if (buf == SWLM_BUF_HIDDEN || buf == SWLM_BUF_RESIDUAL) return d.hidden;
    if (buf == SWLM_BUF_LOGITS) return d.vocab;
    return d.slot_dim;
}

const DenseTensor* find_dense(swlm_ctx* ctx, const char* name) {
    auto it = ctx->dense.find(name);
    return it == ctx->dense.end() ? nullptr : &it->second;
}

int rope_table_for(swlm_plan* plan, int rope_dim, float base, int* index) {
    for (size_t i = 0; i < plan->rope_tables.size(); ++i)
        if (plan->rope_tables[i].rope_dim == rope_dim && plan->rope_tables[i].base == base) { *index = (int)i; return SWLM_OK; }
    // theta_i = base^(-2i/ropeDim) evaluated in fp32 on the host
    // (Generator/MetalSourceGenerator+Attention.swift:606-609 evaluates the same expression per call).
    std::vector<float> f(rope_dim / 2);
    for (int i = 0; i < rope_dim / 2; ++i) f[i] = powf(base, -2.0f * (float)i / (float)rope_dim);
    RopeTable t{rope_dim, base, nullptr};
    int rc = dev_alloc(&t.inv_freq, f.size());
    if (rc) return rc;
    SWLM_CUDA(cudaMemcpy(t.inv_freq, f.data(), f.size() * 4, cudaMemcpyHostToDevice));
    plan->rope_tables.push_back(t);
    *index = (int)plan->rope_tables.size() - 1;
    return SWLM_OK;
}

bool buf_ok(int b) { return b >= 0 && b < SWLM_BUF_COUNT; }

int compile_plan(swlm_plan* plan) {
    swlm_ctx* ctx = plan->ctx;
    const swlm_buffers_desc& d = plan->desc;
    const std::vector<swlm_step>& st = plan->steps;
    const int m = d.max_batch;
    int rc;
    for (size_t i = 0; i < st.size();) {
        const swlm_step& s = st[i];
        Launch L;
        L.st = s;
        switch (s.kind) {
        case SWLM_STEP_EMBED:
            L.kind = L_EMBED;
            L.d1 = find_dense(ctx, s.weight);
            if (!L.d1) {
                // a quantized table (tied to the output head): gathered from the packed source copy
                auto q = ctx->raw.find(s.weight);
                if (q == ctx->raw.end()) { set_error("embedding table '%s' missing", s.weight); return SWLM_ERR_NOT_FOUND; }
                if (ctx->tp_size > 1) { set_error("a quantized (tied) embedding table is not supported under tensor parallelism"); return SWLM_ERR_UNSUPPORTED; }
                if (q->second.k != s.n) { set_error("embedding table '%s': width %d, hidden %d", s.weight, q->second.k, s.n); return SWLM_ERR_INVALID; }
                L.q_embed = &q->second;
            }
            if (!buf_ok(s.out_buf) || s.n > buf_width(d, s.out_buf)) { set_error("embed: bad output buffer"); return SWLM_ERR_INVALID; }
            L.label = std::string("embed ") + s.weight;
            break;
        case SWLM_STEP_COPY_RMSNORM:
        case SWLM_STEP_RESADD_COPY_RMSNORM:
        case SWLM_STEP_RESADD_RMSNORM:
            L.kind = L_RMSNORM;
            L.d1 = find_dense(ctx, s.weight);
            if (!L.d1) { set_error("norm weight '%s' missing", s.weight); return SWLM_ERR_NOT_FOUND; }
            if (!buf_ok(s.in_buf) || !buf_ok(s.out_buf) || L.d1->rows * L.d1->cols < s.n) { set_error("rmsnorm: bad buffers"); return SWLM_ERR_INVALID; }
            L.label = std::string("rmsnorm ") + s.weight;
            break;
        case SWLM_STEP_QGEMV: {
            L.kind = L_QGEMV;
            if (!buf_ok(s.in_buf) || !buf_ok(s.out_buf)) { set_error("qgemv: bad buffers"); return SWLM_ERR_INVALID; }
            // gate, up, swiglu -> one launch over row-interleaved weights with a SwiGLU epilogue
            if (i + 2 < st.size() && st[i + 1].kind == SWLM_STEP_QGEMV && (st[i + 2].kind == SWLM_STEP_SWIGLU || st[i + 2].kind == SWLM_STEP_GEGLU) &&
                st[i + 1].in_buf == s.in_buf && st[i + 1].k == s.k && st[i + 1].n == s.n &&
                st[i + 2].in_buf == s.out_buf && st[i + 2].in2_buf == st[i + 1].out_buf && (s.n % 8) == 0) {
                rc = get_tiled(ctx, {s.weight, st[i + 1].weight}, 1, &L.w);
                if (rc) return rc;
                L.w_names = {s.weight, st[i + 1].weight}; L.w_mode = 1;
                L.epilogue = QGEMV_EPI_SWIGLU;
                L.gated_act = st[i + 2].kind == SWLM_STEP_GEGLU ? GATED_ACT_GELU_TANH : GATED_ACT_SILU;
                L.seg_buf[0] = st[i + 2].out_buf;
                L.seg_end[0] = ctx->raw[s.weight].n;
                L.steps_covered = 3;
                L.label = std::string(L.gated_act ? "qgemv+geglu " : "qgemv+swiglu ") + s.weight + " ^ " + st[i + 1].weight;
                break;
            }
            // consecutive projections of one input -> one launch over concatenated rows
            std::vector<std::string> names{s.weight};
            size_t jn = i + 1;
            while (jn < st.size() && names.size() < 3 && st[jn].kind == SWLM_STEP_QGEMV && st[jn].in_buf == s.in_buf &&
                   st[jn].k == s.k && st[jn].out_buf != s.in_buf) {
                bool clash = false;
                for (size_t q = i; q < jn; ++q) clash |= st[q].out_buf == st[jn].out_buf;
                if (clash) break;
                names.push_back(st[jn].weight);
                ++jn;
            }
            if (s.out_buf == s.in_buf && names.size() > 1) names.resize(1);
            rc = get_tiled(ctx, names, 0, &L.w);
            if (rc) return rc;
            L.w_names = names; L.w_mode = 0;
            L.n_seg = (int)names.size();
            int end = 0;
            L.label = "qgemv";
            for (int q = 0; q < L.n_seg; ++q) {
                const Q4Raw& r = ctx->raw[names[q]];
                end += r.n;
                L.seg_buf[q] = st[i + q].out_buf;
                L.seg_end[q] = end;
                if (r.n > buf_width(d, st[i + q].out_buf)) { set_error("qgemv '%s': n=%d exceeds the output buffer", names[q].c_str(), r.n); return SWLM_ERR_INVALID; }
                L.label += " " + names[q];
            }
            if (L.w->k > buf_width(d, s.in_buf)) { set_error("qgemv '%s': k=%d exceeds the input buffer", s.weight, L.w->k); return SWLM_ERR_INVALID; }
            L.steps_covered = L.n_seg;
            break;
        }
        case SWLM_STEP_QK_NORM:
            L.kind = L_QK_NORM;
            L.d1 = find_dense(ctx, s.weight);
            L.d2 = find_dense(ctx, s.weight2);
            if (!L.d1 || !L.d2) { set_error("qk norm weights missing"); return SWLM_ERR_NOT_FOUND; }
            L.label = "qk_norm";
            break;
        case SWLM_STEP_ATTN_DECODE:
            L.kind = L_ATTN;
            if (s.layer < 0 || s.layer >= d.kv_layers) { set_error("attention: layer %d outside the KV cache", s.layer); return SWLM_ERR_INVALID; }
            if (s.head_dim != d.head_dim) { set_error("attention: head_dim differs from the KV cache"); return SWLM_ERR_INVALID; }
            if (s.window_left < 0) { set_error("attention: negative sliding window"); return SWLM_ERR_INVALID; }
            if (s.rope_dim > 0) { rc = rope_table_for(plan, s.rope_dim, s.rope_base, &L.rope_table); if (rc) return rc; }
            L.label = "attn_decode";
            break;
        case SWLM_STEP_SWIGLU:
        case SWLM_STEP_GEGLU:
            L.kind = L_SWIGLU;
            L.gated_act = s.kind == SWLM_STEP_GEGLU ? GATED_ACT_GELU_TANH : GATED_ACT_SILU;
            L.label = L.gated_act ? "geglu" : "swiglu";
            break;
        case SWLM_STEP_CONV_STATE_UPDATE:
            L.kind = L_CONV;
            L.d1 = find_dense(ctx, s.weight);
            if (!L.d1) { set_error("conv weight '%s' missing", s.weight); return SWLM_ERR_NOT_FOUND; }
            if (s.layer < 0 || s.layer >= d.conv_layers) { set_error("conv: layer %d outside the conv state", s.layer); return SWLM_ERR_INVALID; }
            L.label = std::string("conv_state_update ") + s.weight;
            break;
        case SWLM_STEP_SSM_RECURRENCE: {
            L.kind = L_SSM;
            if (ctx->tp_size > 1) { set_error("recurrent layers are not supported under tensor parallelism"); return SWLM_ERR_UNSUPPORTED; }
            const int groups = s.groups > 0 ? s.groups : 1;
            if (s.layer < 0 || s.layer >= d.ssm_layers || s.heads != d.ssm_heads || groups != std::max(1, d.ssm_groups) ||
                s.key_dim != d.ssm_key_dim || s.value_dim != d.ssm_value_dim || s.conv_kernel != d.ssm_conv_kernel ||
                s.heads <= 0 || s.heads % groups || s.key_dim <= 0 || s.value_dim <= 0 || s.conv_kernel < 1) {
                set_error("ssm recurrence: the step's head layout differs from the state's (layer %d)", s.layer);
                return SWLM_ERR_INVALID;
            }
            const int conv_dim = 2 * groups * s.key_dim + s.heads * s.value_dim;
            if (!buf_ok(s.in_buf) || !buf_ok(s.in2_buf) || !buf_ok(s.in3_buf) || !buf_ok(s.in4_buf) || !buf_ok(s.out_buf) ||
                conv_dim > buf_width(d, s.in_buf) || s.heads * s.value_dim > buf_width(d, s.in2_buf) || s.heads > buf_width(d, s.in3_buf) ||
                s.heads > buf_width(d, s.in4_buf) || s.heads * s.value_dim > buf_width(d, s.out_buf)) {
                set_error("ssm recurrence: bad buffers");
                return SWLM_ERR_INVALID;
            }
            L.d1 = find_dense(ctx, s.weight);
            L.d2 = find_dense(ctx, s.weight3);
            auto f1 = ctx->densef.find(s.weight2), f2 = ctx->densef.find(s.weight4);
            if (!L.d1 || !L.d2 || f1 == ctx->densef.end() || f2 == ctx->densef.end()) {
                set_error("ssm recurrence: conv taps / dt_bias (bf16) or norm weight / A_log (fp32) of '%s' missing", s.weight);
                return SWLM_ERR_NOT_FOUND;
            }
            L.f1 = &f1->second; L.f2 = &f2->second;
            if (L.d1->rows * L.d1->cols < (int64_t)conv_dim * s.conv_kernel || L.d2->rows * L.d2->cols < s.heads ||
                L.f1->count < s.value_dim || L.f2->count < s.heads) { set_error("ssm recurrence: tensor sizes of '%s'", s.weight); return SWLM_ERR_INVALID; }
            L.label = std::string("ssm_recurrence ") + s.weight;
            break;
        }
        case SWLM_STEP_ARGMAX:
            L.kind = L_ARGMAX;
            L.label = "argmax";
            break;
        default:
            set_error("step %zu: kind %d is outside the hot path", i, s.kind);
            return SWLM_ERR_UNSUPPORTED;
        }
        i += L.steps_covered;
        if (L.kind == L_QGEMV) {
            plan->qgemv_partial = std::max(plan->qgemv_partial, qgemv_scratch_floats(*L.w, std::min(m, kQGemvMaxRows)));
            plan->qgemv_counters = std::max(plan->qgemv_counters, (size_t)qgemv_counter_count(*L.w));
        }
        plan->launches.push_back(L);
    }
    plan->attn_splits = attn_pick_splits(m, std::max(1, d.kv_heads / std::max(1, ctx->tp_size)), d.max_seq);

    // A gate/up launch with the SwiGLU epilogue writes while other CTAs may still be reading its input:
    // when both are the same buffer, send the result to scratch slot 4 and point the readers there.
    {
        int from = -1, to = -1;
        for (Launch& L : plan->launches) {
            auto redirect = [&](int& b) { if (from >= 0 && b == from) b = to; };
            redirect(L.st.in_buf); redirect(L.st.in2_buf); redirect(L.st.in3_buf);
            if (L.kind == L_SSM) redirect(L.st.in4_buf);
            bool writes = L.st.out_buf == from;
            for (int q = 0; q < L.n_seg; ++q) writes |= L.seg_buf[q] == from;
            if (L.kind == L_QGEMV && L.epilogue == QGEMV_EPI_SWIGLU && L.seg_buf[0] == L.st.in_buf) {
                from = L.seg_buf[0]; to = SWLM_BUF_SCRATCH4;
                L.seg_buf[0] = to;
            } else if (writes && L.kind != L_QK_NORM) {
                from = to = -1;  // the original buffer holds fresh data again
            }
        }
    }

    // Fold each norm into the product that consumes it: the product's CTAs recompute the (tiny) norm in
    // their prologue instead of waiting for a separate launch. Conditions: dimension <= 4096, the product is
    // the very next launch and the only reader of the norm's output.
    const char* no_fuse = getenv("SWLM_NO_NORM_FUSION");
    for (size_t i = 0; i + 1 < plan->launches.size() && !(no_fuse && no_fuse[0] == '1'); ++i) {
        Launch& A = plan->launches[i];
        Launch& B = plan->launches[i + 1];
        if (A.kind != L_RMSNORM || B.kind != L_QGEMV) continue;
        if (B.st.in_buf != A.st.out_buf || B.w->k != A.st.n || A.st.n > 4096 || (A.st.n & 15)) continue;
        bool ok = true;
        for (int q = 0; q < B.n_seg; ++q) ok &= B.seg_buf[q] != A.st.in_buf && B.seg_buf[q] != SWLM_BUF_RESIDUAL;
        for (size_t j = i + 2; j < plan->launches.size() && ok; ++j) {
            const Launch& C = plan->launches[j];
            if (C.st.in_buf == A.st.out_buf || C.st.in2_buf == A.st.out_buf || C.st.in3_buf == A.st.out_buf ||
                (C.kind == L_SSM && C.st.in4_buf == A.st.out_buf)) ok = false;
            bool writes = C.st.out_buf == A.st.out_buf;
            for (int q = 0; q < C.n_seg; ++q) writes |= C.seg_buf[q] == A.st.out_buf;
            if (writes) break;
        }
        if (!ok) continue;
        B.norm = A.st;
        B.norm_w = A.d1;
        B.x_buf = A.st.in_buf;
        B.label = "rmsnorm+" + B.label;
        B.steps_covered += 1;
        plan->launches.erase(plan->launches.begin() + i);
    }
    // residual ping-pong: a fused norm reads one physical residual buffer and writes the other
    int cur = 0;
    for (Launch& L : plan->launches) {
        L.res_in = L.res_out = cur;
        if (L.kind == L_QGEMV && L.norm.kind) {
            L.res_out = 1 - cur;
            if (L.norm.kind != SWLM_STEP_RESADD_RMSNORM) cur = 1 - cur;
        }
    }
    plan->final_res = cur;

    // Cross-launch L2 prefetch (single sequence), off unless SWLM_L2_PREFETCH_MB sets a budget: a product's
    // weights are requested one or two launches early, by attention or by another product, as long as
    // everything requested but not yet consumed stays below the budget (L2 is 126 MB). Measured on a B200 with
    // the Llama-3-8B shape it does not pay: the products are bound by instruction issue, not by HBM, and
    // attention slows down under the extra traffic (527 tok/s without, 501 with a 110 MB budget).
    if (m == 1) {
        double budget = 0;
        if (const char* e = getenv("SWLM_L2_PREFETCH_MB")) budget = atof(e) * 1e6;
        auto wbytes = [&](const Launch& L) { return L.kind == L_QGEMV ? (double)L.w->bytes() : 0.0; };
        for (int j = 0; j < (int)plan->launches.size() && budget > 0; ++j) {
            const Launch& T = plan->launches[j];
            if (T.kind != L_QGEMV || wbytes(T) > 80e6) continue;
            for (int dist = 2; dist >= 1; --dist) {
                const int i = j - dist;
                if (i < 0) continue;
                Launch& P = plan->launches[i];
                if ((P.kind != L_QGEMV && P.kind != L_ATTN) || P.prefetch_launch >= 0) continue;
                double live = wbytes(T);
                for (int l = i; l < j; ++l) live += wbytes(plan->launches[l]);
                if (live > budget) continue;
                P.prefetch_launch = j;
                break;
            }
        }
    }

    // SWLM_KV_PREFETCH=1: the q/k/v product of a single-sequence plan asks for the K/V rows its attention launch
    // is about to read (the cache is static except for the newest row). Measured: attention's main loop gets 1.2 us
    // shorter, the product as much longer; off by default.
    {
        const char* kv = getenv("SWLM_KV_PREFETCH");
        for (int j = 1; j < (int)plan->launches.size() && m == 1 && kv && kv[0] == '1'; ++j) {
            if (plan->launches[j].kind != L_ATTN) continue;
            int i = j - 1;
            if (plan->launches[i].kind == L_QK_NORM && i > 0) --i;
            Launch& P = plan->launches[i];
            if (P.kind == L_QGEMV && P.prefetch_launch < 0) P.kv_prefetch_attn = j;
        }
    }

    // Tensor parallel: a product over a K-sharded (row-parallel) weight yields partial sums. It pushes them
    // to every rank, and the product that follows must be one with a fused norm, which adds them up.
    if (ctx->tp_size > 1) {
        for (const Launch& L : plan->launches)
            if (L.kind == L_ATTN || L.kind == L_QK_NORM)
                if ((rc = swlm_tp_check_heads(L.st.heads, d.kv_heads, ctx->tp_size))) return rc;
        for (size_t i = 0; i < plan->launches.size(); ++i) {
            Launch& L = plan->launches[i];
            if (L.kind == L_CONV) {
                // channels are split across ranks: the B|C|x projection arrives as this rank's three thirds
                // (SWLM_SHARD_COLUMN3), the conv weight rows are this rank's channels, the out projection is row-parallel
                if (L.st.n % ctx->tp_size || L.d1->rows != L.st.n / ctx->tp_size) {
                    set_error("conv '%s': %d channels over %d ranks need a weight of %d rows (add it with SWLM_SHARD_COLUMN)", L.st.weight,
                              L.st.n, ctx->tp_size, L.st.n / ctx->tp_size);
                    return SWLM_ERR_INVALID;
                }
                continue;
            }
            if (L.kind != L_QGEMV) continue;
            auto it = ctx->raw.find(L.st.weight);
            if (it == ctx->raw.end() || it->second.shard_kind != SWLM_SHARD_ROW) continue;
            if (L.n_seg != 1 || L.epilogue != QGEMV_EPI_STORE || L.seg_buf[0] != SWLM_BUF_HIDDEN || L.seg_end[0] != d.hidden) {
                set_error("row-parallel product '%s' must write the hidden buffer", L.st.weight);
                return SWLM_ERR_UNSUPPORTED;
            }
            if (i + 1 >= plan->launches.size() || plan->launches[i + 1].kind != L_QGEMV || !plan->launches[i + 1].norm.kind ||
                plan->launches[i + 1].x_buf != SWLM_BUF_HIDDEN) {
                set_error("row-parallel product '%s' is not followed by a product with a fused norm", L.st.weight);
                return SWLM_ERR_UNSUPPORTED;
            }
            if (L.in_tp) {
                set_error("row-parallel product '%s' would both consume and push partial sums", L.st.weight);
                return SWLM_ERR_UNSUPPORTED;
            }
            L.push = 1;
            plan->launches[i + 1].in_tp = 1;
            L.label = "push " + L.label;
            plan->launches[i + 1].label = "allreduce+" + plan->launches[i + 1].label;
        }
    }

    return SWLM_OK;
}

}  // namespace

// =====================================================================================================
// State
// =====================================================================================================
struct swlm_state {
    swlm_plan* plan = nullptr;
    cudaStream_t own_stream = nullptr, stream = nullptr;
    __nv_bfloat16* buf[SWLM_BUF_COUNT] = {};
    int width[SWLM_BUF_COUNT] = {};
    __nv_bfloat16* kcache = nullptr; __nv_bfloat16* vcache = nullptr; size_t kv_layer_elems = 0;
    // rotated KV schemes: rotors [kv_layers][kv_heads][groups][4], projection matrix [head_dim][qjl_dim], projected K
    // residuals [kv_layers][seq][kv_heads][max_seq][qjl_dim], all fp16
    __half* rotors = nullptr; size_t rotor_layer_elems = 0;
    __half* qjl_matrix = nullptr;
    __half* qjl_res = nullptr; size_t qjl_layer_elems = 0;
    std::vector<uint16_t> rotors_host, qjl_matrix_host;   // host copies for the cache probes
    __nv_bfloat16* conv = nullptr; size_t conv_layer_elems = 0;
    __nv_bfloat16* ssm_conv = nullptr; size_t ssm_conv_layer_elems = 0;   // [layer][seq][kernel][conv_dim]
    float* ssm_state = nullptr; size_t ssm_state_layer_elems = 0;         // [layer][seq][heads][key_dim][value_dim]
    int32_t* position = nullptr; int32_t* step_counter = nullptr;
    int32_t* token_in = nullptr; int32_t* token_out = nullptr; int32_t* ring = nullptr;
    int32_t* prompt = nullptr; size_t prompt_cap = 0;
    int ring_cap = 4096;
    float* attn_scratch = nullptr; float* qgemv_partial = nullptr; unsigned* qgemv_counters = nullptr;
    size_t attn_scratch_cap = 0, qgemv_partial_cap = 0, qgemv_counters_cap = 0;
    unsigned* attn_counters = nullptr;
    float* argmax_val = nullptr; int32_t* argmax_idx = nullptr;
    __nv_bfloat16* res2 = nullptr;  // second physical residual buffer (ping-pong partner of buf[RESIDUAL])
    // tensor-parallel exchange (tp_size > 1): this rank's buffer, the peers' mappings, local counters
    TpParams tp{};
    bool tp_attached = false;
    int32_t* tp_words = nullptr;  // [0] all-reduce epoch, [1] rows-done counter, [2] status, [3] argmax epoch, [4] CTAs done pushing a prompt chunk
    int tp_rows_epoch = 0;        // prompt-chunk exchanges issued so far (the same count on every rank)
    int32_t* h_tok = nullptr;  // pinned host staging, 2 * max_batch
    std::vector<int> pos_host;   // host mirror of the per-sequence positions
    long long steps_host = 0;
    cudaGraphExec_t graph_full = nullptr, graph_body = nullptr;
    int graph_full_launches = 0, graph_body_launches = 0;
    int64_t launches = 0;
    // prompt ingestion in chunks: activation rows for `pf_rows` tokens per logical buffer, attention scratch
    __nv_bfloat16* pf_buf[SWLM_BUF_COUNT] = {};
    int pf_rows = 0;
    unsigned* pf_attn_counters = nullptr;
    unsigned char* wide_xh = nullptr;  // the same for a decode step of more than kQGemvMaxRows sequences
    unsigned char* pf_xh = nullptr;  // scratch of the tensor-core product: fp16 copy of a chunk's widest activations
    int* pf_status = nullptr;      // device word: a bounded wait of the tensor-core product expired
    int prefill_chunk = 2048;      // tokens per chunk; 0 = one token at a time through the decode graph
    int* tc_status = nullptr;      // pinned host word (mapped): a bounded wait of a kernel expired
};

struct swlm_snap {
    std::vector<void*> dev;
    std::vector<size_t> bytes;
    std::vector<int> pos_host;
};

namespace {

// ---- rotated KV schemes on the host: parameters by the reference's rule, and the arithmetic of the cache probes ----
uint16_t host_f16_bits(float f) { const __half h = __float2half_rn(f); uint16_t u; memcpy(&u, &h, 2); return u; }
float host_f16_value(uint16_t u) { __half h; memcpy(static_cast<void*>(&h), &u, 2); return __half2float(h); }

// initializeRandomUnitRotors (Buffer/MetalGraphAllocator.swift:349-390): rotor i of [layer][kv_head][group] takes four
// successive values of the 64-bit LCG x -> x * 6364136223846793005 + 1442695040888963407 started from that map of i,
// each mapped to [-1, 1) by its top 31 bits, normalised to a unit quaternion in fp32 and stored as fp16 (s, b12, b13, b23).
void kv_rotor_init_host(int layers, int kv_heads, int groups, std::vector<uint16_t>* out) {
    const size_t total = (size_t)layers * kv_heads * groups;
    out->assign(total * 4, 0);
    const float unit = 1.0f / (float)(1 << 30);
    for (size_t i = 0; i < total; ++i) {
        uint64_t h = (uint64_t)i;
        float c[4];
        for (int j = 0; j < 4; ++j) {
            h = h * 6364136223846793005ull + 1442695040888963407ull;
            c[j] = (float)((int64_t)(h >> 33) - ((int64_t)1 << 30)) * unit;
        }
        const float norm = sqrtf(c[0] * c[0] + c[1] * c[1] + c[2] * c[2] + c[3] * c[3]);
        if (norm < 1e-8f) { c[0] = 1.0f; c[1] = c[2] = c[3] = 0.0f; }
        else { const float inv = 1.0f / norm; for (int j = 0; j < 4; ++j) c[j] *= inv; }
        for (int j = 0; j < 4; ++j) (*out)[i * 4 + j] = host_f16_bits(c[j]);
    }
}
// initializeRademacherMatrix (:393-411): entry i of [head_dim][qjl_dim] is +1/sqrt(qjl_dim) when bit 33 of the first
// LCG value of i is clear, else -1/sqrt(qjl_dim).
void kv_qjl_matrix_init_host(int head_dim, int qjl_dim, std::vector<uint16_t>* out) {
    const float scale = 1.0f / sqrtf((float)qjl_dim);
    const uint16_t pos = host_f16_bits(scale), neg = host_f16_bits(-scale);
    out->assign((size_t)head_dim * qjl_dim, 0);
    for (size_t i = 0; i < out->size(); ++i) {
        const uint64_t h = (uint64_t)i * 6364136223846793005ull + 1442695040888963407ull;
        (*out)[i] = ((h >> 33) & 1) == 0 ? pos : neg;
    }
}
// rotor_sandwich / rotor_sandwich_inverse over every group of three values of a row (rotor_apply_forward / _inverse,
// Generator/MetalSourceGenerator+Attention.swift:1807-1884); R = [groups][4] fp16
void kv_rotor_turn_row_host(float* row, int hd, const uint16_t* R, bool inverse) {
    for (int g = 0; 3 * g < hd; ++g) {
        const int base = 3 * g;
        const float x = row[base], y = base + 1 < hd ? row[base + 1] : 0.0f, z = base + 2 < hd ? row[base + 2] : 0.0f;
        const float s = host_f16_value(R[4 * g]);
        float px = host_f16_value(R[4 * g + 3]), py = -host_f16_value(R[4 * g + 2]), pz = host_f16_value(R[4 * g + 1]);
        if (inverse) { px = -px; py = -py; pz = -pz; }
        const float tx = 2.0f * (py * z - pz * y), ty = 2.0f * (pz * x - px * z), tz = 2.0f * (px * y - py * x);
        row[base] = x + s * tx + (py * tz - pz * ty);
        if (base + 1 < hd) row[base + 1] = y + s * ty + (pz * tx - px * tz);
        if (base + 2 < hd) row[base + 2] = z + s * tz + (px * ty - py * tx);
    }
}

PrefetchTarget prefetch_of(const Launch& L) {
    PrefetchTarget t;
    t.p[0] = L.w->tiles; t.bytes[0] = (unsigned long long)L.w->row_tiles * L.w->kt_pad * 512;
    t.p[1] = L.w->sb; t.bytes[1] = (unsigned long long)L.w->row_tiles * (L.w->kt_pad / 4) * 256;
    return t;
}

__nv_bfloat16* res_buf(swlm_state* s, int phys) { return phys ? s->res2 : s->buf[SWLM_BUF_RESIDUAL]; }

size_t kv_row_bytes(const swlm_buffers_desc& d) {
    return (size_t)swlm_kv_row_bytes(d.kv_scheme, d.head_dim);
}

int kv_heads_local(const swlm_plan* p) { return std::max(1, p->desc.kv_heads / std::max(1, p->ctx->tp_size)); }

size_t head_begin_of(const swlm_plan* plan, bool body_only) {
    size_t head_begin = plan->launches.size();
    while (body_only && head_begin > 0 &&
           (plan->launches[head_begin - 1].kind == L_ARGMAX ||
            (plan->launches[head_begin - 1].kind == L_QGEMV && plan->launches[head_begin - 1].seg_buf[0] == SWLM_BUF_LOGITS) ||
            (plan->launches[head_begin - 1].kind == L_RMSNORM && plan->launches[head_begin - 1].st.kind == SWLM_STEP_RESADD_RMSNORM)))
        --head_begin;
    return head_begin;
}

int enqueue_rows(swlm_state* s, bool wide, const int32_t* tokens, int c, int pos0, int seq, int head_row, bool body_only,
                 cudaStream_t stream);

// Enqueue the launches of one decode step. body_only skips the output head (lm_head + argmax) and
// advances the position with a one-thread kernel instead.
int enqueue_step(swlm_state* s, bool body_only, cudaStream_t stream, int only_kind = -1) {
    const swlm_plan* plan = s->plan;
    const swlm_buffers_desc& d = plan->desc;
    const int m = d.max_batch;
    int rc = SWLM_OK;
    const size_t n_launch = plan->launches.size();
    // the output head is the trailing [norm, lm_head, argmax] group
    (void)n_launch;
    if (m > kQGemvMaxRows) {
        if (only_kind >= 0) { set_error("per-kind timing is for plans of up to %d sequences", kQGemvMaxRows); return SWLM_ERR_UNSUPPORTED; }
        return enqueue_rows(s, true, s->token_in, m, 0, 0, -1, body_only, stream);
    }
    const size_t head_begin = head_begin_of(plan, body_only);
    bool advanced = false;
    auto gemv_launch_of = [&](const Launch& L) {
        const swlm_step& st = L.st;
        QGemvLaunch a;
        const int xb = L.norm.kind ? L.x_buf : st.in_buf;
        a.w = L.w; a.x = s->buf[xb]; a.x_stride = s->width[xb]; a.m = m; a.epilogue = L.epilogue; a.gated_act = L.gated_act;
        if (L.norm.kind) {
            a.norm.mode = L.norm.kind;
            a.norm.res_in = res_buf(s, L.res_in); a.norm.res_out = res_buf(s, L.res_out);
            a.norm.res_stride = s->width[SWLM_BUF_RESIDUAL];
            a.norm.weight = L.norm_w->data; a.norm.eps = L.norm.eps; a.norm.weight_bias = L.norm.weight_bias;
        }
        for (int q = 0; q < L.n_seg; ++q) { a.y[q] = s->buf[L.seg_buf[q]]; a.y_stride[q] = s->width[L.seg_buf[q]]; a.seg_end[q] = L.seg_end[q]; }
        a.partial = s->qgemv_partial; a.counters = s->qgemv_counters;
        if (L.prefetch_launch >= 0) a.prefetch = prefetch_of(plan->launches[L.prefetch_launch]);
        if (L.kv_prefetch_attn >= 0) {
            const swlm_step& at = plan->launches[L.kv_prefetch_attn].st;
            a.prefetch.p[0] = s->kcache + (size_t)at.layer * s->kv_layer_elems;
            a.prefetch.p[1] = s->vcache + (size_t)at.layer * s->kv_layer_elems;
            a.prefetch.heads = kv_heads_local(plan);
            a.prefetch.row_bytes = (unsigned)kv_row_bytes(d);
            a.prefetch.head_stride = (unsigned long long)d.max_seq * kv_row_bytes(d);
            a.prefetch.position = s->position;
        }
        return a;
    };
    for (size_t li = 0; li < head_begin; ++li) {
        const Launch& L = plan->launches[li];
        const swlm_step& st = L.st;
        if (only_kind >= 0 && L.kind != only_kind) continue;
        switch (L.kind) {
        case L_EMBED:
            rc = L.q_embed ? launch_embed_q4(m, st.n, s->token_in, *L.q_embed, s->buf[st.out_buf], s->width[st.out_buf], stream)
                           : launch_embed(m, st.n, s->token_in, d.vocab, L.d1->data, s->buf[st.out_buf], s->width[st.out_buf], stream);
            s->launches += 1;
            break;
        case L_RMSNORM:
            rc = launch_rmsnorm(st.kind, m, st.n, s->buf[st.in_buf], s->width[st.in_buf], res_buf(s, L.res_in),
                                s->width[SWLM_BUF_RESIDUAL], L.d1->data, st.eps, st.weight_bias, s->buf[st.out_buf],
                                s->width[st.out_buf], stream);
            s->launches += 1;
            break;
        case L_QGEMV: {
            QGemvLaunch a = gemv_launch_of(L);
            if (L.push || L.in_tp) {
                if (!s->tp_attached) { set_error("tensor-parallel plan: call swlm_tp_export / swlm_tp_attach on the state first"); return SWLM_ERR_STATE; }
                a.push = L.push; a.in_tp = L.in_tp; a.tp = s->tp;
            }
            rc = launch_qgemv(a, stream);
            s->launches += 1;
            break;
        }
        case L_QK_NORM:
            rc = launch_qk_norm(m, st.heads / plan->ctx->tp_size, kv_heads_local(plan), st.head_dim, s->buf[st.in_buf], s->width[st.in_buf],
                                s->buf[st.in2_buf], s->width[st.in2_buf], L.d1->data, L.d2->data, st.eps, st.weight_bias, stream);
            s->launches += 1;
            break;
        case L_ATTN: {
            AttnLaunch a;
            a.m = m; a.heads = st.heads / plan->ctx->tp_size; a.kv_heads = kv_heads_local(plan); a.head_dim = st.head_dim;
            a.rope_dim = st.rope_dim; a.inv_freq = L.rope_table >= 0 ? plan->rope_tables[L.rope_table].inv_freq : nullptr;
            a.scale = st.scale; a.window = st.window_left; a.kv_scheme = d.kv_scheme;
            if (swlm_kv_is_rotor(d.kv_scheme)) {
                a.rotors = s->rotors + (size_t)st.layer * s->rotor_layer_elems;
                a.qjl_dim = d.kv_qjl_dim; a.qjl_matrix = s->qjl_matrix;
                a.qjl_res = s->qjl_res ? s->qjl_res + (size_t)st.layer * s->qjl_layer_elems : nullptr;
            }
            a.q = s->buf[st.in_buf]; a.q_stride = s->width[st.in_buf];
            a.k = s->buf[st.in2_buf]; a.k_stride = s->width[st.in2_buf];
            a.v = s->buf[st.in3_buf]; a.v_stride = s->width[st.in3_buf];
            a.kcache = s->kcache + (size_t)st.layer * s->kv_layer_elems;
            a.vcache = s->vcache + (size_t)st.layer * s->kv_layer_elems;
            a.max_seq = d.max_seq; a.position = s->position;
            a.out = s->buf[st.out_buf]; a.out_stride = s->width[st.out_buf];
            a.scratch = s->attn_scratch; a.counters = s->attn_counters; a.splits = plan->attn_splits;
            if (L.prefetch_launch >= 0) a.prefetch = prefetch_of(plan->launches[L.prefetch_launch]);
            rc = launch_attn_decode(a, stream);
            s->launches += 1;
            break;
        }
        case L_SWIGLU:
            rc = launch_swiglu(m, st.n, s->buf[st.in_buf], s->width[st.in_buf], s->buf[st.in2_buf], s->width[st.in2_buf],
                               s->buf[st.out_buf], s->width[st.out_buf], L.gated_act, stream);
            s->launches += 1;
            break;
        case L_CONV:
            // under tensor parallelism a rank owns n / tp channels (its slab is used from the front)
            rc = launch_conv_step(m, st.n / plan->ctx->tp_size, st.conv_kernel, s->conv + (size_t)st.layer * s->conv_layer_elems,
                                  (size_t)d.conv_kernel * d.conv_dim, s->buf[st.in_buf], s->width[st.in_buf], L.d1->data,
                                  s->buf[st.out_buf], s->width[st.out_buf], stream);
            s->launches += 1;
            break;
        case L_SSM: {
            SsmLaunch a;
            a.m = m; a.heads = st.heads; a.groups = std::max(1, st.groups); a.key_dim = st.key_dim; a.value_dim = st.value_dim; a.kernel = st.conv_kernel;
            a.qkv = s->buf[st.in_buf]; a.qkv_stride = s->width[st.in_buf];
            a.z = s->buf[st.in2_buf]; a.z_stride = s->width[st.in2_buf];
            a.beta = s->buf[st.in3_buf]; a.beta_stride = s->width[st.in3_buf];
            a.alpha = s->buf[st.in4_buf]; a.alpha_stride = s->width[st.in4_buf];
            a.conv_weight = L.d1->data; a.dt_bias = L.d2->data; a.norm_weight = L.f1->data; a.a_log = L.f2->data;
            a.conv_seq_stride = s->ssm_conv_layer_elems / d.max_batch;
            a.conv_state = s->ssm_conv + (size_t)st.layer * s->ssm_conv_layer_elems;
            a.state_seq_stride = s->ssm_state_layer_elems / d.max_batch;
            a.state = s->ssm_state + (size_t)st.layer * s->ssm_state_layer_elems;
            a.out = s->buf[st.out_buf]; a.out_stride = s->width[st.out_buf];
            rc = launch_ssm_recurrence(a, stream);
            s->launches += 1;
            break;
        }
        case L_ARGMAX:
            if (plan->ctx->tp_size > 1 && !s->tp_attached) { set_error("tensor-parallel plan: call swlm_tp_export / swlm_tp_attach on the state first"); return SWLM_ERR_STATE; }
            {
                // a vocabulary-sharded output head gives local indices; shift them to global ones
                const int local_n = plan->ctx->tp_size > 1 ? st.n / plan->ctx->tp_size : st.n;
                rc = launch_argmax(m, local_n, s->buf[st.in_buf], s->width[st.in_buf], s->token_out, s->token_in, s->ring,
                                   s->step_counter, s->ring_cap, s->position, 1, s->argmax_val, s->argmax_idx, s->tp,
                                   s->tp_words ? s->tp_words + 3 : nullptr, plan->ctx->tp_rank * local_n, stream);
            }
            s->launches += 2;
            advanced = true;
            break;
        }
        if (rc) return rc;
    }
    if (!advanced && only_kind < 0) {
        rc = launch_advance(m, s->position, nullptr, stream);
        s->launches += 1;
    }
    return rc;
}

int capture_graph(swlm_state* s, bool body_only, cudaGraphExec_t* out) {
    cudaGraph_t graph = nullptr;
    const int64_t before = s->launches;
    SWLM_CUDA(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_step(s, body_only, s->stream);
    cudaError_t e = cudaStreamEndCapture(s->stream, &graph);
    (body_only ? s->graph_body_launches : s->graph_full_launches) = (int)(s->launches - before);
    s->launches = before;  // capture does not execute
    if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture");
    e = cudaGraphInstantiate(out, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
    return SWLM_OK;
}

int launches_per_step(const swlm_plan* plan, bool body_only) {
    int n = 0;
    bool has_argmax = false;
    if (plan->desc.max_batch > kQGemvMaxRows) {
        // more than 16 sequences: the unfused steps, as enqueue_rows issues them
        int converted_buf = -1, converted_k = 0;
        for (const swlm_step& st : plan->steps) {
            const bool head = st.kind == SWLM_STEP_RESADD_RMSNORM || st.kind == SWLM_STEP_ARGMAX ||
                              (st.kind == SWLM_STEP_QGEMV && st.out_buf == SWLM_BUF_LOGITS);
            if (head && body_only) continue;
            if (st.kind == SWLM_STEP_QGEMV) {
                const size_t si = (size_t)(&st - plan->steps.data());
                const Q4Raw* raw = nullptr;
                if (plan->rows_groups_ready) {
                    if (plan->rows_groups[si].count == 0) continue;
                    raw = plan->rows_groups[si].raw;
                } else {
                    auto it = plan->ctx->raw.find(st.weight);
                    if (it != plan->ctx->raw.end()) raw = &it->second;
                }
                if (!raw) continue;
                const bool reuse = converted_buf == st.in_buf && converted_k == raw->k;
                n += qgemm_tc_launch_count(*raw, plan->desc.max_batch, reuse);
                converted_buf = st.in_buf; converted_k = raw->k;
                continue;
            }
            converted_buf = -1;
            n += st.kind == SWLM_STEP_ARGMAX ? 2 : 1;
            has_argmax |= st.kind == SWLM_STEP_ARGMAX;
        }
        return n + (has_argmax ? 0 : 1);
    }
    const size_t end = head_begin_of(plan, body_only);
    for (size_t li = 0; li < end; ++li) {
        const Launch& L = plan->launches[li];
        n += L.kind == L_ARGMAX ? 2 : 1;
        has_argmax |= L.kind == L_ARGMAX;
    }
    if (body_only || !has_argmax) n += 1;
    return n;
}

int run_graph(swlm_state* s, bool body_only) {
    cudaGraphExec_t* g = body_only ? &s->graph_body : &s->graph_full;
    if (!*g) {
        int rc = capture_graph(s, body_only, g);
        if (rc) return rc;
    }
    SWLM_CUDA(cudaGraphLaunch(*g, s->stream));
    s->launches += body_only ? s->graph_body_launches : s->graph_full_launches;
    for (int& p : s->pos_host) p += 1;
    s->steps_host += body_only ? 0 : 1;
    return SWLM_OK;
}

void drop_graphs(swlm_state* s) {
    if (s->graph_full) { cudaGraphExecDestroy(s->graph_full); s->graph_full = nullptr; }
    if (s->graph_body) { cudaGraphExecDestroy(s->graph_body); s->graph_body = nullptr; }
}

struct Region { void* p; size_t bytes; };
std::vector<Region> state_regions(swlm_state* s) {
    const swlm_buffers_desc& d = s->plan->desc;
    std::vector<Region> r;
    for (int i = 0; i < SWLM_BUF_COUNT; ++i) r.push_back({s->buf[i], (size_t)d.max_batch * s->width[i] * 2});
    r.push_back({s->kcache, (size_t)d.kv_layers * s->kv_layer_elems * 2});
    r.push_back({s->vcache, (size_t)d.kv_layers * s->kv_layer_elems * 2});
    r.push_back({s->qjl_res, (size_t)d.kv_layers * s->qjl_layer_elems * 2});
    r.push_back({s->conv, (size_t)d.conv_layers * s->conv_layer_elems * 2});
    r.push_back({s->res2, (size_t)d.max_batch * s->width[SWLM_BUF_RESIDUAL] * 2});
    r.push_back({s->ssm_conv, (size_t)d.ssm_layers * s->ssm_conv_layer_elems * 2});
    r.push_back({s->ssm_state, (size_t)d.ssm_layers * s->ssm_state_layer_elems * 4});
    r.push_back({s->position, (size_t)d.max_batch * 4});
    r.push_back({s->token_in, (size_t)d.max_batch * 4});
    r.push_back({s->token_out, (size_t)d.max_batch * 4});
    return r;
}

// Scratch of the split kernels: attention partials, split-K partial sums and their arrival counters.
// Grown (never shrunk) to what a plan needs; the counters must be zero between launches.
int grow_scratch(swlm_state* s, size_t attn_floats, size_t partial_floats, size_t counters) {
    int rc;
    if (attn_floats > s->attn_scratch_cap) {
        SWLM_CUDA(cudaStreamSynchronize(s->stream));
        cudaFree(s->attn_scratch); s->attn_scratch = nullptr; s->attn_scratch_cap = 0;
        if ((rc = dev_alloc(&s->attn_scratch, attn_floats))) return rc;
        s->attn_scratch_cap = attn_floats;
    }
    if (partial_floats > s->qgemv_partial_cap) {
        SWLM_CUDA(cudaStreamSynchronize(s->stream));
        cudaFree(s->qgemv_partial); s->qgemv_partial = nullptr; s->qgemv_partial_cap = 0;
        if ((rc = dev_alloc(&s->qgemv_partial, partial_floats))) return rc;
        s->qgemv_partial_cap = partial_floats;
    }
    if (counters > s->qgemv_counters_cap) {
        SWLM_CUDA(cudaStreamSynchronize(s->stream));
        cudaFree(s->qgemv_counters); s->qgemv_counters = nullptr; s->qgemv_counters_cap = 0;
        if ((rc = dev_alloc(&s->qgemv_counters, counters))) return rc;
        SWLM_CUDA(cudaMemset(s->qgemv_counters, 0, counters * sizeof(unsigned)));
        s->qgemv_counters_cap = counters;
    }
    return SWLM_OK;
}

size_t plan_attn_scratch(const swlm_plan* plan) {
    size_t need = 0;
    for (const Launch& L : plan->launches)
        if (L.kind == L_ATTN)
            need = std::max(need, attn_scratch_floats(plan->desc.max_batch, L.st.heads / plan->ctx->tp_size, L.st.head_dim, plan->attn_splits));
    return need;
}

// After a synchronisation: did a bounded wait of the tensor-core GEMV give up since the last check?
int check_tc_status(swlm_state* s) {
    if (s->tc_status && *s->tc_status) {
        set_error(*s->tc_status == 21 ? "a bounded wait on another tensor-parallel rank expired (code %d); re-create the state on every rank"
                                      : "a bounded device-side wait expired (code %d)", *s->tc_status);
        *s->tc_status = 0;
        return SWLM_ERR_TIMEOUT;
    }
    return SWLM_OK;
}

int check_position_room(swlm_state* s, int steps) {
    const int furthest = *std::max_element(s->pos_host.begin(), s->pos_host.end());
    if (furthest + steps > s->plan->desc.max_seq) {
        set_error("position %d + %d steps exceeds max_seq %d", furthest, steps, s->plan->desc.max_seq);
        return SWLM_ERR_STATE;
    }
    return SWLM_OK;
}

// ---- prompt ingestion in chunks ---------------------------------------------------------------------
// The reference's prefill runs sequence kernels over the whole prompt (Execution/MetalPrefillExecutor.swift,
// gemm_q4_g64 or dequantise-then-matmul for the products) and replays the decode head for the last position.
// Here all prompt tokens but the last go through the plan's steps, unfused, in chunks of up to
// `prefill_chunk` tokens with one activation row per token: products on the tensor cores (tcgen05), norms and
// SwiGLU row-wise, rope + KV append for the whole chunk, causal attention over the cache, the short-conv
// recurrence walked in order inside one kernel. The last token (and a tail shorter than kPrefillMinChunk)
// takes the decode graph, so the state a decode step sees afterwards is the one it would have produced itself.
constexpr int kPrefillMinChunk = 32;

// can the plan's steps run row-wise (enqueue_rows)?
// The rows of several source-layout tensors one after the other (q | k | v, gate | up), built once per set of names.
int get_raw_cat(swlm_ctx* ctx, const std::vector<std::string>& names, const Q4Raw** out) {
    std::string key = names[0];
    for (size_t i = 1; i < names.size(); ++i) key += "|" + names[i];
    auto hit = ctx->raw_cat.find(key);
    if (hit != ctx->raw_cat.end()) { *out = &hit->second; return SWLM_OK; }
    Q4Raw cat;
    const Q4Raw& first = ctx->raw.at(names[0]);
    cat.k = first.k; cat.sb_f16 = first.sb_f16; cat.shard_kind = first.shard_kind;
    for (const std::string& nm : names) cat.n += ctx->raw.at(nm).n;
    const size_t wpr = (size_t)cat.k / 8, gpr = (size_t)cat.k / 64;
    int rc;
    if ((rc = dev_alloc(&cat.w, (size_t)cat.n * wpr, ctx))) return rc;
    if ((rc = dev_alloc(&cat.scales, (size_t)cat.n * gpr, ctx))) return rc;
    if ((rc = dev_alloc(&cat.biases, (size_t)cat.n * gpr, ctx))) return rc;
    size_t row = 0;
    for (const std::string& nm : names) {
        const Q4Raw& r = ctx->raw.at(nm);
        SWLM_CUDA(cudaMemcpy(cat.w + row * wpr, r.w, (size_t)r.n * wpr * 4, cudaMemcpyDeviceToDevice));
        SWLM_CUDA(cudaMemcpy(cat.scales + row * gpr, r.scales, (size_t)r.n * gpr * 2, cudaMemcpyDeviceToDevice));
        SWLM_CUDA(cudaMemcpy(cat.biases + row * gpr, r.biases, (size_t)r.n * gpr * 2, cudaMemcpyDeviceToDevice));
        row += r.n;
    }
    ctx->raw_cat[key] = cat;
    *out = &ctx->raw_cat[key];
    return SWLM_OK;
}

// Decide which products of the unfused step list run together (allocates: never call while a stream is capturing).
// SWLM_ROWS_FUSE=0 keeps one product per step.
int ensure_rows_groups(swlm_plan* plan) {
    if (plan->rows_groups_ready) return SWLM_OK;
    static const bool fuse = [] { const char* v = getenv("SWLM_ROWS_FUSE"); return !(v && v[0] == '0'); }();
    swlm_ctx* ctx = plan->ctx;
    const std::vector<swlm_step>& st = plan->steps;
    plan->rows_groups.assign(st.size(), swlm_plan::RowsGroup{});
    for (size_t i = 0; i < st.size(); ++i) {
        if (plan->rows_groups[i].count == 0 || st[i].kind != SWLM_STEP_QGEMV) continue;
        auto it = ctx->raw.find(st[i].weight);
        if (it == ctx->raw.end()) { set_error("tensor '%s' not in the weight store", st[i].weight); return SWLM_ERR_NOT_FOUND; }
        const Q4Raw& r0 = it->second;
        plan->rows_groups[i].raw = &r0;
        const bool partial = ctx->tp_size > 1 && r0.shard_kind == SWLM_SHARD_ROW;   // its rows go through an exchange
        if (!fuse || st[i].out_buf == SWLM_BUF_LOGITS || partial) continue;
        std::vector<std::string> names{st[i].weight};
        size_t j = i + 1;
        while (j < st.size() && names.size() < 3 && st[j].kind == SWLM_STEP_QGEMV && st[j].in_buf == st[i].in_buf &&
               st[j].out_buf != st[i].in_buf && st[j].out_buf != SWLM_BUF_LOGITS) {
            auto jt = ctx->raw.find(st[j].weight);
            if (jt == ctx->raw.end()) break;
            const Q4Raw& rj = jt->second;
            if (rj.k != r0.k || rj.sb_f16 != r0.sb_f16 || (ctx->tp_size > 1 && rj.shard_kind == SWLM_SHARD_ROW)) break;
            bool clash = false;
            for (size_t q = i; q < j; ++q) clash |= st[q].out_buf == st[j].out_buf;
            if (clash) break;
            names.push_back(st[j].weight);
            ++j;
        }
        if (names.size() < 2) continue;
        const Q4Raw* cat = nullptr;
        int rc = get_raw_cat(ctx, names, &cat);
        if (rc) return rc;
        plan->rows_groups[i].count = (int)names.size();
        plan->rows_groups[i].raw = cat;
        for (size_t q = i + 1; q < j; ++q) plan->rows_groups[q].count = 0;
    }
    plan->rows_groups_ready = true;
    return SWLM_OK;
}

// Prompt chunks of one sequence under tensor parallelism: up to this many token rows per exchange.
constexpr int kTpChunkRows = 1024;

bool rows_capable(const swlm_plan* plan, bool allow_tp = false) {
    if ((plan->ctx->tp_size != 1 && !allow_tp) || plan->desc.head_dim > 128) return false;
    if (swlm_kv_bits(plan->desc.kv_scheme)) return false;   // prompts over a quantized cache go token by token
    if (plan->ctx->tp_size > 1 && (plan->desc.hidden & 7)) return false;
    for (const swlm_step& st : plan->steps) {
        if (st.kind == SWLM_STEP_QGEMV && st.in_buf == st.out_buf) return false;
        if (st.kind == SWLM_STEP_QGEMV && (st.k & 63)) return false;
        if (st.kind == SWLM_STEP_CONV_STATE_UPDATE && st.conv_kernel > 8) return false;
        if (st.kind == SWLM_STEP_SSM_RECURRENCE && plan->ctx->tp_size > 1) return false;
    }
    return true;
}

bool prefill_batchable(const swlm_plan* plan) { return plan->desc.max_batch == 1 && rows_capable(plan, true); }

int widest_activation(const swlm_state* s) {
    int widest = 0;
    for (int i = 0; i < SWLM_BUF_COUNT; ++i) widest = std::max(widest, s->width[i] * (i == SWLM_BUF_LOGITS ? 0 : 1));
    return widest;
}

int ensure_pf_status(swlm_state* s) {
    if (s->pf_status) return SWLM_OK;
    int rc;
    if ((rc = dev_alloc(&s->pf_status, 1))) return rc;
    SWLM_CUDA(cudaMemset(s->pf_status, 0, sizeof(int)));
    return SWLM_OK;
}

// after a synchronize: did a bounded wait of the tensor-core product expire? Reported once.
int check_pf_status(swlm_state* s) {
    if (!s->pf_status) return SWLM_OK;
    int st = 0;
    SWLM_CUDA(cudaMemcpy(&st, s->pf_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (!st) return SWLM_OK;
    SWLM_CUDA(cudaMemset(s->pf_status, 0, sizeof(int)));
    set_error("a bounded wait in the tensor-core product expired");
    return SWLM_ERR_TIMEOUT;
}

int prefill_workspace(swlm_state* s, int rows) {
    int rc;
    if ((rc = ensure_pf_status(s))) return rc;
    if ((rc = ensure_rows_groups(s->plan))) return rc;
    if (rows <= s->pf_rows) return SWLM_OK;
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    for (int i = 0; i < SWLM_BUF_COUNT; ++i) { cudaFree(s->pf_buf[i]); s->pf_buf[i] = nullptr; }
    cudaFree(s->pf_attn_counters); s->pf_attn_counters = nullptr;
    cudaFree(s->pf_xh); s->pf_xh = nullptr;
    s->pf_rows = 0;
    for (int i = 0; i < SWLM_BUF_COUNT; ++i) {
        if (i == SWLM_BUF_LOGITS) continue;  // the output head never runs on a chunk
        if ((rc = dev_alloc(&s->pf_buf[i], (size_t)rows * s->width[i]))) return rc;
    }
    if ((rc = dev_alloc(&s->pf_xh, qgemm_tc_scratch_bytes(rows, widest_activation(s))))) return rc;
    const size_t n_ctr = (size_t)rows * std::max(1, s->plan->desc.kv_heads);
    if ((rc = dev_alloc(&s->pf_attn_counters, n_ctr))) return rc;
    SWLM_CUDA(cudaMemset(s->pf_attn_counters, 0, n_ctr * sizeof(unsigned)));
    size_t attn_floats = 0;
    for (const swlm_step& st : s->plan->steps)
        if (st.kind == SWLM_STEP_ATTN_DECODE) attn_floats = std::max(attn_floats, attn_scratch_floats(rows, st.heads, st.head_dim, 1));
    if ((rc = grow_scratch(s, attn_floats, 0, 0))) return rc;
    s->pf_rows = rows;
    return SWLM_OK;
}

// The plan's steps, unfused, over `c` activation rows with the products on the tensor cores. Two uses:
//   * chunk (wide == false): the rows are consecutive prompt tokens of sequence `seq` (ids on the device at
//     `tokens`), the first at position pos0; causal attention over that sequence's cache, the short-conv recurrence
//     walked in order. The output head is skipped unless `head_row` >= 0: then the final norm, the output product
//     and argmax run on that one row and the token lands in token_out[seq] / token_in[seq].
//   * wide (wide == true): the rows are the state's sequences (17..kMaxSequences of them) in one decode step, each
//     at its own position: decode attention and the short-conv step per sequence, output head and argmax for all.
int enqueue_rows(swlm_state* s, bool wide, const int32_t* tokens, int c, int pos0, int seq, int head_row, bool body_only,
                 cudaStream_t stream) {
    swlm_plan* plan = s->plan;
    swlm_ctx* ctx = plan->ctx;
    const swlm_buffers_desc& d = plan->desc;
    __nv_bfloat16** pf = wide ? s->buf : s->pf_buf;
    const int* wd = s->width;
    int rc = SWLM_OK;
    const __nv_bfloat16* converted = nullptr;  // rows whose fp16 copy the product scratch still holds
    int converted_k = 0;
    auto product = [&](const Q4Raw& raw, int rows, const __nv_bfloat16* x, int xs, __nv_bfloat16* y, int ys, const TcSegments* seg = nullptr) {
        const bool reuse = converted == x && converted_k == raw.k;
        const int r = launch_qgemm_tc(raw, rows, x, xs, y, ys, wide ? s->wide_xh : s->pf_xh, s->pf_status, stream, reuse, seg);
        converted = x; converted_k = raw.k;
        s->launches += qgemm_tc_launch_count(raw, rows, reuse);
        return r;
    };
    bool advanced = false;
    const int tp = ctx->tp_size;   // > 1 only for prompt chunks: heads, conv channels and the products' rows are this rank's share
    if (!plan->rows_groups_ready) { set_error("row-wise execution was not prepared for this plan"); return SWLM_ERR_STATE; }
    for (size_t si = 0; si < plan->steps.size(); ++si) {
        const swlm_step& st = plan->steps[si];
        const swlm_plan::RowsGroup& grp = plan->rows_groups[si];
        if (grp.count == 0) continue;   // ran with an earlier product
        const bool is_product = st.kind == SWLM_STEP_QGEMV;
        switch (st.kind) {
        case SWLM_STEP_EMBED:
            if (const DenseTensor* table = find_dense(ctx, st.weight))
                rc = launch_embed(c, st.n, tokens, d.vocab, table->data, pf[st.out_buf], wd[st.out_buf], stream);
            else
                rc = launch_embed_q4(c, st.n, tokens, ctx->raw.at(st.weight), pf[st.out_buf], wd[st.out_buf], stream);
            s->launches += 1;
            break;
        case SWLM_STEP_COPY_RMSNORM:
        case SWLM_STEP_RESADD_COPY_RMSNORM:
            rc = launch_rmsnorm(st.kind, c, st.n, pf[st.in_buf], wd[st.in_buf], pf[SWLM_BUF_RESIDUAL], wd[SWLM_BUF_RESIDUAL],
                                find_dense(ctx, st.weight)->data, st.eps, st.weight_bias, pf[st.out_buf], wd[st.out_buf], stream);
            s->launches += 1;
            break;
        case SWLM_STEP_RESADD_RMSNORM: {  // final norm: part of the output head
            if (wide ? body_only : head_row < 0) break;
            const int r0 = wide ? 0 : head_row, rows = wide ? c : 1;
            rc = launch_rmsnorm(st.kind, rows, st.n, pf[st.in_buf] + (size_t)r0 * wd[st.in_buf], wd[st.in_buf],
                                pf[SWLM_BUF_RESIDUAL] + (size_t)r0 * wd[SWLM_BUF_RESIDUAL], wd[SWLM_BUF_RESIDUAL],
                                find_dense(ctx, st.weight)->data, st.eps, st.weight_bias,
                                pf[st.out_buf] + (size_t)r0 * wd[st.out_buf], wd[st.out_buf], stream);
            s->launches += 1;
            break;
        }
        case SWLM_STEP_QGEMV: {
            const Q4Raw& raw = *grp.raw;
            if (grp.count > 1) {
                // q | k | v or gate | up: one product over the concatenated rows, each part to its own buffer
                TcSegments seg;
                seg.count = grp.count;
                int end = 0;
                for (int q = 0; q < grp.count; ++q) {
                    const swlm_step& sq = plan->steps[si + q];
                    end += ctx->raw.at(sq.weight).n;
                    seg.end[q] = end; seg.y[q] = pf[sq.out_buf]; seg.stride[q] = wd[sq.out_buf];
                }
                rc = product(raw, c, pf[st.in_buf], wd[st.in_buf], nullptr, 0, &seg);
                break;
            }
            if (st.out_buf == SWLM_BUF_LOGITS) {
                if (wide ? body_only : head_row < 0) break;
                // the logits buffer belongs to the state (one row per sequence), also for a chunk's last token
                if (wide) rc = product(raw, c, pf[st.in_buf], wd[st.in_buf], s->buf[SWLM_BUF_LOGITS], wd[SWLM_BUF_LOGITS]);
                else rc = product(raw, 1, pf[st.in_buf] + (size_t)head_row * wd[st.in_buf], wd[st.in_buf],
                                  s->buf[SWLM_BUF_LOGITS] + (size_t)seq * wd[SWLM_BUF_LOGITS], wd[SWLM_BUF_LOGITS]);
                break;
            }
            rc = product(raw, c, pf[st.in_buf], wd[st.in_buf], pf[st.out_buf], wd[st.out_buf]);
            if (!rc && tp > 1 && raw.shard_kind == SWLM_SHARD_ROW) {
                // row-parallel weight: the rows are partial sums; add them up across the ranks, in place
                rc = launch_tp_rows_allreduce(s->tp, pf[st.out_buf], wd[st.out_buf], c, raw.n, ++s->tp_rows_epoch,
                                              reinterpret_cast<unsigned*>(s->tp_words + 4), stream);
                s->launches += 2;
                converted = nullptr;
            }
            break;
        }
        case SWLM_STEP_QK_NORM:
            rc = launch_qk_norm(c, st.heads / tp, kv_heads_local(plan), st.head_dim, pf[st.in_buf], wd[st.in_buf], pf[st.in2_buf], wd[st.in2_buf],
                                find_dense(ctx, st.weight)->data, find_dense(ctx, st.weight2)->data, st.eps, st.weight_bias, stream);
            s->launches += 1;
            break;
        case SWLM_STEP_ATTN_DECODE: {
            AttnLaunch a;
            a.m = c; a.heads = st.heads / tp; a.kv_heads = kv_heads_local(plan); a.head_dim = st.head_dim;
            a.rope_dim = st.rope_dim;
            if (st.rope_dim > 0) {
                int ti = -1;
                if ((rc = rope_table_for(plan, st.rope_dim, st.rope_base, &ti))) return rc;
                a.inv_freq = plan->rope_tables[ti].inv_freq;
            }
            a.scale = st.scale; a.window = st.window_left; a.kv_scheme = d.kv_scheme;
            if (swlm_kv_is_rotor(d.kv_scheme)) {   // (only decode steps of many sequences get here with a quantized cache)
                a.rotors = s->rotors + (size_t)st.layer * s->rotor_layer_elems;
                a.qjl_dim = d.kv_qjl_dim; a.qjl_matrix = s->qjl_matrix;
                a.qjl_res = s->qjl_res ? s->qjl_res + (size_t)st.layer * s->qjl_layer_elems : nullptr;
            }
            a.q = pf[st.in_buf]; a.q_stride = wd[st.in_buf];
            a.k = pf[st.in2_buf]; a.k_stride = wd[st.in2_buf];
            a.v = pf[st.in3_buf]; a.v_stride = wd[st.in3_buf];
            const size_t seq_elems = s->kv_layer_elems / d.max_batch;
            a.kcache = s->kcache + (size_t)st.layer * s->kv_layer_elems + (wide ? 0 : (size_t)seq * seq_elems);
            a.vcache = s->vcache + (size_t)st.layer * s->kv_layer_elems + (wide ? 0 : (size_t)seq * seq_elems);
            a.max_seq = d.max_seq; a.position = s->position; a.pos_base = wide ? -1 : pos0;
            a.out = pf[st.out_buf]; a.out_stride = wd[st.out_buf];
            a.scratch = s->attn_scratch;
            a.counters = wide ? s->attn_counters : s->pf_attn_counters;
            a.splits = wide ? plan->attn_splits : 1;
            rc = launch_attn_decode(a, stream);
            s->launches += wide ? 1 : 2;
            break;
        }
        case SWLM_STEP_SWIGLU:
        case SWLM_STEP_GEGLU:
            rc = launch_swiglu(c, st.n / tp, pf[st.in_buf], wd[st.in_buf], pf[st.in2_buf], wd[st.in2_buf], pf[st.out_buf], wd[st.out_buf],
                               st.kind == SWLM_STEP_GEGLU ? GATED_ACT_GELU_TANH : GATED_ACT_SILU, stream);
            s->launches += 1;
            break;
        case SWLM_STEP_CONV_STATE_UPDATE:
            if (wide)
                rc = launch_conv_step(c, st.n, st.conv_kernel, s->conv + (size_t)st.layer * s->conv_layer_elems,
                                      (size_t)d.conv_kernel * d.conv_dim, pf[st.in_buf], wd[st.in_buf], find_dense(ctx, st.weight)->data,
                                      pf[st.out_buf], wd[st.out_buf], stream);
            else
                rc = launch_conv_prefill(c, st.n / tp, st.conv_kernel,
                                         s->conv + (size_t)st.layer * s->conv_layer_elems + (size_t)seq * d.conv_kernel * d.conv_dim,
                                         pf[st.in_buf], wd[st.in_buf], find_dense(ctx, st.weight)->data, pf[st.out_buf], wd[st.out_buf], stream);
            s->launches += 1;
            break;
        case SWLM_STEP_SSM_RECURRENCE: {
            SsmLaunch a;
            a.m = wide ? c : 1; a.tokens = wide ? 1 : c;
            a.heads = st.heads; a.groups = std::max(1, st.groups); a.key_dim = st.key_dim; a.value_dim = st.value_dim; a.kernel = st.conv_kernel;
            a.qkv = pf[st.in_buf]; a.qkv_stride = wd[st.in_buf];
            a.z = pf[st.in2_buf]; a.z_stride = wd[st.in2_buf];
            a.beta = pf[st.in3_buf]; a.beta_stride = wd[st.in3_buf];
            a.alpha = pf[st.in4_buf]; a.alpha_stride = wd[st.in4_buf];
            a.conv_weight = find_dense(ctx, st.weight)->data; a.dt_bias = find_dense(ctx, st.weight3)->data;
            a.norm_weight = ctx->densef.at(st.weight2).data; a.a_log = ctx->densef.at(st.weight4).data;
            a.conv_seq_stride = s->ssm_conv_layer_elems / d.max_batch;
            a.state_seq_stride = s->ssm_state_layer_elems / d.max_batch;
            // a chunk belongs to one sequence: its slabs; a decode step of many sequences: all slabs
            a.conv_state = s->ssm_conv + (size_t)st.layer * s->ssm_conv_layer_elems + (wide ? 0 : (size_t)seq * a.conv_seq_stride);
            a.state = s->ssm_state + (size_t)st.layer * s->ssm_state_layer_elems + (wide ? 0 : (size_t)seq * a.state_seq_stride);
            a.out = pf[st.out_buf]; a.out_stride = wd[st.out_buf];
            rc = launch_ssm_recurrence(a, stream);
            s->launches += 1;
            break;
        }
        case SWLM_STEP_ARGMAX:
            if (wide ? body_only : head_row < 0) break;
            if (wide) {
                rc = launch_argmax(c, st.n, s->buf[st.in_buf], wd[st.in_buf], s->token_out, s->token_in, s->ring, s->step_counter,
                                   s->ring_cap, s->position, 1, s->argmax_val, s->argmax_idx, s->tp, nullptr, 0, stream);
                advanced = true;
            } else {
                rc = launch_argmax(1, st.n, s->buf[st.in_buf] + (size_t)seq * wd[st.in_buf], wd[st.in_buf], s->token_out + seq,
                                   s->token_in + seq, nullptr, s->step_counter, s->ring_cap, s->position, 0, s->argmax_val,
                                   s->argmax_idx, s->tp, nullptr, 0, stream);
            }
            s->launches += 2;
            break;
        default:
            set_error("row-wise plan: step kind %d", st.kind);
            return SWLM_ERR_UNSUPPORTED;
        }
        if (rc) return rc;
        if (!is_product) converted = nullptr;
    }
    if (wide) {
        if (!advanced) { rc = launch_advance(c, s->position, nullptr, stream); s->launches += 1; }
    } else {
        rc = launch_fill_u32(reinterpret_cast<uint32_t*>(s->position + seq), 1, (uint32_t)(pos0 + c), stream);
        s->launches += 1;
    }
    return rc;
}

int enqueue_prefill_chunk(swlm_state* s, const int32_t* tokens, int c, int pos0, int seq, cudaStream_t stream, int head_row = -1) {
    return enqueue_rows(s, false, tokens, c, pos0, seq, head_row, false, stream);
}

}  // namespace

// =====================================================================================================
// C ABI
// =====================================================================================================
extern "C" {

const char* swlm_version(void) { return "swlm-cuda 0.1 (sm_100a)"; }
const char* swlm_last_error(void) { return g_error; }

int swlm_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

int swlm_ctx_create(int device_id, int tp_rank, int tp_size, swlm_ctx** out) {
    if (!out) { set_error("null out"); return SWLM_ERR_INVALID; }
    *out = nullptr;
    if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) { set_error("bad tp rank/size %d/%d", tp_rank, tp_size); return SWLM_ERR_INVALID; }
    int n = swlm_device_count();
    if (n <= 0) { set_error("no CUDA device: this library has no CPU path"); return SWLM_ERR_CUDA; }
    if (device_id < 0 || device_id >= n) { set_error("device %d of %d", device_id, n); return SWLM_ERR_INVALID; }
    SWLM_CUDA(cudaSetDevice(device_id));
    cudaDeviceProp prop;
    SWLM_CUDA(cudaGetDeviceProperties(&prop, device_id));
    if (prop.major != 10) { set_error("device %d is sm_%d%d; this library is built for sm_100a only", device_id, prop.major, prop.minor); return SWLM_ERR_UNSUPPORTED; }
    swlm_ctx* ctx = new swlm_ctx();
    ctx->device = device_id; ctx->tp_rank = tp_rank; ctx->tp_size = tp_size;
    cudaError_t e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete ctx; return cuda_fail(e, "cudaStreamCreate"); }
    int rc = qgemv_init();
    if (!rc) rc = attn_init();
    if (!rc) rc = qgemm_tc_init();
    if (rc) { cudaStreamDestroy(ctx->stream); delete ctx; return rc; }
    *out = ctx;
    return SWLM_OK;
}

void swlm_ctx_destroy(swlm_ctx* ctx) {
    if (!ctx) return;
    if (ctx->users > 0) { ctx->destroy_requested = true; return; }
    qgemv_trace_report();
    cudaSetDevice(ctx->device);
    for (auto& kv : ctx->raw) { cudaFree(kv.second.w); cudaFree(kv.second.scales); cudaFree(kv.second.biases); }
    for (auto& kv : ctx->tiled) { cudaFree(kv.second.tiles); cudaFree(kv.second.sb); }
    for (auto& kv : ctx->raw_cat) { cudaFree(kv.second.w); cudaFree(kv.second.scales); cudaFree(kv.second.biases); }
    for (auto& kv : ctx->dense) cudaFree(kv.second.data);
    for (auto& kv : ctx->densef) cudaFree(kv.second.data);
    cudaFree(ctx->op_partial);
    cudaFree(ctx->tc_status);
    cudaFree(ctx->op_xh);
    cudaFree(ctx->op_counters);
    cudaFree(ctx->op_attn_counters);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

int swlm_weights_add_q4g64_mlx(swlm_ctx* ctx, const char* name, int n, int k, const uint32_t* weight,
                               const uint16_t* scales_bf16, const uint16_t* biases_bf16, int shard_kind) {
    return add_q4_raw(ctx, name, n, k, weight, scales_bf16, biases_bf16, false, shard_kind);
}

int swlm_weights_add_q4g64_staf(swlm_ctx* ctx, const char* name, int n, int k, const void* blocks36, int shard_kind) {
    if (!ctx || !name || !blocks36 || n <= 0 || k <= 0 || k % 64) { set_error("bad STAF tensor"); return SWLM_ERR_INVALID; }
    // De-interleave the 36-byte blocks into the three planes of the source layout; the payload bytes are
    // the same LSB-first stream (Sources/MetalCompiler/STAF/STAFPayloadConverter.swift:268-274), and the
    // fp16 scale/zero bits are kept as they are.
    const int groups = k / 64;
    std::vector<uint32_t> w((size_t)n * (k / 8));
    std::vector<uint16_t> s((size_t)n * groups), z((size_t)n * groups);
    const uint8_t* src = static_cast<const uint8_t*>(blocks36);
    for (size_t g = 0; g < (size_t)n * groups; ++g) {
        const uint8_t* blk = src + g * 36;
        memcpy(&s[g], blk, 2);
        memcpy(&z[g], blk + 2, 2);
        memcpy(reinterpret_cast<uint8_t*>(w.data()) + g * 32, blk + 4, 32);
    }
    return add_q4_raw(ctx, name, n, k, w.data(), s.data(), z.data(), true, shard_kind);
}

int swlm_weights_add_q4g128_mlx(swlm_ctx* ctx, const char* name, int n, int k, const uint32_t* weight,
                                const uint16_t* scales_bf16, const uint16_t* biases_bf16, int shard_kind) {
    if (!ctx || !name || !weight || !scales_bf16 || !biases_bf16 || n <= 0 || k <= 0 || k % 128) { set_error("q4g128 tensor: k must be a positive multiple of 128"); return SWLM_ERR_INVALID; }
    // every (scale, bias) pair serves both 64-weight halves of its group
    const size_t g128 = (size_t)n * (k / 128);
    std::vector<uint16_t> s(2 * g128), z(2 * g128);
    for (size_t g = 0; g < g128; ++g) { s[2 * g] = s[2 * g + 1] = scales_bf16[g]; z[2 * g] = z[2 * g + 1] = biases_bf16[g]; }
    return add_q4_raw(ctx, name, n, k, weight, s.data(), z.data(), false, shard_kind);
}

int swlm_weights_add_q4g128_staf(swlm_ctx* ctx, const char* name, int n, int k, const void* blocks68, int shard_kind) {
    if (!ctx || !name || !blocks68 || n <= 0 || k <= 0 || k % 128) { set_error("bad STAF tensor"); return SWLM_ERR_INVALID; }
    const size_t g128 = (size_t)n * (k / 128);
    std::vector<uint32_t> w((size_t)n * (k / 8));
    std::vector<uint16_t> s(2 * g128), z(2 * g128);
    const uint8_t* src = static_cast<const uint8_t*>(blocks68);
    for (size_t g = 0; g < g128; ++g) {
        const uint8_t* blk = src + g * 68;
        memcpy(&s[2 * g], blk, 2); s[2 * g + 1] = s[2 * g];
        memcpy(&z[2 * g], blk + 2, 2); z[2 * g + 1] = z[2 * g];
        memcpy(reinterpret_cast<uint8_t*>(w.data()) + g * 64, blk + 4, 64);
    }
    return add_q4_raw(ctx, name, n, k, w.data(), s.data(), z.data(), true, shard_kind);
}

int swlm_weights_add_dense_bf16(swlm_ctx* ctx, const char* name, int64_t rows, int64_t cols, const uint16_t* data,
                                int shard_kind) {
    if (!ctx || !name || !data || rows <= 0 || cols <= 0) { set_error("bad dense tensor"); return SWLM_ERR_INVALID; }
    int rc = ensure_device(ctx);
    if (rc) return rc;
    Slice sl;
    rc = shard_slice(ctx, shard_kind == SWLM_SHARD_ROW ? SWLM_SHARD_REPLICATE : shard_kind, (int)rows, (int)cols, &sl);
    if (rc) return rc;
    if (sl.parts != 1) { set_error("dense tensors are replicated or split by rows"); return SWLM_ERR_UNSUPPORTED; }
    auto old = ctx->dense.find(name);
    if (old != ctx->dense.end()) {
        SWLM_CUDA(cudaDeviceSynchronize());
        cudaFree(old->second.data);
        ctx->dense.erase(old);
    }
    DenseTensor t;
    t.rows = sl.rows; t.cols = cols; t.shard_kind = shard_kind;
    if ((rc = dev_alloc(&t.data, (size_t)t.rows * cols, ctx))) return rc;
    SWLM_CUDA(cudaMemcpy(t.data, data + (size_t)sl.row0 * cols, (size_t)t.rows * cols * 2, cudaMemcpyHostToDevice));
    ctx->dense[name] = t;
    return SWLM_OK;
}

int swlm_weights_add_dense_f32(swlm_ctx* ctx, const char* name, int64_t count, const float* data) {
    if (!ctx || !name || !data || count <= 0) { set_error("bad fp32 tensor"); return SWLM_ERR_INVALID; }
    int rc = ensure_device(ctx);
    if (rc) return rc;
    auto old = ctx->densef.find(name);
    if (old != ctx->densef.end()) {
        SWLM_CUDA(cudaDeviceSynchronize());
        cudaFree(old->second.data);
        ctx->densef.erase(old);
    }
    DenseF32 t;
    t.count = count;
    if ((rc = dev_alloc(&t.data, (size_t)count, ctx))) return rc;
    SWLM_CUDA(cudaMemcpy(t.data, data, (size_t)count * 4, cudaMemcpyHostToDevice));
    ctx->densef[name] = t;
    return SWLM_OK;
}

int64_t swlm_weights_bytes(const swlm_ctx* ctx) { return ctx ? ctx->bytes : 0; }

int swlm_plan_build(swlm_ctx* ctx, const swlm_step* steps, int n_steps, const swlm_buffers_desc* desc, swlm_plan** out) {
    if (!ctx || !steps || n_steps <= 0 || !desc || !out) { set_error("null argument"); return SWLM_ERR_INVALID; }
    *out = nullptr;
    if (!swlm_kv_scheme_supported(desc->kv_scheme)) {
        set_error("KV cache scheme %#x not supported (0x01 bf16; 0x10 / 0x11 / 0x12 8-bit groups of 32 / 64 / 128; 0x40 / 0x41 / 0x42 4-bit groups of 64 / 128 / 128; 0x70 / 0x71 rotated 8-bit groups of 32 / 4-bit groups of 64)", desc->kv_scheme);
        return SWLM_ERR_UNSUPPORTED;
    }
    if (desc->kv_qjl_dim < 0 || desc->kv_qjl_dim > 64 || (desc->kv_qjl_dim > 0 && !swlm_kv_is_rotor(desc->kv_scheme))) {
        set_error("kv_qjl_dim %d: 0..64, and only with a rotated KV scheme", desc->kv_qjl_dim);
        return SWLM_ERR_INVALID;
    }
    if (swlm_kv_is_rotor(desc->kv_scheme) && ctx->tp_size > 1) {
        set_error("rotated KV schemes are not supported under tensor parallelism");
        return SWLM_ERR_UNSUPPORTED;
    }
    if (swlm_kv_bits(desc->kv_scheme) && desc->kv_layers > 0 &&
        ((desc->head_dim != 64 && desc->head_dim != 128) || swlm_kv_group(desc->kv_scheme) > desc->head_dim)) {
        set_error("a quantized KV cache needs head_dim 64 or 128 and groups no wider than head_dim");
        return SWLM_ERR_UNSUPPORTED;
    }
    if (desc->max_batch < 1 || desc->max_batch > kMaxSequences) { set_error("max_batch %d outside 1..%d", desc->max_batch, kMaxSequences); return SWLM_ERR_INVALID; }
    if (desc->max_batch > kQGemvMaxRows && ctx->tp_size > 1) { set_error("more than %d sequences per step are not supported under tensor parallelism", kQGemvMaxRows); return SWLM_ERR_UNSUPPORTED; }
    if (desc->hidden % 8 || desc->slot_dim % 8 || desc->vocab % 8) { set_error("hidden, slot_dim and vocab must be multiples of 8"); return SWLM_ERR_INVALID; }
    int rc = ensure_device(ctx);
    if (rc) return rc;
    swlm_plan* plan = new swlm_plan();
    plan->ctx = ctx;
    ctx->users += 1;
    plan->desc = *desc;
    plan->steps.assign(steps, steps + n_steps);
    rc = compile_plan(plan);
    // Row-wise execution (prompt chunks; more than 16 sequences, inside a CUDA graph): build the concatenated tensors
    // now, not inside the first prompt's latency and not while a stream is capturing.
    if (!rc && (desc->max_batch > kQGemvMaxRows || rows_capable(plan, true))) rc = ensure_rows_groups(plan);
    if (rc) { swlm_plan_destroy(plan); return rc; }
    plan->attn_scratch = plan_attn_scratch(plan);
    *out = plan;
    return SWLM_OK;
}

void swlm_plan_destroy(swlm_plan* plan) {
    if (!plan) return;
    if (plan->users > 0) { plan->destroy_requested = true; return; }
    swlm_ctx* ctx = plan->ctx;
    cudaSetDevice(ctx->device);
    for (RopeTable& t : plan->rope_tables) cudaFree(t.inv_freq);
    delete plan;
    ctx->users -= 1;
    if (ctx->users == 0 && ctx->destroy_requested) swlm_ctx_destroy(ctx);
}

int swlm_plan_launch_count(const swlm_plan* plan) { return plan ? launches_per_step(plan, false) : 0; }

int swlm_plan_describe(const swlm_plan* plan, char* dst, int cap) {
    if (!plan) return 0;
    std::string s;
    char line[256];
    for (size_t i = 0; i < plan->launches.size(); ++i) {
        const Launch& L = plan->launches[i];
        snprintf(line, sizeof(line), "%3zu %-60s steps=%d\n", i, L.label.c_str(), L.steps_covered);
        s += line;
    }
    if (dst && cap > 0) {
        const size_t c = std::min((size_t)cap - 1, s.size());
        memcpy(dst, s.data(), c);
        dst[c] = 0;
    }
    return (int)s.size() + 1;
}

int swlm_state_create(swlm_plan* plan, swlm_state** out) {
    if (!plan || !out) { set_error("null argument"); return SWLM_ERR_INVALID; }
    *out = nullptr;
    int rc = ensure_device(plan->ctx);
    if (rc) return rc;
    const swlm_buffers_desc& d = plan->desc;
    swlm_state* s = new swlm_state();
    s->plan = plan;
    plan->users += 1;
    auto fail = [&](int code) { swlm_state_destroy(s); return code; };
    cudaError_t e = cudaStreamCreateWithFlags(&s->own_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return fail(cuda_fail(e, "cudaStreamCreate"));
    s->stream = s->own_stream;
    for (int i = 0; i < SWLM_BUF_COUNT; ++i) {
        s->width[i] = buf_width(d, i);
        if ((rc = dev_alloc(&s->buf[i], (size_t)d.max_batch * s->width[i]))) return fail(rc);
    }
    // (counted in 2-byte units whatever the scheme: an 8-bit row of head_dim values is head_dim / 32 blocks of 36 bytes)
    s->kv_layer_elems = (size_t)d.max_batch * kv_heads_local(plan) * d.max_seq * kv_row_bytes(d) / 2;
    if ((rc = dev_alloc(&s->kcache, (size_t)d.kv_layers * s->kv_layer_elems))) return fail(rc);
    if ((rc = dev_alloc(&s->vcache, (size_t)d.kv_layers * s->kv_layer_elems))) return fail(rc);
    if (swlm_kv_is_rotor(d.kv_scheme) && d.kv_layers > 0) {
        // rotors and projection matrix by the reference's deterministic rule (initializeRandomUnitRotors /
        // initializeRademacherMatrix, Buffer/MetalGraphAllocator.swift:349-411)
        const int groups = swlm_kv_rotor_groups(d.head_dim);
        s->rotor_layer_elems = (size_t)d.kv_heads * groups * 4;
        kv_rotor_init_host(d.kv_layers, d.kv_heads, groups, &s->rotors_host);
        if ((rc = dev_alloc(&s->rotors, s->rotors_host.size()))) return fail(rc);
        cudaError_t ce = cudaMemcpy(s->rotors, s->rotors_host.data(), s->rotors_host.size() * 2, cudaMemcpyHostToDevice);
        if (ce != cudaSuccess) return fail(cuda_fail(ce, "cudaMemcpy(rotors)"));
        if (d.kv_qjl_dim > 0) {
            kv_qjl_matrix_init_host(d.head_dim, d.kv_qjl_dim, &s->qjl_matrix_host);
            if ((rc = dev_alloc(&s->qjl_matrix, s->qjl_matrix_host.size()))) return fail(rc);
            ce = cudaMemcpy(s->qjl_matrix, s->qjl_matrix_host.data(), s->qjl_matrix_host.size() * 2, cudaMemcpyHostToDevice);
            if (ce != cudaSuccess) return fail(cuda_fail(ce, "cudaMemcpy(projection matrix)"));
            s->qjl_layer_elems = (size_t)d.max_batch * d.kv_heads * d.max_seq * d.kv_qjl_dim;
            if ((rc = dev_alloc(&s->qjl_res, (size_t)d.kv_layers * s->qjl_layer_elems))) return fail(rc);
            ce = cudaMemset(s->qjl_res, 0, (size_t)d.kv_layers * s->qjl_layer_elems * 2);
            if (ce != cudaSuccess) return fail(cuda_fail(ce, "cudaMemset(residual rows)"));
        }
    }
    s->conv_layer_elems = (size_t)d.max_batch * d.conv_kernel * d.conv_dim;
    if ((rc = dev_alloc(&s->conv, (size_t)d.conv_layers * s->conv_layer_elems))) return fail(rc);
    if ((rc = dev_alloc(&s->res2, (size_t)d.max_batch * s->width[SWLM_BUF_RESIDUAL]))) return fail(rc);
    if (d.ssm_layers > 0) {
        const size_t ssm_conv_dim = (size_t)2 * std::max(1, d.ssm_groups) * d.ssm_key_dim + (size_t)d.ssm_heads * d.ssm_value_dim;
        s->ssm_conv_layer_elems = (size_t)d.max_batch * d.ssm_conv_kernel * ssm_conv_dim;
        s->ssm_state_layer_elems = (size_t)d.max_batch * d.ssm_heads * d.ssm_key_dim * d.ssm_value_dim;
        if ((rc = dev_alloc(&s->ssm_conv, (size_t)d.ssm_layers * s->ssm_conv_layer_elems))) return fail(rc);
        if ((rc = dev_alloc(&s->ssm_state, (size_t)d.ssm_layers * s->ssm_state_layer_elems))) return fail(rc);
    }
    if ((rc = dev_alloc(&s->position, d.max_batch))) return fail(rc);
    s->pos_host.assign(d.max_batch, 0);
    if ((rc = dev_alloc(&s->step_counter, 1))) return fail(rc);
    if ((rc = dev_alloc(&s->token_in, d.max_batch))) return fail(rc);
    if ((rc = dev_alloc(&s->token_out, d.max_batch))) return fail(rc);
    if ((rc = dev_alloc(&s->ring, (size_t)s->ring_cap * d.max_batch))) return fail(rc);
    if ((rc = grow_scratch(s, plan->attn_scratch, plan->qgemv_partial, plan->qgemv_counters))) return fail(rc);
    if ((rc = dev_alloc(&s->attn_counters, (size_t)d.max_batch * std::max(1, d.kv_heads)))) return fail(rc);
    {
        cudaError_t ce = cudaMemset(s->attn_counters, 0, (size_t)d.max_batch * std::max(1, d.kv_heads) * sizeof(unsigned));
        if (ce != cudaSuccess) return fail(cuda_fail(ce, "cudaMemset"));
    }
    if (d.max_batch > kQGemvMaxRows) {
        if ((rc = ensure_pf_status(s))) return fail(rc);
        if ((rc = dev_alloc(&s->wide_xh, qgemm_tc_scratch_bytes(d.max_batch, widest_activation(s))))) return fail(rc);
    }
    if ((rc = dev_alloc(&s->argmax_val, argmax_scratch_elems(d.max_batch)))) return fail(rc);
    if ((rc = dev_alloc(&s->argmax_idx, argmax_scratch_elems(d.max_batch)))) return fail(rc);
    e = cudaMallocHost((void**)&s->h_tok, sizeof(int32_t) * 2 * d.max_batch);
    if (e != cudaSuccess) return fail(cuda_fail(e, "cudaMallocHost"));
    // pinned and mapped: the kernels write it only when a wait expires, the host reads it after every sync for free
    e = cudaHostAlloc((void**)&s->tc_status, sizeof(int), cudaHostAllocMapped);
    if (e != cudaSuccess) return fail(cuda_fail(e, "cudaHostAlloc"));
    *s->tc_status = 0;
    *out = s;
    rc = swlm_state_reset(s);
    if (rc) { *out = nullptr; return fail(rc); }
    return SWLM_OK;
}

void swlm_state_destroy(swlm_state* s) {
    if (!s) return;
    cudaSetDevice(s->plan->ctx->device);
    if (s->stream) cudaStreamSynchronize(s->stream);
    drop_graphs(s);
    for (int i = 0; i < SWLM_BUF_COUNT; ++i) cudaFree(s->buf[i]);
    cudaFree(s->kcache); cudaFree(s->vcache); cudaFree(s->conv); cudaFree(s->res2);
    cudaFree(s->rotors); cudaFree(s->qjl_matrix); cudaFree(s->qjl_res);
    cudaFree(s->ssm_conv); cudaFree(s->ssm_state);
    if (s->tp.tp > 1) {
        for (int r = 0; r < s->tp.tp; ++r)
            if (r != s->tp.rank && s->tp_attached && s->tp.peer[r]) cudaIpcCloseMemHandle(s->tp.peer[r]);
        cudaFree(s->tp.peer[s->tp.rank]);
    }
    cudaFree(s->tp_words);
    cudaFree(s->position); cudaFree(s->step_counter); cudaFree(s->token_in); cudaFree(s->token_out); cudaFree(s->ring);
    cudaFree(s->prompt);
    cudaFree(s->attn_scratch); cudaFree(s->qgemv_partial); cudaFree(s->qgemv_counters); cudaFree(s->attn_counters);
    cudaFree(s->argmax_val); cudaFree(s->argmax_idx);
    for (int i = 0; i < SWLM_BUF_COUNT; ++i) cudaFree(s->pf_buf[i]);
    cudaFree(s->pf_attn_counters); cudaFree(s->pf_status); cudaFree(s->pf_xh); cudaFree(s->wide_xh);
    if (s->h_tok) cudaFreeHost(s->h_tok);
    if (s->tc_status) cudaFreeHost(s->tc_status);
    if (s->own_stream) cudaStreamDestroy(s->own_stream);
    swlm_plan* plan = s->plan;
    delete s;
    plan->users -= 1;
    if (plan->users == 0 && plan->destroy_requested) swlm_plan_destroy(plan);
}

int swlm_state_set_stream(swlm_state* s, void* cuda_stream) {
    if (!s) { set_error("null state"); return SWLM_ERR_INVALID; }
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    s->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : s->own_stream;
    return SWLM_OK;
}

int swlm_state_reset(swlm_state* s) {
    if (!s) { set_error("null state"); return SWLM_ERR_INVALID; }
    int rc = ensure_device(s->plan->ctx);
    if (rc) return rc;
    for (const Region& r : state_regions(s))
        if (r.bytes) SWLM_CUDA(cudaMemsetAsync(r.p, 0, r.bytes, s->stream));
    SWLM_CUDA(cudaMemsetAsync(s->step_counter, 0, 4, s->stream));
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    std::fill(s->pos_host.begin(), s->pos_host.end(), 0);
    s->steps_host = 0;
    return SWLM_OK;
}

int swlm_state_snapshot(swlm_state* s, swlm_snap** out) {
    if (!s || !out) { set_error("null argument"); return SWLM_ERR_INVALID; }
    *out = nullptr;
    int rc = ensure_device(s->plan->ctx);
    if (rc) return rc;
    swlm_snap* snap = new swlm_snap();
    for (const Region& r : state_regions(s)) {
        void* p = nullptr;
        if (r.bytes) {
            cudaError_t e = cudaMalloc(&p, r.bytes);
            if (e != cudaSuccess) { swlm_snap_destroy(snap); return cuda_fail(e, "cudaMalloc(snapshot)"); }
            e = cudaMemcpyAsync(p, r.p, r.bytes, cudaMemcpyDeviceToDevice, s->stream);
            if (e != cudaSuccess) { cudaFree(p); swlm_snap_destroy(snap); return cuda_fail(e, "cudaMemcpyAsync(snapshot)"); }
        }
        snap->dev.push_back(p);
        snap->bytes.push_back(r.bytes);
    }
    snap->pos_host = s->pos_host;
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    *out = snap;
    return SWLM_OK;
}

int swlm_state_restore(swlm_state* s, const swlm_snap* snap) {
    if (!s || !snap) { set_error("null argument"); return SWLM_ERR_INVALID; }
    std::vector<Region> regions = state_regions(s);
    if (regions.size() != snap->dev.size()) { set_error("snapshot belongs to another plan"); return SWLM_ERR_STATE; }
    for (size_t i = 0; i < regions.size(); ++i) {
        if (regions[i].bytes != snap->bytes[i]) { set_error("snapshot belongs to another plan"); return SWLM_ERR_STATE; }
        if (regions[i].bytes) SWLM_CUDA(cudaMemcpyAsync(regions[i].p, snap->dev[i], regions[i].bytes, cudaMemcpyDeviceToDevice, s->stream));
    }
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    s->pos_host = snap->pos_host;
    return SWLM_OK;
}

void swlm_snap_destroy(swlm_snap* snap) {
    if (!snap) return;
    for (void* p : snap->dev) cudaFree(p);
    delete snap;
}

int swlm_position(const swlm_state* s) { return s ? s->pos_host[0] : -1; }

int swlm_set_position(swlm_state* s, int position) {
    if (!s || position < 0 || position > s->plan->desc.max_seq) { set_error("bad position"); return SWLM_ERR_INVALID; }
    std::vector<int32_t> all(s->plan->desc.max_batch, position);
    return swlm_set_positions(s, all.data());
}

int swlm_set_positions(swlm_state* s, const int32_t* positions) {
    if (!s || !positions) { set_error("null argument"); return SWLM_ERR_INVALID; }
    const int m = s->plan->desc.max_batch;
    for (int b = 0; b < m; ++b)
        if (positions[b] < 0 || positions[b] > s->plan->desc.max_seq) { set_error("bad position %d of sequence %d", positions[b], b); return SWLM_ERR_INVALID; }
    SWLM_CUDA(cudaMemcpyAsync(s->position, positions, sizeof(int32_t) * m, cudaMemcpyHostToDevice, s->stream));
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    s->pos_host.assign(positions, positions + m);
    return SWLM_OK;
}

int swlm_get_positions(const swlm_state* s, int32_t* positions) {
    if (!s || !positions) { set_error("null argument"); return SWLM_ERR_INVALID; }
    std::copy(s->pos_host.begin(), s->pos_host.end(), positions);
    return SWLM_OK;
}

int swlm_sync(swlm_state* s) {
    if (!s) { set_error("null state"); return SWLM_ERR_INVALID; }
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    return check_tc_status(s);
}

int swlm_decode(swlm_state* s, const int32_t* token_in, int32_t* token_out) {
    if (!s || !token_in || !token_out) { set_error("null argument"); return SWLM_ERR_INVALID; }
    const int m = s->plan->desc.max_batch;
    for (int b = 0; b < m; ++b) token_out[b] = -1;
    int rc = ensure_device(s->plan->ctx);
    if (!rc) rc = check_position_room(s, 1);
    if (rc) return rc;
    memcpy(s->h_tok, token_in, sizeof(int32_t) * m);
    SWLM_CUDA(cudaMemcpyAsync(s->token_in, s->h_tok, sizeof(int32_t) * m, cudaMemcpyHostToDevice, s->stream));
    rc = run_graph(s, false);
    if (rc) return rc;
    SWLM_CUDA(cudaMemcpyAsync(s->h_tok + m, s->token_out, sizeof(int32_t) * m, cudaMemcpyDeviceToHost, s->stream));
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    memcpy(token_out, s->h_tok + m, sizeof(int32_t) * m);
    rc = check_tc_status(s);
    if (!rc) rc = check_pf_status(s);
    if (rc) for (int b = 0; b < m; ++b) token_out[b] = -1;
    return rc;
}

int swlm_decode_n_async(swlm_state* s, const int32_t* token_in, int n) {
    if (!s || n < 0) { set_error("bad argument"); return SWLM_ERR_INVALID; }
    const int m = s->plan->desc.max_batch;
    int rc = ensure_device(s->plan->ctx);
    if (!rc) rc = check_position_room(s, n);
    if (rc) return rc;
    if (n > s->ring_cap) { set_error("decode_n: n=%d exceeds the token ring (%d)", n, s->ring_cap); return SWLM_ERR_INVALID; }
    if (token_in) {
        memcpy(s->h_tok, token_in, sizeof(int32_t) * m);
        SWLM_CUDA(cudaMemcpyAsync(s->token_in, s->h_tok, sizeof(int32_t) * m, cudaMemcpyHostToDevice, s->stream));
    }
    for (int i = 0; i < n; ++i) {
        rc = run_graph(s, false);
        if (rc) return rc;
    }
    return SWLM_OK;
}

int swlm_read_tokens(swlm_state* s, int n, int32_t* tokens_out) {
    if (!s || !tokens_out || n < 0 || n > s->ring_cap) { set_error("bad argument"); return SWLM_ERR_INVALID; }
    const int m = s->plan->desc.max_batch;
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    // the last n steps occupy ring slots (steps-n .. steps-1) mod ring_cap
    for (int i = 0; i < n; ++i) {
        const long long step = s->steps_host - n + i;
        if (step < 0) { set_error("fewer than %d steps decoded", n); return SWLM_ERR_STATE; }
        SWLM_CUDA(cudaMemcpy(tokens_out + (size_t)i * m, s->ring + (size_t)(step % s->ring_cap) * m, sizeof(int32_t) * m, cudaMemcpyDeviceToHost));
    }
    int rc = check_tc_status(s);
    if (!rc) rc = check_pf_status(s);
    if (rc) for (size_t i = 0; i < (size_t)n * m; ++i) tokens_out[i] = -1;
    return rc;
}

int swlm_decode_n(swlm_state* s, const int32_t* token_in, int n, int32_t* tokens_out) {
    if (!tokens_out) { set_error("null argument"); return SWLM_ERR_INVALID; }
    int rc = swlm_decode_n_async(s, token_in, n);
    if (rc) return rc;
    return swlm_read_tokens(s, n, tokens_out);
}

int swlm_prefill(swlm_state* s, const int32_t* tokens, int n, int32_t* first_token) {
    if (!s || !tokens || !first_token || n <= 0) { set_error("bad argument"); return SWLM_ERR_INVALID; }
    const int m = s->plan->desc.max_batch;
    for (int b = 0; b < m; ++b) first_token[b] = -1;
    int rc = ensure_device(s->plan->ctx);
    if (!rc) rc = check_position_room(s, n);
    if (rc) return rc;
    // several sequences with prompts long enough for chunks: one sequence after the other through the row-wise path
    if (m > 1 && n >= kPrefillMinChunk && s->prefill_chunk >= kPrefillMinChunk && rows_capable(s->plan)) {
        for (int b = 0; b < m; ++b)
            if ((rc = swlm_prefill_seq(s, b, tokens + (size_t)b * n, n, first_token + b))) {
                for (int q = 0; q < m; ++q) first_token[q] = -1;
                return rc;
            }
        return SWLM_OK;
    }
    // token-major copy of the prompt so that step t reads m consecutive ids
    std::vector<int32_t> tm((size_t)n * m);
    for (int b = 0; b < m; ++b)
        for (int t = 0; t < n; ++t) tm[(size_t)t * m + b] = tokens[(size_t)b * n + t];
    if (s->prompt_cap < tm.size()) {
        cudaFree(s->prompt);
        s->prompt = nullptr; s->prompt_cap = 0;
        if ((rc = dev_alloc(&s->prompt, tm.size()))) return rc;
        s->prompt_cap = tm.size();
    }
    SWLM_CUDA(cudaMemcpyAsync(s->prompt, tm.data(), tm.size() * 4, cudaMemcpyHostToDevice, s->stream));
    // Every prompt token runs the layer stack; only the last one runs the output head, as the reference's
    // prefill replays the decode plan's lm_head + argmax for the final position
    // (Execution/MetalPrefillExecutor.swift:1320-1359).
    int t = 0;
    // under tensor parallelism a chunk is bounded by what one exchange of partial rows carries
    const bool tp_run = s->plan->ctx->tp_size > 1;
    const int chunk_cap = tp_run ? std::min(s->prefill_chunk, s->tp.lay.rows) : s->prefill_chunk;
    if (chunk_cap >= kPrefillMinChunk && prefill_batchable(s->plan) && (!tp_run || s->tp_attached)) {
        while (n - 1 - t >= kPrefillMinChunk) {
            const int c = std::min(chunk_cap, n - 1 - t);
            if ((rc = prefill_workspace(s, std::min(chunk_cap, n - 1)))) return rc;
            if ((rc = enqueue_prefill_chunk(s, s->prompt + t, c, s->pos_host[0], 0, s->stream))) return rc;
            s->pos_host[0] += c;
            t += c;
        }
    }
    for (; t < n; ++t) {
        SWLM_CUDA(cudaMemcpyAsync(s->token_in, s->prompt + (size_t)t * m, sizeof(int32_t) * m, cudaMemcpyDeviceToDevice, s->stream));
        rc = run_graph(s, t + 1 < n);
        if (rc) return rc;
    }
    SWLM_CUDA(cudaMemcpyAsync(s->h_tok + m, s->token_out, sizeof(int32_t) * m, cudaMemcpyDeviceToHost, s->stream));
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    memcpy(first_token, s->h_tok + m, sizeof(int32_t) * m);
    if ((rc = check_pf_status(s))) {
        for (int b = 0; b < m; ++b) first_token[b] = -1;
        return rc;
    }
    rc = check_tc_status(s);
    if (rc) for (int b = 0; b < m; ++b) first_token[b] = -1;
    return rc;
}

int swlm_prefill_seq(swlm_state* s, int seq, const int32_t* tokens, int n, int32_t* first_token) {
    if (!s || !tokens || !first_token || n <= 0) { set_error("bad argument"); return SWLM_ERR_INVALID; }
    *first_token = -1;
    const swlm_buffers_desc& d = s->plan->desc;
    if (seq < 0 || seq >= d.max_batch) { set_error("sequence %d outside 0..%d", seq, d.max_batch - 1); return SWLM_ERR_INVALID; }
    if (!rows_capable(s->plan)) { set_error("this plan cannot ingest a prompt into one sequence (tensor parallel, head_dim > 128 or an in-place product)"); return SWLM_ERR_UNSUPPORTED; }
    int rc = ensure_device(s->plan->ctx);
    if (rc) return rc;
    if (s->pos_host[seq] + n > d.max_seq) {
        set_error("sequence %d: position %d + %d tokens exceeds max_seq %d", seq, s->pos_host[seq], n, d.max_seq);
        return SWLM_ERR_STATE;
    }
    if (s->prompt_cap < (size_t)n) {
        cudaFree(s->prompt);
        s->prompt = nullptr; s->prompt_cap = 0;
        if ((rc = dev_alloc(&s->prompt, (size_t)n))) return rc;
        s->prompt_cap = (size_t)n;
    }
    SWLM_CUDA(cudaMemcpyAsync(s->prompt, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, s->stream));
    const int chunk = s->prefill_chunk >= kPrefillMinChunk ? s->prefill_chunk : 2048;
    if ((rc = prefill_workspace(s, std::min(chunk, n)))) return rc;
    for (int t = 0; t < n;) {
        const int c = std::min(chunk, n - t);
        // the chunk that holds the prompt's last token also runs the output head on that row
        if ((rc = enqueue_prefill_chunk(s, s->prompt + t, c, s->pos_host[seq], seq, s->stream, t + c == n ? c - 1 : -1))) return rc;
        s->pos_host[seq] += c;
        t += c;
    }
    SWLM_CUDA(cudaMemcpyAsync(s->h_tok, s->token_out + seq, sizeof(int32_t), cudaMemcpyDeviceToHost, s->stream));
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    if ((rc = check_pf_status(s))) return rc;
    if ((rc = check_tc_status(s))) return rc;
    *first_token = s->h_tok[0];
    return SWLM_OK;
}

int swlm_state_reset_seq(swlm_state* s, int seq) {
    if (!s) { set_error("null state"); return SWLM_ERR_INVALID; }
    const swlm_buffers_desc& d = s->plan->desc;
    if (seq < 0 || seq >= d.max_batch) { set_error("sequence %d outside 0..%d", seq, d.max_batch - 1); return SWLM_ERR_INVALID; }
    int rc = ensure_device(s->plan->ctx);
    if (rc) return rc;
    // the cache needs no clearing (rows at and beyond the position are never read); the conv state does
    const size_t per_seq = (size_t)d.conv_kernel * d.conv_dim;
    for (int l = 0; l < d.conv_layers && per_seq; ++l)
        SWLM_CUDA(cudaMemsetAsync(s->conv + (size_t)l * s->conv_layer_elems + (size_t)seq * per_seq, 0, per_seq * 2, s->stream));
    for (int l = 0; l < d.ssm_layers; ++l) {
        const size_t cs = s->ssm_conv_layer_elems / d.max_batch, rs = s->ssm_state_layer_elems / d.max_batch;
        SWLM_CUDA(cudaMemsetAsync(s->ssm_conv + (size_t)l * s->ssm_conv_layer_elems + (size_t)seq * cs, 0, cs * 2, s->stream));
        SWLM_CUDA(cudaMemsetAsync(s->ssm_state + (size_t)l * s->ssm_state_layer_elems + (size_t)seq * rs, 0, rs * 4, s->stream));
    }
    SWLM_CUDA(cudaMemsetAsync(s->position + seq, 0, 4, s->stream));
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    s->pos_host[seq] = 0;
    return SWLM_OK;
}

int swlm_state_set_prefill_chunk(swlm_state* s, int tokens) {
    if (!s || tokens < 0) { set_error("bad argument"); return SWLM_ERR_INVALID; }
    s->prefill_chunk = tokens;
    return SWLM_OK;
}

int swlm_read_buffer(swlm_state* s, int buf, uint16_t* dst, int count_per_row) {
    if (!s || !dst || !buf_ok(buf) || count_per_row > s->width[buf]) { set_error("bad buffer read"); return SWLM_ERR_INVALID; }
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    // the residual stream ends a step in whichever of its two physical buffers the plan wrote last
    const __nv_bfloat16* src = buf == SWLM_BUF_RESIDUAL ? res_buf(s, s->plan->final_res) : s->buf[buf];
    SWLM_CUDA(cudaMemcpy2D(dst, (size_t)count_per_row * 2, src, (size_t)s->width[buf] * 2, (size_t)count_per_row * 2,
                           s->plan->desc.max_batch, cudaMemcpyDeviceToHost));
    return SWLM_OK;
}

int swlm_write_buffer(swlm_state* s, int buf, const uint16_t* src, int count_per_row) {
    if (!s || !src || !buf_ok(buf) || count_per_row > s->width[buf]) { set_error("bad buffer write"); return SWLM_ERR_INVALID; }
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    SWLM_CUDA(cudaMemcpy2D(s->buf[buf], (size_t)s->width[buf] * 2, src, (size_t)count_per_row * 2, (size_t)count_per_row * 2,
                           s->plan->desc.max_batch, cudaMemcpyHostToDevice));
    if (buf == SWLM_BUF_RESIDUAL)
        SWLM_CUDA(cudaMemcpy2D(s->res2, (size_t)s->width[buf] * 2, src, (size_t)count_per_row * 2, (size_t)count_per_row * 2,
                               s->plan->desc.max_batch, cudaMemcpyHostToDevice));
    return SWLM_OK;
}

int swlm_read_logits(swlm_state* s, uint16_t* dst, size_t count) {
    if (!s || !dst) { set_error("null argument"); return SWLM_ERR_INVALID; }
    const swlm_buffers_desc& d = s->plan->desc;
    if (count != (size_t)d.max_batch * d.vocab) { set_error("logits are [%d][%d]", d.max_batch, d.vocab); return SWLM_ERR_INVALID; }
    return swlm_read_buffer(s, SWLM_BUF_LOGITS, dst, d.vocab);
}

static int kv_ptr(swlm_state* s, int which, int layer, int b, int head, int count, __nv_bfloat16** p) {
    const swlm_buffers_desc& d = s->plan->desc;
    if (layer < 0 || layer >= d.kv_layers || b < 0 || b >= d.max_batch || head < 0 || head >= kv_heads_local(s->plan) ||
        count < 0 || count > d.max_seq) { set_error("bad KV address"); return SWLM_ERR_INVALID; }
    __nv_bfloat16* base = which ? s->vcache : s->kcache;
    *p = base + (size_t)layer * s->kv_layer_elems + ((size_t)b * kv_heads_local(s->plan) + head) * d.max_seq * kv_row_bytes(d) / 2;
    return SWLM_OK;
}

// 8-bit group-32 rows on the host, for the probes: the arithmetic of write_kv_quantized_q8 / read_kv_element
// (Generator/MetalSourceGenerator+Attention.swift:2057-2101, 1923-1956).
static void kv_q8_quantise_host(const float* v, int hd, int scheme, unsigned char* row) {
    const int bits = swlm_kv_bits(scheme), group = swlm_kv_group(scheme), bb = swlm_kv_block_bytes(scheme), levels = bits == 8 ? 255 : 15;
    for (int g = 0; g * group < hd; ++g) {
        float lo = v[g * group], hi = v[g * group];
        for (int i = 1; i < group; ++i) { lo = std::min(lo, v[g * group + i]); hi = std::max(hi, v[g * group + i]); }
        float scale = (hi - lo) / (float)levels;
        if (scale < 1e-10f) scale = 1e-10f;
        unsigned char* blk = row + (size_t)g * bb;
        const __half hs = __float2half_rn(scale), hz = __float2half_rn(lo);
        memcpy(blk, &hs, 2);
        memcpy(blk + 2, &hz, 2);
        auto quant = [&](float x) { return (unsigned char)std::min(levels, std::max(0, (int)roundf((x - lo) / scale))); };
        if (bits == 8) for (int i = 0; i < group; ++i) blk[4 + i] = quant(v[g * group + i]);
        else for (int i = 0; i < group / 2; ++i) blk[4 + i] = (unsigned char)(quant(v[g * group + 2 * i]) | (quant(v[g * group + 2 * i + 1]) << 4));
    }
}
static float kv_q8_read_host(const unsigned char* row, int e, int scheme) {
    const int bits = swlm_kv_bits(scheme), group = swlm_kv_group(scheme);
    const unsigned char* blk = row + (size_t)(e / group) * swlm_kv_block_bytes(scheme);
    __half hs, hz;
    memcpy(&hs, blk, 2);
    memcpy(&hz, blk + 2, 2);
    const int i = e % group;
    const int q = bits == 8 ? blk[4 + i] : (i % 2 == 0 ? blk[4 + i / 2] & 0x0F : blk[4 + i / 2] >> 4);
    return __half2float(hs) * (float)q + __half2float(hz);
}
static float bf16_bits_to_float(uint16_t h) { const uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }
static uint16_t float_to_bf16_bits(float f) { uint32_t u; memcpy(&u, &f, 4); u += 0x7FFFu + ((u >> 16) & 1u); return (uint16_t)(u >> 16); }

int swlm_read_kv(swlm_state* s, int which, int layer, int b, int head, int count, uint16_t* dst) {
    if (!s || !dst) { set_error("null argument"); return SWLM_ERR_INVALID; }
    __nv_bfloat16* p;
    int rc = kv_ptr(s, which, layer, b, head, count, &p);
    if (rc) return rc;
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    const swlm_buffers_desc& d = s->plan->desc;
    if (swlm_kv_bits(d.kv_scheme)) {   // the dequantised rows (of a rotated scheme: turned back), rounded to bf16
        std::vector<unsigned char> rows((size_t)count * kv_row_bytes(d));
        SWLM_CUDA(cudaMemcpy(rows.data(), p, rows.size(), cudaMemcpyDeviceToHost));
        std::vector<float> f(d.head_dim);
        const uint16_t* R = swlm_kv_is_rotor(d.kv_scheme) ? s->rotors_host.data() + ((size_t)layer * d.kv_heads + head) * swlm_kv_rotor_groups(d.head_dim) * 4 : nullptr;
        for (int t = 0; t < count; ++t) {
            for (int e = 0; e < d.head_dim; ++e) f[e] = kv_q8_read_host(rows.data() + (size_t)t * kv_row_bytes(d), e, d.kv_scheme);
            if (R) kv_rotor_turn_row_host(f.data(), d.head_dim, R, true);
            for (int e = 0; e < d.head_dim; ++e) dst[(size_t)t * d.head_dim + e] = float_to_bf16_bits(f[e]);
        }
        return SWLM_OK;
    }
    SWLM_CUDA(cudaMemcpy(dst, p, (size_t)count * s->plan->desc.head_dim * 2, cudaMemcpyDeviceToHost));
    return SWLM_OK;
}

int swlm_write_kv(swlm_state* s, int which, int layer, int b, int head, int count, const uint16_t* src) {
    if (!s || !src) { set_error("null argument"); return SWLM_ERR_INVALID; }
    __nv_bfloat16* p;
    int rc = kv_ptr(s, which, layer, b, head, count, &p);
    if (rc) return rc;
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    const swlm_buffers_desc& d = s->plan->desc;
    if (swlm_kv_bits(d.kv_scheme)) {   // quantised (a rotated scheme: turned first, K rows with their projected residual) as an appended row would be
        std::vector<unsigned char> rows((size_t)count * kv_row_bytes(d));
        std::vector<float> f(d.head_dim);
        const bool rotor = swlm_kv_is_rotor(d.kv_scheme);
        const uint16_t* R = rotor ? s->rotors_host.data() + ((size_t)layer * d.kv_heads + head) * swlm_kv_rotor_groups(d.head_dim) * 4 : nullptr;
        const int qjl = rotor && which == 0 ? d.kv_qjl_dim : 0;
        std::vector<uint16_t> res((size_t)count * qjl);
        for (int t = 0; t < count; ++t) {
            for (int e = 0; e < d.head_dim; ++e) f[e] = bf16_bits_to_float(src[(size_t)t * d.head_dim + e]);
            if (R) kv_rotor_turn_row_host(f.data(), d.head_dim, R, false);
            unsigned char* row = rows.data() + (size_t)t * kv_row_bytes(d);
            kv_q8_quantise_host(f.data(), d.head_dim, d.kv_scheme, row);
            if (qjl > 0) {   // qjl_compute_residual (:1983-2013)
                for (int e = 0; e < d.head_dim; ++e) f[e] -= kv_q8_read_host(row, e, d.kv_scheme);
                for (int j = 0; j < qjl; ++j) {
                    float a = 0.0f;
                    for (int e = 0; e < d.head_dim; ++e) a += f[e] * host_f16_value(s->qjl_matrix_host[(size_t)e * qjl + j]);
                    res[(size_t)t * qjl + j] = host_f16_bits(a);
                }
            }
        }
        SWLM_CUDA(cudaMemcpy(p, rows.data(), rows.size(), cudaMemcpyHostToDevice));
        if (qjl > 0)
            SWLM_CUDA(cudaMemcpy(s->qjl_res + (size_t)layer * s->qjl_layer_elems + ((size_t)b * d.kv_heads + head) * d.max_seq * qjl,
                                 res.data(), res.size() * 2, cudaMemcpyHostToDevice));
        return SWLM_OK;
    }
    SWLM_CUDA(cudaMemcpy(p, src, (size_t)count * s->plan->desc.head_dim * 2, cudaMemcpyHostToDevice));
    return SWLM_OK;
}

int swlm_kv_scheme_supported(int scheme) { return scheme == 0 || scheme == SWLM_KV_BF16 || swlm_kv_bits(scheme) != 0; }

int swlm_state_get_rotors(swlm_state* s, uint16_t* dst, size_t count) {
    if (!s || !dst) { set_error("null argument"); return SWLM_ERR_INVALID; }
    if (count != s->rotors_host.size() || count == 0) { set_error("this state holds %zu rotor values", s->rotors_host.size()); return SWLM_ERR_INVALID; }
    memcpy(dst, s->rotors_host.data(), count * 2);
    return SWLM_OK;
}

int swlm_state_set_rotors(swlm_state* s, const uint16_t* src, size_t count) {
    if (!s || !src) { set_error("null argument"); return SWLM_ERR_INVALID; }
    if (count != s->rotors_host.size() || count == 0) { set_error("this state holds %zu rotor values", s->rotors_host.size()); return SWLM_ERR_INVALID; }
    int rc = ensure_device(s->plan->ctx);
    if (rc) return rc;
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    s->rotors_host.assign(src, src + count);
    SWLM_CUDA(cudaMemcpy(s->rotors, src, count * 2, cudaMemcpyHostToDevice));
    return SWLM_OK;
}

int swlm_read_qjl(swlm_state* s, int layer, int b, int head, int count, uint16_t* dst) {
    if (!s || !dst) { set_error("null argument"); return SWLM_ERR_INVALID; }
    const swlm_buffers_desc& d = s->plan->desc;
    if (!s->qjl_res) { set_error("this state keeps no projected residuals (kv_qjl_dim 0 or no rotated scheme)"); return SWLM_ERR_STATE; }
    if (layer < 0 || layer >= d.kv_layers || b < 0 || b >= d.max_batch || head < 0 || head >= d.kv_heads || count < 0 || count > d.max_seq) {
        set_error("bad KV address"); return SWLM_ERR_INVALID;
    }
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    SWLM_CUDA(cudaMemcpy(dst, s->qjl_res + (size_t)layer * s->qjl_layer_elems + ((size_t)b * d.kv_heads + head) * d.max_seq * d.kv_qjl_dim,
                         (size_t)count * d.kv_qjl_dim * 2, cudaMemcpyDeviceToHost));
    return SWLM_OK;
}

int swlm_read_conv(swlm_state* s, int layer, int b, uint16_t* dst) {
    if (!s || !dst) { set_error("null argument"); return SWLM_ERR_INVALID; }
    const swlm_buffers_desc& d = s->plan->desc;
    if (layer < 0 || layer >= d.conv_layers || b < 0 || b >= d.max_batch) { set_error("bad conv address"); return SWLM_ERR_INVALID; }
    const size_t n = (size_t)d.conv_kernel * d.conv_dim;
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    SWLM_CUDA(cudaMemcpy(dst, s->conv + (size_t)layer * s->conv_layer_elems + (size_t)b * n, n * 2, cudaMemcpyDeviceToHost));
    return SWLM_OK;
}

int swlm_read_ssm_state(swlm_state* s, int layer, int b, float* dst) {
    if (!s || !dst) { set_error("null argument"); return SWLM_ERR_INVALID; }
    const swlm_buffers_desc& d = s->plan->desc;
    if (layer < 0 || layer >= d.ssm_layers || b < 0 || b >= d.max_batch) { set_error("bad recurrent state address"); return SWLM_ERR_INVALID; }
    const size_t n = s->ssm_state_layer_elems / d.max_batch;
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    SWLM_CUDA(cudaMemcpy(dst, s->ssm_state + (size_t)layer * s->ssm_state_layer_elems + (size_t)b * n, n * 4, cudaMemcpyDeviceToHost));
    return SWLM_OK;
}

int swlm_run_step(swlm_state* s, const swlm_step* step, const int32_t* token_in, int32_t* token_out) {
    if (!s || !step) { set_error("null argument"); return SWLM_ERR_INVALID; }
    const int m = s->plan->desc.max_batch;
    int rc = ensure_device(s->plan->ctx);
    if (rc) return rc;
    // compile a one-step plan against the same weight store and buffer set, run it eagerly
    swlm_plan tmp;
    tmp.ctx = s->plan->ctx;
    tmp.desc = s->plan->desc;
    tmp.steps.assign(step, step + 1);
    rc = compile_plan(&tmp);
    if (!rc && m > kQGemvMaxRows) rc = ensure_rows_groups(&tmp);
    if (rc) return rc;
    // a step the state's own plan does not contain may need more scratch than the state holds
    rc = grow_scratch(s, plan_attn_scratch(&tmp), tmp.qgemv_partial, tmp.qgemv_counters);
    if (rc) { for (RopeTable& t : tmp.rope_tables) cudaFree(t.inv_freq); return rc; }
    if (token_in) SWLM_CUDA(cudaMemcpyAsync(s->token_in, token_in, sizeof(int32_t) * m, cudaMemcpyHostToDevice, s->stream));
    swlm_plan* saved = s->plan;
    const std::vector<int> saved_pos = s->pos_host;
    // an argmax step advances the device position; keep single-step runs position-neutral
    s->plan = &tmp;
    rc = enqueue_step(s, false, s->stream);
    s->plan = saved;
    cudaError_t e = cudaStreamSynchronize(s->stream);
    for (RopeTable& t : tmp.rope_tables) cudaFree(t.inv_freq);
    if (rc) return rc;
    if (e != cudaSuccess) return cuda_fail(e, "run_step sync");
    SWLM_CUDA(cudaMemcpy(s->position, saved_pos.data(), sizeof(int32_t) * m, cudaMemcpyHostToDevice));
    const int32_t saved_steps = (int32_t)s->steps_host;
    SWLM_CUDA(cudaMemcpy(s->step_counter, &saved_steps, 4, cudaMemcpyHostToDevice));
    if (token_out) SWLM_CUDA(cudaMemcpy(token_out, s->token_out, sizeof(int32_t) * m, cudaMemcpyDeviceToHost));
    return SWLM_OK;
}

int64_t swlm_launches(const swlm_state* s) { return s ? s->launches : 0; }

int swlm_tp_export(swlm_state* s, void* handle_out) {
    if (!s || !handle_out) { set_error("null argument"); return SWLM_ERR_INVALID; }
    swlm_ctx* ctx = s->plan->ctx;
    if (ctx->tp_size < 2) { set_error("context was created with tp_size 1"); return SWLM_ERR_STATE; }
    if (ctx->tp_size > kTpMax) { set_error("tp_size %d exceeds %d", ctx->tp_size, kTpMax); return SWLM_ERR_UNSUPPORTED; }
    int rc = ensure_device(ctx);
    if (rc) return rc;
    if (!s->tp.peer[ctx->tp_rank]) {
        s->tp.tp = ctx->tp_size; s->tp.rank = ctx->tp_rank;
        s->tp.lay = TpLayout{ctx->tp_size, s->plan->desc.max_batch, s->plan->desc.hidden, prefill_batchable(s->plan) ? kTpChunkRows : 0};
        unsigned char* buf = nullptr;
        if ((rc = dev_alloc(&buf, s->tp.lay.total()))) return rc;
        SWLM_CUDA(cudaMemset(buf, 0, s->tp.lay.total()));
        s->tp.peer[ctx->tp_rank] = buf;
        if ((rc = dev_alloc(&s->tp_words, 8))) return rc;
        SWLM_CUDA(cudaMemset(s->tp_words, 0, 32));
        s->tp.epoch = s->tp_words; s->tp.done = reinterpret_cast<unsigned*>(s->tp_words + 1); s->tp.status = s->tp_words + 2;
        s->tp.host_status = s->tc_status;
        SWLM_CUDA(cudaDeviceSynchronize());
    }
    cudaIpcMemHandle_t h;
    SWLM_CUDA(cudaIpcGetMemHandle(&h, s->tp.peer[ctx->tp_rank]));
    static_assert(sizeof(h) == SWLM_TP_HANDLE_BYTES, "IPC handle size");
    memcpy(handle_out, &h, sizeof(h));
    return SWLM_OK;
}

int swlm_tp_attach(swlm_state* s, const void* handles) {
    if (!s || !handles) { set_error("null argument"); return SWLM_ERR_INVALID; }
    swlm_ctx* ctx = s->plan->ctx;
    if (ctx->tp_size < 2 || !s->tp.peer[ctx->tp_rank]) { set_error("call swlm_tp_export first"); return SWLM_ERR_STATE; }
    if (s->tp_attached) return SWLM_OK;
    int rc = ensure_device(ctx);
    if (rc) return rc;
    const unsigned char* hb = static_cast<const unsigned char*>(handles);
    for (int r = 0; r < ctx->tp_size; ++r) {
        if (r == ctx->tp_rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, hb + (size_t)r * SWLM_TP_HANDLE_BYTES, sizeof(h));
        void* p = nullptr;
        SWLM_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        s->tp.peer[r] = static_cast<unsigned char*>(p);
    }
    s->tp_attached = true;
    drop_graphs(s);
    return SWLM_OK;
}

int swlm_tp_status(swlm_state* s) {
    if (!s) { set_error("null state"); return SWLM_ERR_INVALID; }
    if (!s->tp_words) return SWLM_OK;
    int32_t w[4];
    SWLM_CUDA(cudaStreamSynchronize(s->stream));
    SWLM_CUDA(cudaMemcpy(w, s->tp_words, sizeof(w), cudaMemcpyDeviceToHost));
    if (w[2]) { set_error("a bounded wait on another rank expired (all-reduce epoch %d, argmax epoch %d)", w[0], w[3]); return SWLM_ERR_TIMEOUT; }
    return SWLM_OK;
}

int swlm_tp_check_heads(int heads, int kv_heads, int tp_size) {
    if (heads <= 0 || kv_heads <= 0 || tp_size < 1) { set_error("bad argument"); return SWLM_ERR_INVALID; }
    if (tp_size == 1) return SWLM_OK;
    if (heads % tp_size || kv_heads % tp_size || (heads / tp_size) % (kv_heads / tp_size)) {
        set_error("%d query heads over %d KV heads cannot be cut into %d equal shards of whole GQA groups", heads, kv_heads, tp_size);
        return SWLM_ERR_UNSUPPORTED;
    }
    return SWLM_OK;
}

/* Rank-local slice of an n x k tensor under a shard kind: out = {row0, rows, col0, cols}. Host-only. */
int swlm_shard_range(int shard_kind, int n, int k, int tp_rank, int tp_size, int* out4) {
    if (!out4 || tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) { set_error("bad argument"); return SWLM_ERR_INVALID; }
    swlm_ctx fake;
    fake.tp_rank = tp_rank; fake.tp_size = tp_size;
    Slice sl;
    int rc = shard_slice(&fake, shard_kind, n, k, &sl);
    if (rc) return rc;
    out4[0] = sl.row0; out4[1] = sl.rows; out4[2] = sl.col0; out4[3] = sl.cols;
    return SWLM_OK;
}

int swlm_profile_kind(swlm_state* s, int step_kind, int repeats) {
    if (!s || repeats < 0) { set_error("bad argument"); return SWLM_ERR_INVALID; }
    int kind;
    switch (step_kind) {
    case SWLM_STEP_QGEMV: kind = L_QGEMV; break;
    case SWLM_STEP_ATTN_DECODE: kind = L_ATTN; break;
    case SWLM_STEP_RESADD_COPY_RMSNORM: kind = L_RMSNORM; break;
    default: set_error("profile: step kind %d has no per-kind loop", step_kind); return SWLM_ERR_UNSUPPORTED;
    }
    int rc = ensure_device(s->plan->ctx);
    for (int i = 0; i < repeats && !rc; ++i) rc = enqueue_step(s, false, s->stream, kind);
    return rc;
}

// ---- op-level ------------------------------------------------------------------------------------------

static int op_scratch_sized(swlm_ctx* ctx, size_t pf, size_t cc);
static int op_scratch(swlm_ctx* ctx, const Q4Tiled& w, int m) {
    return op_scratch_sized(ctx, qgemv_scratch_floats(w, m), (size_t)qgemv_counter_count(w));
}
static int op_scratch_sized(swlm_ctx* ctx, size_t pf, size_t cc) {
    if (pf > ctx->op_partial_floats) {
        cudaFree(ctx->op_partial);
        ctx->op_partial = nullptr; ctx->op_partial_floats = 0;
        int rc = dev_alloc(&ctx->op_partial, pf);
        if (rc) return rc;
        ctx->op_partial_floats = pf;
    }
    if (cc > ctx->op_counter_count) {
        cudaFree(ctx->op_counters);
        ctx->op_counters = nullptr; ctx->op_counter_count = 0;
        int rc = dev_alloc(&ctx->op_counters, cc);
        if (rc) return rc;
        SWLM_CUDA(cudaMemset(ctx->op_counters, 0, cc * sizeof(unsigned)));
        ctx->op_counter_count = cc;
    }
    return SWLM_OK;
}

int swlm_op_qgemm_dev(swlm_ctx* ctx, const char* weight, int m, const void* x_dev, void* y_dev, void* cuda_stream) {
    if (!ctx || !weight || !x_dev || !y_dev) { set_error("null argument"); return SWLM_ERR_INVALID; }
    int rc = ensure_device(ctx);
    if (rc) return rc;
    const Q4Tiled* w;
    rc = get_tiled(ctx, {weight}, 0, &w);
    if (rc) return rc;
    cudaStream_t stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : ctx->stream;
    if (!ctx->tc_status) {
        if ((rc = dev_alloc(&ctx->tc_status, 1))) return rc;
        SWLM_CUDA(cudaMemsetAsync(ctx->tc_status, 0, sizeof(int), ctx->stream));
        SWLM_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    // m >= 64: tensor-core contraction straight from the packed source copy
    auto raw = ctx->raw.find(weight);
    if (m >= kQGemmTcMinRows && raw != ctx->raw.end() && raw->second.k % 64 == 0) {
        const size_t need = qgemm_tc_scratch_bytes(m, raw->second.k);
        if (need > ctx->op_xh_bytes) {
            SWLM_CUDA(cudaDeviceSynchronize());
            cudaFree(ctx->op_xh);
            ctx->op_xh = nullptr; ctx->op_xh_bytes = 0;
            if ((rc = dev_alloc(&ctx->op_xh, need))) return rc;
            ctx->op_xh_bytes = need;
        }
        return launch_qgemm_tc(raw->second, m, static_cast<const __nv_bfloat16*>(x_dev), raw->second.k,
                               static_cast<__nv_bfloat16*>(y_dev), raw->second.n, ctx->op_xh, ctx->tc_status, stream);
    }
    // 16 < m < 64 runs as passes of 16 rows: each pass re-streams the weights
    for (int m0 = 0; m0 < m; m0 += 16) {
        const int mc = std::min(16, m - m0);
        rc = op_scratch(ctx, *w, mc);
        if (rc) return rc;
        QGemvLaunch a;
        a.w = w; a.m = mc;
        a.x = static_cast<const __nv_bfloat16*>(x_dev) + (size_t)m0 * w->k; a.x_stride = w->k;
        a.y[0] = static_cast<__nv_bfloat16*>(y_dev) + (size_t)m0 * w->n; a.y_stride[0] = w->n; a.seg_end[0] = w->n;
        a.partial = ctx->op_partial; a.counters = ctx->op_counters;
        rc = launch_qgemv(a, stream);
        if (rc) return rc;
    }
    return SWLM_OK;
}

int swlm_op_qgemm(swlm_ctx* ctx, const char* weight, int m, const uint16_t* x_bf16, uint16_t* y_bf16) {
    if (!ctx || !weight || !x_bf16 || !y_bf16 || m <= 0) { set_error("bad argument"); return SWLM_ERR_INVALID; }
    int rc = ensure_device(ctx);
    if (rc) return rc;
    const Q4Tiled* w;
    rc = get_tiled(ctx, {weight}, 0, &w);
    if (rc) return rc;
    __nv_bfloat16 *x = nullptr, *y = nullptr;
    if ((rc = dev_alloc(&x, (size_t)m * w->k))) return rc;
    if ((rc = dev_alloc(&y, (size_t)m * w->n))) { cudaFree(x); return rc; }
    cudaError_t e = cudaMemcpyAsync(x, x_bf16, (size_t)m * w->k * 2, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) {
        rc = swlm_op_qgemm_dev(ctx, weight, m, x, y, ctx->stream);
        if (!rc) e = cudaMemcpyAsync(y_bf16, y, (size_t)m * w->n * 2, cudaMemcpyDeviceToHost, ctx->stream);
    }
    cudaError_t e2 = cudaStreamSynchronize(ctx->stream);
    cudaFree(x); cudaFree(y);
    if (rc) return rc;
    if (e != cudaSuccess) return cuda_fail(e, "qgemm copies");
    if (e2 != cudaSuccess) return cuda_fail(e2, "qgemm sync");
    if (ctx->tc_status) {
        int st = 0;
        SWLM_CUDA(cudaMemcpy(&st, ctx->tc_status, sizeof(int), cudaMemcpyDeviceToHost));
        if (st) {
            set_error("qgemm: a bounded wait in a tensor-core kernel expired (code %d)", st);
            cudaMemset(ctx->tc_status, 0, sizeof(int));
            return SWLM_ERR_TIMEOUT;
        }
    }
    return SWLM_OK;
}

int swlm_op_dequant_bf16(swlm_ctx* ctx, const char* weight, uint16_t* out_bf16) {
    if (!ctx || !weight || !out_bf16) { set_error("null argument"); return SWLM_ERR_INVALID; }
    int rc = ensure_device(ctx);
    if (rc) return rc;
    const Q4Tiled* w;
    rc = get_tiled(ctx, {weight}, 0, &w);
    if (rc) return rc;
    __nv_bfloat16* d = nullptr;
    if ((rc = dev_alloc(&d, (size_t)w->n * w->k))) return rc;
    rc = launch_untile_bf16(*w, d, ctx->stream);
    cudaError_t e = cudaSuccess;
    if (!rc) e = cudaMemcpyAsync(out_bf16, d, (size_t)w->n * w->k * 2, cudaMemcpyDeviceToHost, ctx->stream);
    cudaError_t e2 = cudaStreamSynchronize(ctx->stream);
    cudaFree(d);
    if (rc) return rc;
    if (e != cudaSuccess) return cuda_fail(e, "dequant copy");
    if (e2 != cudaSuccess) return cuda_fail(e2, "dequant sync");
    return SWLM_OK;
}

static int flash_splits(int b, int kv_heads, int ctx_len) { return attn_pick_splits(b, kv_heads, ctx_len); }

// Arguments shared by the flash-decode entry points, checked before anything is launched, cleared or divided: the
// kernel reads q, k, v and the scratch with 128-bit loads, so a misaligned pointer would fault on the GPU instead
// of returning a status.
static int flash_args_ok(int b, int heads, int kv_heads, int hd, int ctx_len, int ctx_stride, const void* q, const void* k,
                         const void* v, const void* out, const void* scratch) {
    if (b <= 0 || heads <= 0 || kv_heads <= 0 || hd <= 0 || ctx_len <= 0 || ctx_stride <= 0 || ctx_len > ctx_stride) {
        set_error("flash-decode: batch, head counts, head_dim, context length and stride must be positive, context <= stride");
        return SWLM_ERR_INVALID;
    }
    if (heads % kv_heads) { set_error("flash-decode: %d query heads do not divide by %d KV heads", heads, kv_heads); return SWLM_ERR_INVALID; }
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
         reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(scratch)) & 15) {
        set_error("flash-decode: q, k, v, out and scratch must be 16-byte aligned");
        return SWLM_ERR_INVALID;
    }
    return SWLM_OK;
}

size_t swlm_op_flash_decode_scratch_bytes(int b, int heads, int kv_heads, int hd, int ctx_len) {
    if (b <= 0 || heads <= 0 || kv_heads <= 0 || hd <= 0 || ctx_len <= 0) return 0;
    return attn_scratch_floats(b, heads, hd, flash_splits(b, kv_heads, ctx_len)) * sizeof(float);
}

int swlm_op_flash_decode_dev(swlm_ctx* ctx, int b, int heads, int kv_heads, int hd, int ctx_len, int ctx_stride,
                             float scale, const void* q_dev, const void* k_dev, const void* v_dev, void* out_dev,
                             void* scratch_dev, void* cuda_stream) {
    if (!ctx || !q_dev || !k_dev || !v_dev || !out_dev || !scratch_dev) { set_error("null argument"); return SWLM_ERR_INVALID; }
    int rc = flash_args_ok(b, heads, kv_heads, hd, ctx_len, ctx_stride, q_dev, k_dev, v_dev, out_dev, scratch_dev);
    if (rc) return rc;
    rc = ensure_device(ctx);
    if (rc) return rc;
    cudaStream_t stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : ctx->stream;
    const size_t need = (size_t)b * kv_heads;
    if (need > ctx->op_attn_counter_count) {
        SWLM_CUDA(cudaDeviceSynchronize());
        cudaFree(ctx->op_attn_counters);
        ctx->op_attn_counters = nullptr; ctx->op_attn_counter_count = 0;
        if ((rc = dev_alloc(&ctx->op_attn_counters, need))) return rc;
        SWLM_CUDA(cudaMemset(ctx->op_attn_counters, 0, need * sizeof(unsigned)));
        ctx->op_attn_counter_count = need;
    }
    return launch_flash_decode_plain(b, heads, kv_heads, hd, ctx_len, ctx_stride, scale, static_cast<const __nv_bfloat16*>(q_dev),
                                     static_cast<const __nv_bfloat16*>(k_dev), static_cast<const __nv_bfloat16*>(v_dev),
                                     static_cast<__nv_bfloat16*>(out_dev), static_cast<float*>(scratch_dev), ctx->op_attn_counters,
                                     flash_splits(b, kv_heads, ctx_len), stream);
}

int swlm_op_flash_decode_noalloc_dev(swlm_ctx* ctx, int b, int heads, int kv_heads, int hd, int ctx_len, int ctx_stride,
                                     float scale, const void* q_dev, const void* k_dev, const void* v_dev, void* out_dev,
                                     void* cuda_stream) {
    if (!ctx || !q_dev || !k_dev || !v_dev || !out_dev) { set_error("null argument"); return SWLM_ERR_INVALID; }
    int rc = flash_args_ok(b, heads, kv_heads, hd, ctx_len, ctx_stride, q_dev, k_dev, v_dev, out_dev, nullptr);
    if (rc) return rc;
    rc = ensure_device(ctx);
    if (rc) return rc;
    cudaStream_t stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : ctx->stream;
    return launch_flash_decode_static(ctx->device, b, heads, kv_heads, hd, ctx_len, ctx_stride, scale,
                                      static_cast<const __nv_bfloat16*>(q_dev), static_cast<const __nv_bfloat16*>(k_dev),
                                      static_cast<const __nv_bfloat16*>(v_dev), static_cast<__nv_bfloat16*>(out_dev), stream);
}

size_t swlm_op_flash_decode_noalloc_capacity(void) { return flash_decode_static_capacity(); }

}  // extern "C"
