/*
 * swlm_oracle.cpp — TEST INFRASTRUCTURE, not product code.
 *
 * A scalar CPU restatement of the arithmetic of swift-lm's decode hot path,
 * written as an interpreter of the same `swlm_step` plan that the CUDA backend
 * executes. Nothing in the product library links or calls this file; only the
 * test-suite, the smoke check and the benchmark's CPU-baseline leg load it.
 *
 * The reference's kernels are Metal Shading Language strings that cannot be
 * run outside Apple platforms, and its Swift host code cannot be compiled
 * here, so parity is pinned on the known-answer vectors of the reference's
 * own kernel tests (see tests/golden): each routine below cites the reference
 * source it follows (paths relative to the reference project root).
 *
 * Rounding discipline (Sources/MetalCompiler/Buffer/MetalBufferAllocator.swift:9-30):
 * every decode buffer is bf16, so each step rounds its result to bf16 once,
 * on store; all arithmetic in between is fp32.
 */
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../include/swlm_plan.h"

namespace {

// ---- bf16 / fp16 -----------------------------------------------------------

// Sources/MetalCompiler/BFloat16.swift:25-32 — round to nearest even by adding
// 0x7FFF + lsb and truncating.
inline uint16_t f32_to_bf16(float f) {
    uint32_t bits;
    std::memcpy(&bits, &f, 4);
    uint32_t lsb = (bits >> 16) & 1u;
    bits += 0x7FFFu + lsb;
    return (uint16_t)(bits >> 16);
}
inline float bf16_to_f32(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}
inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

inline uint16_t f32_to_f16(float f) {
    _Float16 h = (_Float16)f;
    uint16_t b;
    std::memcpy(&b, &h, 2);
    return b;
}
inline float f16_to_f32(uint16_t b) {
    _Float16 h;
    std::memcpy(&h, &b, 2);
    return (float)h;
}

int g_threads = 1;

// ---- Q4 group-64 affine format ----------------------------------------------

// MLX source layout: weight u32[N][K/8], element j of a row in bits
// [4(j%8), 4(j%8)+4) of word j/8 (Sources/MetalCompiler/STAF/STAFPayloadConverter.swift:268-274);
// scales/biases bf16 [N][K/64].
inline uint32_t mlx_nibble(const uint32_t* row_words, int j) {
    return (row_words[j >> 3] >> (4 * (j & 7))) & 0xFu;
}

// STAF execution block: 36 bytes per 64 weights = fp16 scale | fp16 zero | 32 payload bytes;
// weight k in byte k>>1, low nibble when k is even
// (Sources/MetalCompiler/STAF/QuantizationFormat.swift:463-528, :1070-1090).
constexpr int kGroup = 64;
constexpr int kBlockBytes = 36;

struct Q4Tensor {
    int n = 0, k = 0;
    int group = kGroup;        // 64, or 128 (AffineQ4Group128Format, STAF/QuantizationFormat.swift:539-604)
    std::vector<uint32_t> w;   // [n][k/8]
    std::vector<float> scale;  // [n][k/group], widened exactly from bf16 (or through fp16)
    std::vector<float> zero;
};

// w = scale * float(q) + zero — Sources/SwiftLM/CPUWeightStore.swift:147-170.
inline float dequant(const Q4Tensor& t, int row, int col) {
    const uint32_t* words = t.w.data() + (size_t)row * (t.k / 8);
    int g = col / t.group;
    float s = t.scale[(size_t)row * (t.k / t.group) + g];
    float z = t.zero[(size_t)row * (t.k / t.group) + g];
    return s * (float)mlx_nibble(words, col) + z;
}

// gemv_q4_g64 — Generator/MetalSourceGenerator+Quantized.swift:552-572: per weight
// w = scale*q + zero, sum += w * x, fp32, output rounded once to the buffer type.
// y64 (optional) receives the same dot product accumulated in fp64, unrounded.
void qgemm(const Q4Tensor& t, int m, const uint16_t* x, int x_stride, uint16_t* y, int y_stride,
           double* y64) {
    const int groups = t.k / t.group;
#pragma omp parallel for schedule(static) num_threads(g_threads)
    for (int row = 0; row < t.n; ++row) {
        const uint32_t* words = t.w.data() + (size_t)row * (t.k / 8);
        for (int b = 0; b < m; ++b) {
            const uint16_t* xb = x + (size_t)b * x_stride;
            float sum = 0.0f;
            double sum64 = 0.0;
            for (int g = 0; g < groups; ++g) {
                float s = t.scale[(size_t)row * groups + g];
                float z = t.zero[(size_t)row * groups + g];
                for (int e = 0; e < t.group; ++e) {
                    int col = g * t.group + e;
                    float w = s * (float)mlx_nibble(words, col) + z;
                    float xv = bf16_to_f32(xb[col]);
                    sum += w * xv;
                    if (y64) sum64 += (double)w * (double)xv;
                }
            }
            y[(size_t)b * y_stride + row] = f32_to_bf16(sum);
            if (y64) y64[(size_t)b * t.n + row] = sum64;
        }
    }
}

// ---- RMSNorm family --------------------------------------------------------

// Primitives/Reduction.swift:91-113: fp32 sum of squares, rsqrt(total/dim + eps),
// value * rms * (weight + weightBias).
inline float rms_scale(const float* v, int dim, float eps) {
    float total = 0.0f;
    for (int i = 0; i < dim; ++i) total += v[i] * v[i];
    return 1.0f / std::sqrt(total / (float)dim + eps);
}

// ---- RoPE ------------------------------------------------------------------

// Generator/MetalSourceGenerator+Attention.swift:314-351 / :596-617: rotate-half,
// pairs (i, i + ropeDim/2), theta = pos * base^(-2i/ropeDim), fp32 pow/cos/sin.
void rope_inplace(float* v, int rope_dim, float base, int position) {
    int pairs = rope_dim / 2;
    for (int i = 0; i < pairs; ++i) {
        float theta = (float)position * std::pow(base, -2.0f * (float)i / (float)rope_dim);
        float c = std::cos(theta), s = std::sin(theta);
        float a = v[i], b = v[i + pairs];
        v[i] = a * c - b * s;
        v[i + pairs] = a * s + b * c;
    }
}

}  // namespace

// =============================================================================
// Plan interpreter
// =============================================================================

struct orc_model {
    swlm_buffers_desc desc{};
    std::map<std::string, Q4Tensor> q4;
    std::map<std::string, std::vector<uint16_t>> dense;
    std::vector<swlm_step> steps;
    // runtime buffers, bf16, [max_batch][width]
    std::vector<uint16_t> buf[SWLM_BUF_COUNT];
    int width[SWLM_BUF_COUNT]{};
    std::vector<uint16_t> kcache, vcache;  // [layer][b][kv_head][max_seq][head_dim]
    std::vector<uint8_t> kq8, vq8;         // the same rows as quantized blocks when desc.kv_scheme is one of the 8- / 4-bit schemes
    // rotated schemes: fp16 rotors [layer][kv_head][group][4], projection matrix [head_dim][qjl], projected K residuals
    // [layer][b][kv_head][max_seq][qjl]
    std::vector<uint16_t> rotors, qjl_matrix, qjl_res;
    std::vector<uint16_t> conv;            // [layer][b][conv_kernel][conv_dim]
    std::map<std::string, std::vector<float>> densef;   // fp32 tensors (recurrent layers' norm weight, A_log)
    std::vector<uint16_t> ssm_conv;        // [layer][b][ssm_conv_kernel][ssm conv dim]
    std::vector<float> ssm_state;          // [layer][b][heads][key_dim][value_dim]
    std::vector<int32_t> token_in, token_out;
    int position = 0;
    std::string error;
};

namespace {

uint16_t* row(orc_model* m, int buf, int b) { return m->buf[buf].data() + (size_t)b * m->width[buf]; }

size_t kv_index(const orc_model* m, int layer, int b, int head, int t) {
    const swlm_buffers_desc& d = m->desc;
    return ((((size_t)layer * d.max_batch + b) * d.kv_heads + head) * d.max_seq + t) * d.head_dim;
}

// ---- quantized KV rows ------------------------------------------------------------
// write_kv_quantized_q8 / _q4 (Generator/MetalSourceGenerator+Attention.swift:2057-2101, 2108-2150): per group of
// `group` values scale = max((max - min) / levels, 1e-10) with levels = 255 or 15, q = clamp(round((v - min) / scale), 0,
// levels) with the fp32 scale and min; the block stores half(scale), half(min), then the payload (4-bit: value 2i in
// the low nibble of byte i, value 2i + 1 in the high one).
void kv_q_write_row(uint8_t* row, const float* v, int hd, int scheme) {
    const int bits = swlm_kv_bits(scheme), group = swlm_kv_group(scheme), bb = swlm_kv_block_bytes(scheme);
    const int levels = bits == 8 ? 255 : 15;
    for (int g = 0; g * group < hd; ++g) {
        float lo = HUGE_VALF, hi = -HUGE_VALF;
        for (int i = 0; i < group; ++i) { lo = std::fmin(lo, v[g * group + i]); hi = std::fmax(hi, v[g * group + i]); }
        float scale = (hi - lo) / (float)levels;
        if (scale < 1e-10f) scale = 1e-10f;
        uint8_t* blk = row + (size_t)g * bb;
        uint16_t hs = f32_to_f16(scale), hz = f32_to_f16(lo);
        std::memcpy(blk, &hs, 2);
        std::memcpy(blk + 2, &hz, 2);
        auto quant = [&](float x) { int q = (int)std::round((x - lo) / scale); return (uint8_t)(q < 0 ? 0 : q > levels ? levels : q); };
        if (bits == 8) for (int i = 0; i < group; ++i) blk[4 + i] = quant(v[g * group + i]);
        else for (int i = 0; i < group / 2; ++i) blk[4 + i] = (uint8_t)(quant(v[g * group + 2 * i]) | (quant(v[g * group + 2 * i + 1]) << 4));
    }
}
// read_kv_element (:1923-1956): scale * float(q) + zero with the stored fp16 scale and zero.
inline float kv_q_read(const uint8_t* row, int e, int scheme) {
    const int bits = swlm_kv_bits(scheme), group = swlm_kv_group(scheme);
    const uint8_t* blk = row + (size_t)(e / group) * swlm_kv_block_bytes(scheme);
    uint16_t hs, hz;
    std::memcpy(&hs, blk, 2);
    std::memcpy(&hz, blk + 2, 2);
    const int i = e % group;
    const int q = bits == 8 ? blk[4 + i] : (i % 2 == 0 ? blk[4 + i / 2] & 0x0F : blk[4 + i / 2] >> 4);
    return f16_to_f32(hs) * (float)q + f16_to_f32(hz);
}
size_t kv_q_index(const orc_model* m, int layer, int b, int head, int t) {
    const swlm_buffers_desc& d = m->desc;
    return ((((size_t)layer * d.max_batch + b) * d.kv_heads + head) * d.max_seq + t) * (size_t)swlm_kv_row_bytes(d.kv_scheme, d.head_dim);
}

// ---- rotated schemes ----------------------------------------------------------------
// rotor_sandwich / rotor_sandwich_inverse (Generator/MetalSourceGenerator+Attention.swift:1807-1821) over the groups
// of three values of a row (rotor_apply_forward / _inverse, :1827-1884): R = (s, b12, b13, b23) acts like the unit
// quaternion (s, b23, -b13, b12); values past the end of the row enter as zeros and are not stored.
void rotor_turn_row(float* row, int hd, const uint16_t* R, bool inverse) {
    for (int g = 0; 3 * g < hd; ++g) {
        const int base = 3 * g;
        const float x = row[base], y = base + 1 < hd ? row[base + 1] : 0.0f, z = base + 2 < hd ? row[base + 2] : 0.0f;
        const float s = f16_to_f32(R[4 * g]);
        float px = f16_to_f32(R[4 * g + 3]), py = -f16_to_f32(R[4 * g + 2]), pz = f16_to_f32(R[4 * g + 1]);
        if (inverse) { px = -px; py = -py; pz = -pz; }
        const float tx = 2.0f * (py * z - pz * y), ty = 2.0f * (pz * x - px * z), tz = 2.0f * (px * y - py * x);
        row[base] = x + s * tx + (py * tz - pz * ty);
        if (base + 1 < hd) row[base + 1] = y + s * ty + (pz * tx - px * tz);
        if (base + 2 < hd) row[base + 2] = z + s * tz + (px * ty - py * tx);
    }
}
const uint16_t* head_rotors(const orc_model* m, int layer, int head) {
    const swlm_buffers_desc& d = m->desc;
    return m->rotors.data() + ((size_t)layer * d.kv_heads + head) * swlm_kv_rotor_groups(d.head_dim) * 4;
}
uint16_t* qjl_row(orc_model* m, int layer, int b, int head, int t) {
    const swlm_buffers_desc& d = m->desc;
    return m->qjl_res.data() + ((((size_t)layer * d.max_batch + b) * d.kv_heads + head) * d.max_seq + t) * d.kv_qjl_dim;
}
// qjl_compute_residual (:1983-2013): Phi . (row - the values its quantized blocks give back), as fp16
void qjl_store_residual(orc_model* m, int layer, int b, int head, int t, const float* turned, const uint8_t* blocks) {
    const swlm_buffers_desc& d = m->desc;
    const int hd = d.head_dim, qjl = d.kv_qjl_dim;
    std::vector<float> res(hd);
    for (int e = 0; e < hd; ++e) res[e] = turned[e] - kv_q_read(blocks, e, d.kv_scheme);
    uint16_t* out = qjl_row(m, layer, b, head, t);
    for (int j = 0; j < qjl; ++j) {
        float a = 0.0f;
        for (int e = 0; e < hd; ++e) a += res[e] * f16_to_f32(m->qjl_matrix[(size_t)e * qjl + j]);
        out[j] = f32_to_f16(a);
    }
}
// initializeRandomUnitRotors / initializeRademacherMatrix (Buffer/MetalGraphAllocator.swift:349-411)
void rotor_defaults(orc_model* m) {
    const swlm_buffers_desc& d = m->desc;
    const size_t total = (size_t)d.kv_layers * d.kv_heads * swlm_kv_rotor_groups(d.head_dim);
    m->rotors.assign(total * 4, 0);
    const float unit = 1.0f / (float)(1 << 30);
    for (size_t i = 0; i < total; ++i) {
        uint64_t h = (uint64_t)i;
        float c[4];
        for (int j = 0; j < 4; ++j) {
            h = h * 6364136223846793005ull + 1442695040888963407ull;
            c[j] = (float)((int64_t)(h >> 33) - ((int64_t)1 << 30)) * unit;
        }
        const float norm = std::sqrt(c[0] * c[0] + c[1] * c[1] + c[2] * c[2] + c[3] * c[3]);
        if (norm < 1e-8f) { c[0] = 1.0f; c[1] = c[2] = c[3] = 0.0f; }
        else { const float inv = 1.0f / norm; for (int j = 0; j < 4; ++j) c[j] *= inv; }
        for (int j = 0; j < 4; ++j) m->rotors[i * 4 + j] = f32_to_f16(c[j]);
    }
    const int qjl = d.kv_qjl_dim;
    if (qjl <= 0) return;
    const float scale = 1.0f / std::sqrt((float)qjl);
    m->qjl_matrix.assign((size_t)d.head_dim * qjl, 0);
    for (size_t i = 0; i < m->qjl_matrix.size(); ++i) {
        const uint64_t h = (uint64_t)i * 6364136223846793005ull + 1442695040888963407ull;
        m->qjl_matrix[i] = f32_to_f16(((h >> 33) & 1) == 0 ? scale : -scale);
    }
    m->qjl_res.assign((size_t)d.kv_layers * d.max_batch * d.kv_heads * d.max_seq * qjl, 0);
}

int run_step(orc_model* m, const swlm_step& st, int batch) {
    const swlm_buffers_desc& d = m->desc;
    switch (st.kind) {
    case SWLM_STEP_EMBED: {
        // Generator/MetalSourceGenerator+Embedding.swift:3-48: row gather.
        auto it = m->dense.find(st.weight);
        if (it == m->dense.end()) {
            // Quantized table (a tied output head reuses it as lm_head,
            // Sources/Models/LlamaFamilyNaming.swift:22-27): embedding_lookup_q4
            // (Generator/MetalSourceGenerator+Embedding.swift:79-154), value = q * scale + zero per element,
            // rounded once to the buffer type.
            auto q = m->q4.find(st.weight);
            if (q == m->q4.end()) { m->error = std::string("missing ") + st.weight; return -3; }
            if (q->second.k != st.n) { m->error = "embedding width mismatch"; return -1; }
            for (int b = 0; b < batch; ++b) {
                int tok = m->token_in[b];
                if (tok < 0 || tok >= q->second.n) { m->error = "token out of range"; return -1; }
                uint16_t* out = row(m, st.out_buf, b);
                for (int i = 0; i < st.n; ++i) out[i] = f32_to_bf16(dequant(q->second, tok, i));
            }
            return 0;
        }
        for (int b = 0; b < batch; ++b) {
            int tok = m->token_in[b];
            if (tok < 0 || tok >= d.vocab) { m->error = "token out of range"; return -1; }
            std::memcpy(row(m, st.out_buf, b), it->second.data() + (size_t)tok * st.n, (size_t)st.n * 2);
        }
        return 0;
    }
    case SWLM_STEP_COPY_RMSNORM:
    case SWLM_STEP_RESADD_COPY_RMSNORM:
    case SWLM_STEP_RESADD_RMSNORM: {
        // Fused kernel: intermediates stay fp32, only buffer stores are cast
        // (Primitives/PrimitiveFragments.swift:98-117), so the norm sees the unrounded sum.
        auto it = m->dense.find(st.weight);
        if (it == m->dense.end()) { m->error = std::string("missing ") + st.weight; return -3; }
        std::vector<float> h(st.n);
        for (int b = 0; b < batch; ++b) {
            uint16_t* in = row(m, st.in_buf, b);
            uint16_t* res = row(m, SWLM_BUF_RESIDUAL, b);
            for (int i = 0; i < st.n; ++i) {
                float v = bf16_to_f32(in[i]);
                if (st.kind != SWLM_STEP_COPY_RMSNORM) v += bf16_to_f32(res[i]);
                h[i] = v;
            }
            if (st.kind != SWLM_STEP_RESADD_RMSNORM)
                for (int i = 0; i < st.n; ++i) res[i] = f32_to_bf16(h[i]);
            float rs = rms_scale(h.data(), st.n, st.eps);
            uint16_t* out = row(m, st.out_buf, b);
            for (int i = 0; i < st.n; ++i)
                out[i] = f32_to_bf16(h[i] * rs * (bf16_to_f32(it->second[i]) + st.weight_bias));
        }
        return 0;
    }
    case SWLM_STEP_QGEMV: {
        auto it = m->q4.find(st.weight);
        if (it == m->q4.end()) { m->error = std::string("missing ") + st.weight; return -3; }
        if (it->second.n != st.n || it->second.k != st.k) { m->error = "qgemv shape mismatch"; return -1; }
        // in_buf may equal out_buf only when widths differ in role; copy the input first.
        std::vector<uint16_t> x((size_t)batch * st.k);
        for (int b = 0; b < batch; ++b) std::memcpy(x.data() + (size_t)b * st.k, row(m, st.in_buf, b), (size_t)st.k * 2);
        qgemm(it->second, batch, x.data(), st.k, m->buf[st.out_buf].data(), m->width[st.out_buf], nullptr);
        return 0;
    }
    case SWLM_STEP_QK_NORM: {
        // Generator/MetalSourceGenerator+Batched.swift:722-757: per head, in place.
        auto wq = m->dense.find(st.weight), wk = m->dense.find(st.weight2);
        if (wq == m->dense.end() || wk == m->dense.end()) { m->error = "missing qk norm weight"; return -3; }
        std::vector<float> v(st.head_dim);
        for (int b = 0; b < batch; ++b)
            for (int which = 0; which < 2; ++which) {
                uint16_t* data = row(m, which ? st.in2_buf : st.in_buf, b);
                const uint16_t* w = which ? wk->second.data() : wq->second.data();
                int heads = which ? st.kv_heads : st.heads;
                for (int h = 0; h < heads; ++h) {
                    uint16_t* p = data + (size_t)h * st.head_dim;
                    for (int i = 0; i < st.head_dim; ++i) v[i] = bf16_to_f32(p[i]);
                    float rs = rms_scale(v.data(), st.head_dim, st.eps);
                    for (int i = 0; i < st.head_dim; ++i)
                        p[i] = f32_to_bf16(v[i] * rs * (bf16_to_f32(w[i]) + st.weight_bias));
                }
            }
        return 0;
    }
    case SWLM_STEP_ATTN_DECODE: {
        // Generator/MetalSourceGenerator+Attention.swift:685-693, 761-805, 842-927.
        const int hd = st.head_dim, pos = m->position;
        if (pos >= d.max_seq) { m->error = "position beyond max_seq"; return -1; }
        const int total = batch * st.heads;
#pragma omp parallel for schedule(static) num_threads(g_threads)
        for (int idx = 0; idx < total; ++idx) {
            int b = idx / st.heads, h = idx % st.heads;
            int kvh = h * st.kv_heads / st.heads;
            std::vector<float> q(hd), kc(hd), vc(hd), out(hd, 0.0f);
            const uint16_t* qin = row(m, st.in_buf, b) + (size_t)h * hd;
            const uint16_t* kin = row(m, st.in2_buf, b) + (size_t)kvh * hd;
            const uint16_t* vin = row(m, st.in3_buf, b) + (size_t)kvh * hd;
            for (int i = 0; i < hd; ++i) { q[i] = bf16_to_f32(qin[i]); kc[i] = bf16_to_f32(kin[i]); vc[i] = bf16_to_f32(vin[i]); }
            if (st.rope_dim > 0) {
                rope_inplace(q.data(), st.rope_dim, st.rope_base, pos);
                rope_inplace(kc.data(), st.rope_dim, st.rope_base, pos);
            }
            // rotated schemes (:708-760, :813-840): q, the new k and the new v are turned; Phi . q for the correction
            const bool rotor = swlm_kv_is_rotor(d.kv_scheme);
            const int qjl = rotor ? d.kv_qjl_dim : 0;
            std::vector<float> qproj(qjl > 0 ? qjl : 1, 0.0f);
            if (rotor) {
                const uint16_t* R = head_rotors(m, st.layer, kvh);
                rotor_turn_row(q.data(), hd, R, false);
                rotor_turn_row(kc.data(), hd, R, false);
                rotor_turn_row(vc.data(), hd, R, false);
                for (int j = 0; j < qjl; ++j) {
                    float a = 0.0f;
                    for (int i = 0; i < hd; ++i) a += q[i] * f16_to_f32(m->qjl_matrix[(size_t)i * qjl + j]);
                    qproj[j] = a;
                }
            }
            const bool q8 = swlm_kv_bits(d.kv_scheme) != 0;
            const size_t q8_row = (size_t)swlm_kv_row_bytes(d.kv_scheme, hd);
            const uint16_t* kbase = q8 ? nullptr : m->kcache.data() + kv_index(m, st.layer, b, kvh, 0);
            const uint16_t* vbase = q8 ? nullptr : m->vcache.data() + kv_index(m, st.layer, b, kvh, 0);
            const uint8_t* kq = q8 ? m->kq8.data() + kv_q_index(m, st.layer, b, kvh, 0) : nullptr;
            const uint8_t* vq = q8 ? m->vq8.data() + kv_q_index(m, st.layer, b, kvh, 0) : nullptr;
            float max_score = -HUGE_VALF, sum_exp = 0.0f;
            // sliding window (:851-853): the current token and the window_left - 1 before it
            const int t_first = st.window_left > 0 && pos + 1 > st.window_left ? pos - st.window_left + 1 : 0;
            for (int t = t_first; t <= pos; ++t) {
                float score = 0.0f;
                if (t == pos) {
                    // the current token's key and value are used unrounded (:866-868, :905-907)
                    for (int i = 0; i < hd; ++i) score += q[i] * kc[i];
                } else if (q8) {
                    for (int i = 0; i < hd; ++i) score += q[i] * kv_q_read(kq + (size_t)t * q8_row, i, d.kv_scheme);
                    if (qjl > 0) {   // qjl_score_correction (:2036-2048), cached rows only (:873-876)
                        const uint16_t* rr = qjl_row(m, st.layer, b, kvh, t);
                        for (int j = 0; j < qjl; ++j) score += qproj[j] * f16_to_f32(rr[j]);
                    }
                } else {
                    const uint16_t* kr = kbase + (size_t)t * hd;
                    for (int i = 0; i < hd; ++i) score += q[i] * bf16_to_f32(kr[i]);
                }
                score *= st.scale;
                float old_max = max_score;
                max_score = std::fmax(max_score, score);
                float corr = std::exp(old_max - max_score);
                sum_exp = sum_exp * corr + std::exp(score - max_score);
                float wgt = std::exp(score - max_score);
                if (t == pos) {
                    for (int i = 0; i < hd; ++i) out[i] = out[i] * corr + wgt * vc[i];
                } else if (q8) {
                    for (int i = 0; i < hd; ++i) out[i] = out[i] * corr + wgt * kv_q_read(vq + (size_t)t * q8_row, i, d.kv_scheme);
                } else {
                    const uint16_t* vr = vbase + (size_t)t * hd;
                    for (int i = 0; i < hd; ++i) out[i] = out[i] * corr + wgt * bf16_to_f32(vr[i]);
                }
            }
            float inv = sum_exp > 0.0f ? 1.0f / sum_exp : 0.0f;
            uint16_t* o = row(m, st.out_buf, b) + (size_t)h * hd;
            for (int i = 0; i < hd; ++i) out[i] *= inv;
            if (rotor) rotor_turn_row(out.data(), hd, head_rotors(m, st.layer, kvh), true);   // (:914-923)
            for (int i = 0; i < hd; ++i) o[i] = f32_to_bf16(out[i]);
        }
        // KV append, once per KV head, rounded to bf16 (:761-805, write_kv_element_dense :1961-1963).
        for (int b = 0; b < batch; ++b)
            for (int kvh = 0; kvh < st.kv_heads; ++kvh) {
                std::vector<float> kc(hd);
                const uint16_t* kin = row(m, st.in2_buf, b) + (size_t)kvh * hd;
                const uint16_t* vin = row(m, st.in3_buf, b) + (size_t)kvh * hd;
                for (int i = 0; i < hd; ++i) kc[i] = bf16_to_f32(kin[i]);
                if (st.rope_dim > 0) rope_inplace(kc.data(), st.rope_dim, st.rope_base, pos);
                if (swlm_kv_bits(d.kv_scheme)) {   // quantized from the unrounded rotated k and from v as given
                    std::vector<float> vf(hd);
                    for (int i = 0; i < hd; ++i) vf[i] = bf16_to_f32(vin[i]);
                    if (swlm_kv_is_rotor(d.kv_scheme)) {
                        rotor_turn_row(kc.data(), hd, head_rotors(m, st.layer, kvh), false);
                        rotor_turn_row(vf.data(), hd, head_rotors(m, st.layer, kvh), false);
                    }
                    uint8_t* kblocks = m->kq8.data() + kv_q_index(m, st.layer, b, kvh, pos);
                    kv_q_write_row(kblocks, kc.data(), hd, d.kv_scheme);
                    kv_q_write_row(m->vq8.data() + kv_q_index(m, st.layer, b, kvh, pos), vf.data(), hd, d.kv_scheme);
                    if (swlm_kv_is_rotor(d.kv_scheme) && d.kv_qjl_dim > 0) qjl_store_residual(m, st.layer, b, kvh, pos, kc.data(), kblocks);
                    continue;
                }
                uint16_t* kw = m->kcache.data() + kv_index(m, st.layer, b, kvh, pos);
                uint16_t* vw = m->vcache.data() + kv_index(m, st.layer, b, kvh, pos);
                for (int i = 0; i < hd; ++i) { kw[i] = f32_to_bf16(kc[i]); vw[i] = vin[i]; }
            }
        return 0;
    }
    case SWLM_STEP_SWIGLU: {
        // Primitives/ElementwiseFragment.swift:49-54.
        for (int b = 0; b < batch; ++b) {
            const uint16_t* g = row(m, st.in_buf, b);
            const uint16_t* u = row(m, st.in2_buf, b);
            uint16_t* o = row(m, st.out_buf, b);
            for (int i = 0; i < st.n; ++i) {
                float gv = bf16_to_f32(g[i]);
                o[i] = f32_to_bf16(gv * (1.0f / (1.0f + std::exp(-gv))) * bf16_to_f32(u[i]));
            }
        }
        return 0;
    }
    case SWLM_STEP_GEGLU: {
        // Generator/MetalSourceGenerator+NormAndElementwise.swift:176-208 (GatedActivation.geluTanh).
        for (int b = 0; b < batch; ++b) {
            const uint16_t* g = row(m, st.in_buf, b);
            const uint16_t* u = row(m, st.in2_buf, b);
            uint16_t* o = row(m, st.out_buf, b);
            for (int i = 0; i < st.n; ++i) {
                float gv = bf16_to_f32(g[i]);
                float act = 0.5f * gv * (1.0f + std::tanh(0.7978845608f * (gv + 0.044715f * gv * gv * gv)));
                o[i] = f32_to_bf16(act * bf16_to_f32(u[i]));
            }
        }
        return 0;
    }
    case SWLM_STEP_CONV_STATE_UPDATE: {
        // Generator/MetalSourceGenerator+ConvAndState.swift:49-67.
        auto it = m->dense.find(st.weight);
        if (it == m->dense.end()) { m->error = std::string("missing ") + st.weight; return -3; }
        const int D = st.n, K = st.conv_kernel;
        for (int b = 0; b < batch; ++b) {
            const uint16_t* in = row(m, st.in_buf, b);
            uint16_t* o = row(m, st.out_buf, b);
            uint16_t* state = m->conv.data() + (((size_t)st.layer * d.max_batch + b) * d.conv_kernel) * d.conv_dim;
            for (int c = 0; c < D; ++c) {
                float B = bf16_to_f32(in[c]), C = bf16_to_f32(in[D + c]), x = bf16_to_f32(in[2 * D + c]);
                float Bx = B * x;
                for (int k = 0; k < K - 1; ++k) state[(size_t)k * D + c] = state[(size_t)(k + 1) * D + c];
                state[(size_t)(K - 1) * D + c] = f32_to_bf16(Bx);
                float acc = 0.0f;
                for (int k = 0; k + 1 < K; ++k)
                    acc += bf16_to_f32(state[(size_t)k * D + c]) * bf16_to_f32(it->second[(size_t)c * K + k]);
                acc += Bx * bf16_to_f32(it->second[(size_t)c * K + (K - 1)]);
                o[c] = f32_to_bf16(C * acc);
            }
        }
        return 0;
    }
    case SWLM_STEP_SSM_RECURRENCE: {
        // Generator/MetalSourceGenerator+ConvAndState.swift:347-497 (ssm_recurrence, bf16 buffers and weights),
        // helpers :224-227. Scalar restatement in the kernel's own order of operations.
        auto cw = m->dense.find(st.weight);
        auto nw = m->densef.find(st.weight2);
        auto db = m->dense.find(st.weight3);
        auto al = m->densef.find(st.weight4);
        if (cw == m->dense.end() || nw == m->densef.end() || db == m->dense.end() || al == m->densef.end()) {
            m->error = std::string("missing tensors of ") + st.weight; return -3;
        }
        const int H = st.heads, G = st.groups > 0 ? st.groups : 1, dk = st.key_dim, dv = st.value_dim, K = st.conv_kernel;
        const int hpg = H / G > 0 ? H / G : 1, kgd = G * dk, conv_dim = 2 * kgd + H * dv;
        auto sigmoid = [](float x) { return 1.0f / (1.0f + std::exp(-x)); };
        auto softplus = [](float x) { return std::fmax(x, 0.0f) + std::log(1.0f + std::exp(-std::fabs(x))); };
        for (int b = 0; b < batch; ++b) {
            const uint16_t* qkv = row(m, st.in_buf, b);
            const uint16_t* zz = row(m, st.in2_buf, b);
            const uint16_t* pbeta = row(m, st.in3_buf, b);
            const uint16_t* palpha = row(m, st.in4_buf, b);
            uint16_t* out = row(m, st.out_buf, b);
            uint16_t* cstate = m->ssm_conv.data() + ((size_t)st.layer * d.max_batch + b) * (size_t)K * conv_dim;
            float* rstate = m->ssm_state.data() + ((size_t)st.layer * d.max_batch + b) * (size_t)H * dk * dv;
            // phase 1: conv shift + SiLU for every channel (:392-414)
            std::vector<float> act(conv_dim);
            for (int ch = 0; ch < conv_dim; ++ch) {
                float sum = 0.0f;
                for (int k = 0; k + 1 < K; ++k) {
                    float val = bf16_to_f32(cstate[(size_t)(k + 1) * conv_dim + ch]);
                    cstate[(size_t)k * conv_dim + ch] = f32_to_bf16(val);
                    sum += val * bf16_to_f32(cw->second[(size_t)ch * K + k]);
                }
                float nv = bf16_to_f32(qkv[ch]);
                cstate[(size_t)(K - 1) * conv_dim + ch] = f32_to_bf16(nv);
                sum += nv * bf16_to_f32(cw->second[(size_t)ch * K + (K - 1)]);
                act[ch] = sum * sigmoid(sum);
            }
            // phases 2 and 3 per head (:418-497)
            for (int h = 0; h < H; ++h) {
                const int g = h / hpg;
                const float* Q = act.data() + (size_t)g * dk;
                const float* Kk = act.data() + kgd + (size_t)g * dk;
                const float* V = act.data() + 2 * kgd + (size_t)h * dv;
                float decay = std::exp(-std::exp(al->second[h]) * softplus(bf16_to_f32(palpha[h]) + bf16_to_f32(db->second[h])));
                float beta = sigmoid(bf16_to_f32(pbeta[h]));
                float* S = rstate + (size_t)h * dk * dv;
                float qn = 0.0f, kn = 0.0f, kq = 0.0f;
                for (int j = 0; j < dk; ++j) { qn += Q[j] * Q[j]; kn += Kk[j] * Kk[j]; kq += Q[j] * Kk[j]; }
                float q_inv = (1.0f / std::sqrt(qn + 1e-6f)) * (1.0f / std::sqrt((float)dk));
                float k_inv = 1.0f / std::sqrt(kn + 1e-6f);
                std::vector<float> stored(dv);
                float norm_sq = 0.0f;
                for (int dd = 0; dd < dv; ++dd) {
                    float kvmem = 0.0f, sq = 0.0f;
                    for (int j = 0; j < dk; ++j) {
                        float s = S[(size_t)j * dv + dd] * decay;
                        kvmem += s * Kk[j];
                        sq += s * Q[j];
                    }
                    float delta = beta * (V[dd] - kvmem * k_inv);
                    float kid = k_inv * delta;
                    float dot = (sq + kid * kq) * q_inv;
                    for (int j = 0; j < dk; ++j) S[(size_t)j * dv + dd] = S[(size_t)j * dv + dd] * decay + Kk[j] * kid;
                    stored[dd] = round_bf16(dot);
                    norm_sq += dot * dot;
                }
                float rms = 1.0f / std::sqrt(norm_sq / (float)dv + 1e-6f);
                for (int dd = 0; dd < dv; ++dd) {
                    float normed = stored[dd] * rms * nw->second[dd];
                    float z = bf16_to_f32(zz[(size_t)h * dv + dd]);
                    out[(size_t)h * dv + dd] = f32_to_bf16(normed * z * sigmoid(z));
                }
            }
        }
        return 0;
    }
    case SWLM_STEP_ARGMAX: {
        // Generator/MetalSourceGenerator+Sampling.swift:79-103: strict '>' comparisons;
        // restated as "lowest index wins among equal maxima" for the whole vector.
        for (int b = 0; b < batch; ++b) {
            const uint16_t* l = row(m, st.in_buf, b);
            float best = -HUGE_VALF;
            int idx = 0;
            for (int i = 0; i < st.n; ++i) {
                float v = bf16_to_f32(l[i]);
                if (v > best) { best = v; idx = i; }
            }
            m->token_out[b] = idx;
        }
        return 0;
    }
    default:
        m->error = "unknown step kind";
        return -4;
    }
}

}  // namespace

extern "C" {

void orc_set_threads(int n) {
#ifdef _OPENMP
    g_threads = n > 0 ? n : omp_get_max_threads();
#else
    (void)n;
    g_threads = 1;
#endif
}
int orc_get_threads(void) { return g_threads; }

uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
float orc_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

orc_model* orc_create(const swlm_buffers_desc* desc) {
    orc_model* m = new orc_model();
    m->desc = *desc;
    const swlm_buffers_desc& d = m->desc;
    for (int i = 0; i < SWLM_BUF_COUNT; ++i) {
        int w = (i == SWLM_BUF_HIDDEN || i == SWLM_BUF_RESIDUAL) ? d.hidden : (i == SWLM_BUF_LOGITS ? d.vocab : d.slot_dim);
        m->width[i] = w;
        m->buf[i].assign((size_t)d.max_batch * w, 0);
    }
    size_t kv = (size_t)d.kv_layers * d.max_batch * d.kv_heads * d.max_seq * d.head_dim;
    if (swlm_kv_bits(d.kv_scheme)) {
        const size_t bytes = (size_t)d.kv_layers * d.max_batch * d.kv_heads * d.max_seq * (size_t)swlm_kv_row_bytes(d.kv_scheme, d.head_dim);
        m->kq8.assign(bytes, 0);
        m->vq8.assign(bytes, 0);
        kv = 0;
        if (swlm_kv_is_rotor(d.kv_scheme)) rotor_defaults(m);
    }
    m->kcache.assign(kv, 0);
    m->vcache.assign(kv, 0);
    m->conv.assign((size_t)d.conv_layers * d.max_batch * d.conv_kernel * d.conv_dim, 0);
    const size_t ssm_conv_dim = (size_t)2 * d.ssm_groups * d.ssm_key_dim + (size_t)d.ssm_heads * d.ssm_value_dim;
    m->ssm_conv.assign((size_t)d.ssm_layers * d.max_batch * d.ssm_conv_kernel * ssm_conv_dim, 0);
    m->ssm_state.assign((size_t)d.ssm_layers * d.max_batch * d.ssm_heads * d.ssm_key_dim * d.ssm_value_dim, 0.0f);
    m->token_in.assign(d.max_batch, 0);
    m->token_out.assign(d.max_batch, 0);
    return m;
}
void orc_destroy(orc_model* m) { delete m; }
const char* orc_error(const orc_model* m) { return m->error.c_str(); }

// staf_fp16 != 0 narrows scale and bias through fp16, as the reference's STAF
// converter does (Sources/MetalCompiler/STAF/STAFPayloadConverter.swift:326-368).
int orc_add_q4_group(orc_model* m, const char* name, int n, int k, int group, const uint32_t* w,
                     const uint16_t* scales_bf16, const uint16_t* biases_bf16, int staf_fp16);
int orc_add_q4(orc_model* m, const char* name, int n, int k, const uint32_t* w,
               const uint16_t* scales_bf16, const uint16_t* biases_bf16, int staf_fp16) {
    return orc_add_q4_group(m, name, n, k, kGroup, w, scales_bf16, biases_bf16, staf_fp16);
}
// group = 64 or 128 weights per scale / bias pair
int orc_add_q4_group(orc_model* m, const char* name, int n, int k, int group, const uint32_t* w,
                     const uint16_t* scales_bf16, const uint16_t* biases_bf16, int staf_fp16) {
    if ((group != 64 && group != 128) || k % group) { m->error = "group must be 64 or 128 and divide k"; return -1; }
    Q4Tensor t;
    t.n = n; t.k = k; t.group = group;
    t.w.assign(w, w + (size_t)n * (k / 8));
    size_t g = (size_t)n * (k / group);
    t.scale.resize(g); t.zero.resize(g);
    for (size_t i = 0; i < g; ++i) {
        float s = bf16_to_f32(scales_bf16[i]), z = bf16_to_f32(biases_bf16[i]);
        if (staf_fp16) { s = f16_to_f32(f32_to_f16(s)); z = f16_to_f32(f32_to_f16(z)); }
        t.scale[i] = s; t.zero[i] = z;
    }
    m->q4[name] = std::move(t);
    return 0;
}
int orc_add_dense(orc_model* m, const char* name, int64_t count, const uint16_t* data) {
    m->dense[name].assign(data, data + count);
    return 0;
}
int orc_set_plan(orc_model* m, const swlm_step* steps, int n) {
    m->steps.assign(steps, steps + n);
    return 0;
}
void orc_reset(orc_model* m) {
    m->position = 0;
    std::fill(m->kcache.begin(), m->kcache.end(), 0);
    std::fill(m->vcache.begin(), m->vcache.end(), 0);
    std::fill(m->kq8.begin(), m->kq8.end(), 0);
    std::fill(m->vq8.begin(), m->vq8.end(), 0);
    std::fill(m->conv.begin(), m->conv.end(), 0);
    std::fill(m->ssm_conv.begin(), m->ssm_conv.end(), 0);
    std::fill(m->ssm_state.begin(), m->ssm_state.end(), 0.0f);
    for (auto& b : m->buf) std::fill(b.begin(), b.end(), 0);
}
int orc_position(const orc_model* m) { return m->position; }

// One decode step for `max_batch` sequences at the shared position
// (Sources/MetalCompiler/Execution/MetalDecodeExecutor.swift:7-43).
int orc_decode(orc_model* m, const int32_t* token_in, int32_t* token_out) {
    int batch = m->desc.max_batch;
    for (int b = 0; b < batch; ++b) m->token_in[b] = token_in[b];
    for (const swlm_step& st : m->steps) {
        int rc = run_step(m, st, batch);
        if (rc) return rc;
    }
    for (int b = 0; b < batch; ++b) token_out[b] = m->token_out[b];
    m->position += 1;
    return 0;
}

// Prompt ingestion as repeated decode: the reference's sequence kernels are built to
// reproduce the token-by-token trace (Generator/MetalSourceGenerator.swift:73-81).
// tokens is [max_batch][n]; first_token receives the token generated after the prompt.
int orc_prefill(orc_model* m, const int32_t* tokens, int n, int32_t* first_token) {
    int batch = m->desc.max_batch;
    std::vector<int32_t> in(batch), out(batch);
    for (int t = 0; t < n; ++t) {
        for (int b = 0; b < batch; ++b) in[b] = tokens[(size_t)b * n + t];
        int rc = orc_decode(m, in.data(), out.data());
        if (rc) return rc;
    }
    for (int b = 0; b < batch; ++b) first_token[b] = out[b];
    return 0;
}

int orc_read_buffer(orc_model* m, int buf, uint16_t* dst, int count_per_row) {
    if (buf < 0 || buf >= SWLM_BUF_COUNT || count_per_row > m->width[buf]) return -1;
    for (int b = 0; b < m->desc.max_batch; ++b)
        std::memcpy(dst + (size_t)b * count_per_row, row(m, buf, b), (size_t)count_per_row * 2);
    return 0;
}
int orc_write_buffer(orc_model* m, int buf, const uint16_t* src, int count_per_row) {
    if (buf < 0 || buf >= SWLM_BUF_COUNT || count_per_row > m->width[buf]) return -1;
    for (int b = 0; b < m->desc.max_batch; ++b)
        std::memcpy(row(m, buf, b), src + (size_t)b * count_per_row, (size_t)count_per_row * 2);
    return 0;
}
void orc_set_position(orc_model* m, int p) { m->position = p; }
// Run a single step on the current buffers (op-level parity tests).
int orc_run_step(orc_model* m, const swlm_step* st, const int32_t* token_in, int32_t* token_out) {
    int batch = m->desc.max_batch;
    if (token_in) for (int b = 0; b < batch; ++b) m->token_in[b] = token_in[b];
    int rc = run_step(m, *st, batch);
    if (token_out) for (int b = 0; b < batch; ++b) token_out[b] = m->token_out[b];
    return rc;
}
// K or V cache rows of one (layer, sequence, head): [count][head_dim] bf16 from token 0.
int orc_read_kv(orc_model* m, int which, int layer, int b, int head, int count, uint16_t* dst) {
    if (swlm_kv_bits(m->desc.kv_scheme)) {   // the dequantised rows, rounded to bf16
        const int hd = m->desc.head_dim, sch = m->desc.kv_scheme;
        const uint8_t* rows = (which ? m->vq8 : m->kq8).data() + kv_q_index(m, layer, b, head, 0);
        std::vector<float> f(hd);
        for (int t = 0; t < count; ++t) {   // (rows of a rotated scheme are turned back)
            for (int e = 0; e < hd; ++e) f[e] = kv_q_read(rows + (size_t)t * swlm_kv_row_bytes(sch, hd), e, sch);
            if (swlm_kv_is_rotor(sch)) rotor_turn_row(f.data(), hd, head_rotors(m, layer, head), true);
            for (int e = 0; e < hd; ++e) dst[(size_t)t * hd + e] = f32_to_bf16(f[e]);
        }
        return 0;
    }
    const std::vector<uint16_t>& c = which ? m->vcache : m->kcache;
    std::memcpy(dst, c.data() + kv_index(m, layer, b, head, 0), (size_t)count * m->desc.head_dim * 2);
    return 0;
}
int orc_write_kv(orc_model* m, int which, int layer, int b, int head, int count, const uint16_t* src) {
    if (swlm_kv_bits(m->desc.kv_scheme)) {   // the rows are quantised as an appended row would be
        const int hd = m->desc.head_dim, sch = m->desc.kv_scheme;
        uint8_t* rows = (which ? m->vq8 : m->kq8).data() + kv_q_index(m, layer, b, head, 0);
        std::vector<float> f(hd);
        for (int t = 0; t < count; ++t) {
            for (int e = 0; e < hd; ++e) f[e] = bf16_to_f32(src[(size_t)t * hd + e]);
            if (swlm_kv_is_rotor(sch)) rotor_turn_row(f.data(), hd, head_rotors(m, layer, head), false);
            uint8_t* blocks = rows + (size_t)t * swlm_kv_row_bytes(sch, hd);
            kv_q_write_row(blocks, f.data(), hd, sch);
            if (swlm_kv_is_rotor(sch) && which == 0 && m->desc.kv_qjl_dim > 0) qjl_store_residual(m, layer, b, head, t, f.data(), blocks);
        }
        return 0;
    }
    std::vector<uint16_t>& c = which ? m->vcache : m->kcache;
    std::memcpy(c.data() + kv_index(m, layer, b, head, 0), src, (size_t)count * m->desc.head_dim * 2);
    return 0;
}
// rotated schemes: all rotors [kv_layers][kv_heads][groups][4] fp16, and the projected K residuals [count][kv_qjl_dim]
int64_t orc_rotor_count(orc_model* m) { return (int64_t)m->rotors.size(); }
int orc_get_rotors(orc_model* m, uint16_t* dst) { std::memcpy(dst, m->rotors.data(), m->rotors.size() * 2); return 0; }
int orc_set_rotors(orc_model* m, const uint16_t* src) { std::memcpy(m->rotors.data(), src, m->rotors.size() * 2); return 0; }
int orc_get_qjl_matrix(orc_model* m, uint16_t* dst) { std::memcpy(dst, m->qjl_matrix.data(), m->qjl_matrix.size() * 2); return 0; }
int orc_read_qjl(orc_model* m, int layer, int b, int head, int count, uint16_t* dst) {
    if (m->qjl_res.empty()) return -1;
    std::memcpy(dst, qjl_row(m, layer, b, head, 0), (size_t)count * m->desc.kv_qjl_dim * 2);
    return 0;
}
int orc_add_dense_f32(orc_model* m, const char* name, int64_t count, const float* data) {
    m->densef[name].assign(data, data + count);
    return 0;
}
int orc_read_ssm_state(orc_model* m, int layer, int b, float* dst) {
    const swlm_buffers_desc& d = m->desc;
    size_t n = (size_t)d.ssm_heads * d.ssm_key_dim * d.ssm_value_dim;
    std::memcpy(dst, m->ssm_state.data() + ((size_t)layer * d.max_batch + b) * n, n * 4);
    return 0;
}
int orc_read_conv(orc_model* m, int layer, int b, uint16_t* dst) {
    const swlm_buffers_desc& d = m->desc;
    size_t n = (size_t)d.conv_kernel * d.conv_dim;
    std::memcpy(dst, m->conv.data() + ((size_t)layer * d.max_batch + b) * n, n * 2);
    return 0;
}

// ---- op-level entry points ----------------------------------------------------

// Dequantise a whole MLX-format matrix to fp32.
void orc_q4_dequant_mlx(int n, int k, const uint32_t* w, const uint16_t* scales_bf16,
                        const uint16_t* biases_bf16, float* out) {
    Q4Tensor t;
    t.n = n; t.k = k;
    t.w.assign(w, w + (size_t)n * (k / 8));
    size_t g = (size_t)n * (k / kGroup);
    t.scale.resize(g); t.zero.resize(g);
    for (size_t i = 0; i < g; ++i) { t.scale[i] = bf16_to_f32(scales_bf16[i]); t.zero[i] = bf16_to_f32(biases_bf16[i]); }
    for (int r = 0; r < n; ++r)
        for (int c = 0; c < k; ++c) out[(size_t)r * k + c] = dequant(t, r, c);
}

// repackMLXQuantized — Sources/MetalCompiler/STAF/STAFPayloadConverter.swift:209-282:
// per (row, group): fp16 scale, fp16 zero, then the group's 32 payload bytes verbatim.
void orc_staf_repack_mlx(int n, int k, const uint32_t* w, const uint16_t* scales_bf16,
                         const uint16_t* biases_bf16, uint8_t* blocks) {
    const int groups = k / kGroup;
    const uint8_t* wb = (const uint8_t*)w;
    for (int r = 0; r < n; ++r)
        for (int g = 0; g < groups; ++g) {
            uint8_t* blk = blocks + ((size_t)r * groups + g) * kBlockBytes;
            uint16_t s = f32_to_f16(bf16_to_f32(scales_bf16[(size_t)r * groups + g]));
            uint16_t z = f32_to_f16(bf16_to_f32(biases_bf16[(size_t)r * groups + g]));
            std::memcpy(blk, &s, 2);
            std::memcpy(blk + 2, &z, 2);
            std::memcpy(blk + 4, wb + (size_t)r * (k / 2) + (size_t)g * 32, 32);
        }
}

// The same repack and block dequant for a group of `group` weights (64: 36-byte blocks, 128: 68-byte blocks,
// AffineQ4Group128Format, Sources/MetalCompiler/STAF/QuantizationFormat.swift:539-604).
void orc_staf_repack_mlx_group(int n, int k, int group, const uint32_t* w, const uint16_t* scales_bf16,
                               const uint16_t* biases_bf16, uint8_t* blocks) {
    const int groups = k / group, block_bytes = 4 + group / 2;
    const uint8_t* wb = (const uint8_t*)w;
    for (int r = 0; r < n; ++r)
        for (int g = 0; g < groups; ++g) {
            uint8_t* blk = blocks + ((size_t)r * groups + g) * block_bytes;
            uint16_t s = f32_to_f16(bf16_to_f32(scales_bf16[(size_t)r * groups + g]));
            uint16_t z = f32_to_f16(bf16_to_f32(biases_bf16[(size_t)r * groups + g]));
            std::memcpy(blk, &s, 2);
            std::memcpy(blk + 2, &z, 2);
            std::memcpy(blk + 4, wb + (size_t)r * (k / 2) + (size_t)g * (group / 2), group / 2);
        }
}
void orc_q4_dequant_staf_group(int n, int k, int group, const uint8_t* blocks, float* out) {
    const int groups = k / group, block_bytes = 4 + group / 2;
    for (int r = 0; r < n; ++r)
        for (int g = 0; g < groups; ++g) {
            const uint8_t* blk = blocks + ((size_t)r * groups + g) * block_bytes;
            uint16_t sb, zb;
            std::memcpy(&sb, blk, 2);
            std::memcpy(&zb, blk + 2, 2);
            float s = f16_to_f32(sb), z = f16_to_f32(zb);
            for (int e = 0; e < group; ++e) {
                uint8_t byte = blk[4 + e / 2];
                uint8_t q = (e % 2 == 0) ? (byte & 0x0F) : (byte >> 4);   // Q4AffineMSL.perWeightExpression, :1084-1089
                out[(size_t)r * k + g * group + e] = s * (float)q + z;
            }
        }
}

// decodeQuantized — Sources/SwiftLM/CPUWeightStore.swift:109-174 (the reference's own CPU dequant).
void orc_q4_dequant_staf(int n, int k, const uint8_t* blocks, float* out) {
    const int groups = k / kGroup;
    for (int r = 0; r < n; ++r)
        for (int g = 0; g < groups; ++g) {
            const uint8_t* blk = blocks + ((size_t)r * groups + g) * kBlockBytes;
            uint16_t sb, zb;
            std::memcpy(&sb, blk, 2);
            std::memcpy(&zb, blk + 2, 2);
            float s = f16_to_f32(sb), z = f16_to_f32(zb);
            for (int e = 0; e < kGroup; ++e) {
                uint8_t byte = blk[4 + e / 2];
                uint8_t q = (e % 2 == 0) ? (byte & 0x0F) : (byte >> 4);
                out[(size_t)r * k + g * kGroup + e] = s * (float)q + z;
            }
        }
}

// generateUnifiedDequantToBFloat — Generator/MetalSourceGenerator+Quantized.swift:361-416.
void orc_q4_dequant_bf16(int n, int k, const uint32_t* w, const uint16_t* scales_bf16,
                         const uint16_t* biases_bf16, uint16_t* out) {
    std::vector<float> f((size_t)n * k);
    orc_q4_dequant_mlx(n, k, w, scales_bf16, biases_bf16, f.data());
    for (size_t i = 0; i < f.size(); ++i) out[i] = f32_to_bf16(f[i]);
}

// Y[m][n] = X[m][k] . W^T, bf16 in/out; y64 optional fp64 accumulation.
// staf_fp16: narrow scale/bias through fp16 first. x_is_f16: x holds fp16 (the
// reference's kernel tests feed fp16 activations), otherwise bf16.
int orc_qgemm_group(int m, int n, int k, int group, const uint16_t* x, const uint32_t* w, const uint16_t* scales_bf16,
                    const uint16_t* biases_bf16, uint16_t* y, double* y64, int staf_fp16);
int orc_qgemm(int m, int n, int k, const uint16_t* x, const uint32_t* w, const uint16_t* scales_bf16,
              const uint16_t* biases_bf16, uint16_t* y, double* y64, int staf_fp16) {
    return orc_qgemm_group(m, n, k, kGroup, x, w, scales_bf16, biases_bf16, y, y64, staf_fp16);
}
int orc_qgemm_group(int m, int n, int k, int group, const uint16_t* x, const uint32_t* w, const uint16_t* scales_bf16,
                    const uint16_t* biases_bf16, uint16_t* y, double* y64, int staf_fp16) {
    if ((group != 64 && group != 128) || k % group) return -1;
    Q4Tensor t;
    t.n = n; t.k = k; t.group = group;
    t.w.assign(w, w + (size_t)n * (k / 8));
    size_t g = (size_t)n * (k / group);
    t.scale.resize(g); t.zero.resize(g);
    for (size_t i = 0; i < g; ++i) {
        float s = bf16_to_f32(scales_bf16[i]), z = bf16_to_f32(biases_bf16[i]);
        if (staf_fp16) { s = f16_to_f32(f32_to_f16(s)); z = f16_to_f32(f32_to_f16(z)); }
        t.scale[i] = s; t.zero[i] = z;
    }
    qgemm(t, m, x, k, y, n, y64);
    return 0;
}

// Same dot product on an STAF block stream with fp32 activations and an fp32 result:
// the exact expression the reference's kernel tests evaluate on the CPU
// (Tests/MetalCompilerTests/Core/UnifiedGEMVBitLevelTests.swift:247-251).
void orc_staf_gemv_f32(int n, int k, const uint8_t* blocks, const float* x, float* y) {
    std::vector<float> wf((size_t)n * k);
    orc_q4_dequant_staf(n, k, blocks, wf.data());
    for (int r = 0; r < n; ++r) {
        float sum = 0.0f;
        for (int c = 0; c < k; ++c) sum += wf[(size_t)r * k + c] * x[c];
        y[r] = sum;
    }
}

// rotate-half RoPE on a bf16 vector in place (standalone `rope` kernel,
// Generator/MetalSourceGenerator+Attention.swift:337-351: result rounded to the buffer type).
void orc_rope_bf16(uint16_t* v, int heads, int head_dim, int rope_dim, float base, int position) {
    std::vector<float> f(head_dim);
    for (int h = 0; h < heads; ++h) {
        uint16_t* p = v + (size_t)h * head_dim;
        for (int i = 0; i < head_dim; ++i) f[i] = bf16_to_f32(p[i]);
        rope_inplace(f.data(), rope_dim, base, position);
        for (int i = 0; i < head_dim; ++i) p[i] = f32_to_bf16(f[i]);
    }
}

// inv_freq[i] = base^(-2i/ropeDim) in fp32, the table a backend may precompute.
void orc_rope_inv_freq(int rope_dim, float base, float* out) {
    for (int i = 0; i < rope_dim / 2; ++i) out[i] = std::pow(base, -2.0f * (float)i / (float)rope_dim);
}

}  // extern "C"
