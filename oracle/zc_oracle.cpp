// TEST INFRASTRUCTURE — not part of the shipped library.
//
// CPU restatement of the ZeroCool Mixture-of-Experts layer arithmetic, used only as the checker
// for the CUDA path (tests, the smoke check and the CPU-baseline leg of the benchmark).
// Nothing in the product may call into this file.
//
// Every function names the reference source it follows (paths relative to the reference project):
//   kernels/metal/qwen.metal      bf :17-21, b16 :22, sigmoid_f :30-32, sigmoid_bf :33-35,
//                                 affine_dot :46-62, q4_gate_up :71-81, affine8_dot :112-125,
//                                 router_mm/router_accumulate :512-534, route :742-765,
//                                 route_simd :768-795, moe_sum :804-816
//   src/engine/model.cpp          Model::moe :431-557 (positions/selected :449-474)
//   src/engine/pipeline.cpp       encode_expert_rows :7-31
//   src/engine/metal.mm           expert_linear :1124-1129 (record layout)
//   src/engine/storage.cpp        round_bf16 :30-35, fp16 :36-41
//
// Two arithmetic modes:
//   arith = 1 ("reference"): every BF16 rounding boundary of the Metal kernels, including the
//            BF16-rounded sum-of-four that multiplies the affine bias in Q4.
//   arith = 0 ("fp32"): the same dataflow with plain fp32 sums and no intermediate rounding.
//
// Pinning: tests/test_oracle_golden.py checks this file against the known-answer vectors of the
// reference's own tests (tests/test_qwen.cpp :634-660, :661-696, :744-754, :755-797, :798-826,
// :827-842, :863-874, :876-897) and against scripts/qwen/reference_numpy.py imported unmodified.
// Apple's simd_sum order is not defined by the source; here it is a fixed xor butterfly.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

enum { DT_BF16 = 0, DT_F32 = 1, DT_F16 = 2 };

struct Desc {
    uint32_t hidden, ffn, experts, top_k, layers, group, max_tokens, first_expert, local_experts, reserved0;
    uint8_t gate_bits, up_bits, down_bits, q8_signed;
    uint8_t meta_dtype, act_dtype, out_dtype, router_dtype;
    uint8_t has_shared, arith, reserved[6];
    uint64_t record_bytes, record_stride;
};

inline uint32_t f2u(float v) { uint32_t u; std::memcpy(&u, &v, 4); return u; }
inline float u2f(uint32_t u) { float v; std::memcpy(&v, &u, 4); return v; }

// qwen.metal:17-21 / storage.cpp:30-35 — round to nearest-even bf16, NaN stays NaN.
inline float bf(float x) {
    uint32_t u = f2u(x);
    if ((u & 0x7fffffffu) > 0x7f800000u) return std::numeric_limits<float>::quiet_NaN();
    return u2f((u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u);
}
inline float b16(uint16_t v) { return u2f(uint32_t(v) << 16); }
// storage.cpp:36-41 — IEEE binary16 to float.
inline float f16(uint16_t v) {
    const int sign = (v & 0x8000) ? -1 : 1;
    const int exp = (v >> 10) & 31, frac = v & 1023;
    if (exp == 31) return frac ? std::numeric_limits<float>::quiet_NaN() : sign * std::numeric_limits<float>::infinity();
    return sign * (exp ? std::ldexp(float(1024 + frac), exp - 25) : std::ldexp(float(frac), -24));
}
inline float meta(const uint16_t* p, size_t i, int dtype) { return dtype == DT_F16 ? f16(p[i]) : b16(p[i]); }

// Metal precise::exp is taken as the correctly rounded single-precision exponential.
inline float exp_precise(float x) { return float(std::exp(double(x))); }
// qwen.metal:30-32
inline float sigmoid_f(float x) {
    float y = 1.0f / (1.0f + exp_precise(std::fabs(x)));
    return x < 0 ? y : 1.0f - y;
}
// qwen.metal:33-35
inline float sigmoid_bf(float x) {
    float y = bf(1.0f / bf(1.0f + bf(exp_precise(std::fabs(x)))));
    return x < 0 ? y : bf(1.0f - y);
}

// Stand-in for simd_sum: xor butterfly, offsets 16, 8, 4, 2, 1; lane 0's value is the result.
inline float simd_sum(float* lanes) {
    for (int off = 16; off >= 1; off >>= 1) {
        float next[32];
        for (int l = 0; l < 32; ++l) next[l] = lanes[l] + lanes[l ^ off];
        std::memcpy(lanes, next, sizeof(next));
    }
    return lanes[0];
}

// qwen.metal:46-62. `ref` selects the BF16 sum-of-four for the bias term.
float affine4_dot(const uint32_t* w, const uint16_t* s, const uint16_t* b, int mdt, const float* x,
                  uint32_t row, uint32_t K, uint32_t N, uint32_t group, bool ref) {
    const uint32_t width = (K % 512 == 0 && N % 8 == 0) ? 16 : 8;
    float lanes[32];
    for (uint32_t lane = 0; lane < 32; ++lane) {
        float result = 0;
        for (uint32_t base = lane * width; base < K; base += 32 * width) {
            float dot = 0, sum = 0;
            for (uint32_t i = 0; i < width && base + i < K; i += 4) {
                const uint32_t k = base + i, packed = (w[size_t(row) * (K / 8) + k / 8] >> (4 * (k % 8))) & 0xffff;
                const float a = x[k], c = x[k + 1], d = x[k + 2], e = x[k + 3];
                if (ref) sum += bf(bf(bf(a + c) + d) + e);
                else sum += ((a + c) + d) + e;
                float part = a * float(packed & 15);
                part += c * float((packed >> 4) & 15);
                part += d * float((packed >> 8) & 15);
                part += e * float((packed >> 12) & 15);
                dot += part;
            }
            const size_t g = size_t(row) * (K / group) + base / group;
            float term = meta(s, g, mdt) * dot;
            term += sum * meta(b, g, mdt);
            result += term;
        }
        lanes[lane] = result;
    }
    return simd_sum(lanes);
}

// qwen.metal:112-125. Codes are unsigned bytes in the reference; `is_signed` reads them as int8.
float affine8_dot(const uint8_t* w, const uint16_t* s, const uint16_t* b, int mdt, const float* x,
                  uint32_t row, uint32_t K, uint32_t N, uint32_t group, bool is_signed) {
    const uint32_t width = (K % 512 == 0 && N % 8 == 0) ? 8 : 4;
    float lanes[32];
    for (uint32_t lane = 0; lane < 32; ++lane) {
        float result = 0;
        for (uint32_t base = lane * width; base < K; base += 32 * width) {
            float dot = 0, sum = 0;
            for (uint32_t i = 0; i < width && base + i < K; ++i) {
                const float value = x[base + i];
                const uint8_t code = w[size_t(row) * K + base + i];
                sum += value;
                dot += value * (is_signed ? float(int8_t(code)) : float(code));
            }
            const size_t g = size_t(row) * (K / group) + base / group;
            float term = meta(s, g, mdt) * dot;
            term += sum * meta(b, g, mdt);
            result += term;
        }
        lanes[lane] = result;
    }
    return simd_sum(lanes);
}

struct Matrix {  // one projection inside a record: metal.mm:1124-1129 generalised
    const uint8_t* codes; const uint16_t* scales; const uint16_t* biases;
    uint32_t K, N, bits;
};
uint64_t projection_bytes(uint32_t N, uint32_t K, uint32_t bits, uint32_t group) {
    return uint64_t(N) * K * bits / 8 + 2 * uint64_t(N) * (K / group) * 2;
}
Matrix projection(const Desc& d, const uint8_t* record, int p) {
    const uint32_t bits[3] = {d.gate_bits, d.up_bits, d.down_bits};
    uint64_t offset = 0;
    for (int i = 0; i < p; ++i) offset += projection_bytes(i == 2 ? d.hidden : d.ffn, i == 2 ? d.ffn : d.hidden, bits[i], d.group);
    const uint32_t N = p == 2 ? d.hidden : d.ffn, K = p == 2 ? d.ffn : d.hidden;
    const uint64_t code_bytes = uint64_t(N) * K * bits[p] / 8, meta_bytes = uint64_t(N) * (K / d.group) * 2;
    return {record + offset, reinterpret_cast<const uint16_t*>(record + offset + code_bytes),
            reinterpret_cast<const uint16_t*>(record + offset + code_bytes + meta_bytes), K, N, bits[p]};
}
float affine_row(const Desc& d, const Matrix& m, const float* x, uint32_t row) {
    if (m.bits == 8)
        return affine8_dot(m.codes, m.scales, m.biases, d.meta_dtype, x, row, m.K, m.N, d.group, d.q8_signed);
    return affine4_dot(reinterpret_cast<const uint32_t*>(m.codes), m.scales, m.biases, d.meta_dtype, x, row, m.K, m.N, d.group, d.arith == 1);
}

// Router accumulation, qwen.metal:512-534 with metal.mm:818-822: sixteen contiguous K partitions,
// each a k-ascending fused multiply-add chain, partials added in order 0..15. This order
// reproduces the sixteen MLX bit patterns held by tests/test_qwen.cpp:810-813.
float router_dot(const float* x, const void* w, int wdt, size_t row, uint32_t H) {
    const uint32_t part = H / 16;
    float sum = 0;
    for (uint32_t s = 0; s < 16; ++s) {
        float c = 0;
        for (uint32_t k = s * part; k < (s + 1) * part; ++k) {
            const float wk = wdt == DT_F32 ? static_cast<const float*>(w)[row * H + k]
                                           : b16(static_cast<const uint16_t*>(w)[row * H + k]);
            c = std::fmaf(x[k], wk, c);
        }
        sum += c;
    }
    return sum;
}

// qwen.metal:742-765 (the serial kernel; route_simd :768-795 is bit-identical by the reference's
// own test): K largest logits, ties to the lower expert, only values > -inf can be selected.
void route_token(const float* logits, uint32_t E, uint32_t K, int32_t* ids, float* weights) {
    std::vector<float> scores(K, -std::numeric_limits<float>::infinity());
    std::vector<int32_t> selected(K, -1);
    for (uint32_t e = 0; e < E; ++e) {
        const float v = logits[e];
        for (uint32_t j = 0; j < K; ++j) if (v > scores[j]) {
            for (uint32_t k = K - 1; k > j; --k) { scores[k] = scores[k - 1]; selected[k] = selected[k - 1]; }
            scores[j] = v; selected[j] = int32_t(e); break;
        }
    }
    // Four values per lane, lane-sequential add, then the lane sum and a reciprocal.
    float lanes[32], values[128];
    for (uint32_t lane = 0; lane < 32; ++lane) {
        float sum = 0;
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t j = lane * 4 + i;
            const float v = j < K ? std::exp(scores[j] - scores[0]) : 0.0f;
            values[j] = v; sum += v;
        }
        lanes[lane] = sum;
    }
    const float inverse = 1.0f / simd_sum(lanes);
    for (uint32_t j = 0; j < K; ++j) { ids[j] = selected[j]; weights[j] = values[j] * inverse; }
}

// qwen.metal:804-816 generalised to any K: partial_i = sum of products j = i, i+8, ... ;
// (partial_0 + partial_1) then + partial_2 .. + partial_7; no contraction.
float combine_sum(const float* y, size_t stride, const float* w, uint32_t K) {
    float partial[8];
    const uint32_t n = K < 8 ? K : 8;
    for (uint32_t i = 0; i < n; ++i) {
        float p = y[i * stride] * w[i];
        for (uint32_t j = i + 8; j < K; j += 8) { float q = y[j * stride] * w[j]; p = p + q; }
        partial[i] = p;
    }
    float sum = n > 1 ? partial[0] + partial[1] : partial[0];
    for (uint32_t i = 2; i < n; ++i) sum = sum + partial[i];
    return sum;
}

// One expert on one row: qwen.metal:71-81 then q4_mm :63-70 (pipeline.cpp:24-29).
void expert_row(const Desc& d, const uint8_t* record, const float* x, float* h, float* y) {
    const Matrix g = projection(d, record, 0), u = projection(d, record, 1), dn = projection(d, record, 2);
    const bool ref = d.arith == 1;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < int64_t(d.ffn); ++r) {
        float gate = affine_row(d, g, x, uint32_t(r)), up = affine_row(d, u, x, uint32_t(r));
        if (ref) { gate = bf(gate); up = bf(up); h[r] = bf(bf(gate * sigmoid_bf(gate)) * up); }
        else h[r] = (gate * sigmoid_f(gate)) * up;
    }
    #pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < int64_t(d.hidden); ++c) {
        const float v = affine_row(d, dn, h, uint32_t(c));
        y[c] = ref ? bf(v) : v;
    }
}

}  // namespace

extern "C" {

// Optional additive per-expert bias on the router logits (the benchmark's skewed-load configuration); the
// reference's router has none. Applied after the partition sum.
static const float* g_router_bias = nullptr;
void zco_set_router_bias(const float* bias) { g_router_bias = bias; }

int zco_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void zco_set_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}

float zco_bf(float x) { return bf(x); }
float zco_sigmoid_bf(float x) { return sigmoid_bf(x); }
float zco_silu_bf(float x) { return bf(x * sigmoid_bf(x)); }  // unary op 0, qwen.metal:571,576

void zco_router_logits(const float* x, const void* w, int w_dtype, uint32_t T, uint32_t H, uint32_t E, float* logits) {
    #pragma omp parallel for schedule(static) collapse(2)
    for (int64_t t = 0; t < int64_t(T); ++t)
        for (int64_t e = 0; e < int64_t(E); ++e)
            logits[t * E + e] = router_dot(x + t * H, w, w_dtype, size_t(e), H) + (g_router_bias ? g_router_bias[e] : 0.0f);
}

void zco_route(const float* logits, uint32_t T, uint32_t E, uint32_t K, int32_t* ids, float* weights) {
    #pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < int64_t(T); ++t) route_token(logits + t * E, E, K, ids + t * K, weights + t * K);
}

// model.cpp:449-461 + pipeline.cpp:18-23 as one stable counting sort of slots p = t*K + j by
// expert id. Returns -1 when an id is outside [0, E) ("invalid router output", model.cpp:459).
int zco_permute(const int32_t* ids, uint32_t T, uint32_t K, uint32_t E, int32_t* offsets, int32_t* perm) {
    std::vector<int32_t> count(E, 0);
    for (uint32_t p = 0; p < T * K; ++p) { if (ids[p] < 0 || uint32_t(ids[p]) >= E) return -1; ++count[ids[p]]; }
    offsets[0] = 0;
    for (uint32_t e = 0; e < E; ++e) offsets[e + 1] = offsets[e] + count[e];
    std::vector<int32_t> cursor(offsets, offsets + E);
    for (uint32_t p = 0; p < T * K; ++p) perm[cursor[ids[p]]++] = int32_t(p);
    return 0;
}

// Metal::linear for an affine matrix (metal.mm:775-827): out[t, n]; round_out applies bf().
void zco_affine(uint32_t bits, int is_signed, int meta_dtype, int ref, const void* codes, const void* scales,
                const void* biases, uint32_t N, uint32_t K, uint32_t group, const float* x, uint32_t T,
                float* out, int round_out) {
    #pragma omp parallel for schedule(static) collapse(2)
    for (int64_t t = 0; t < int64_t(T); ++t)
        for (int64_t n = 0; n < int64_t(N); ++n) {
            const float v = bits == 8
                ? affine8_dot(static_cast<const uint8_t*>(codes), static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases), meta_dtype, x + t * K, uint32_t(n), K, N, group, is_signed)
                : affine4_dot(static_cast<const uint32_t*>(codes), static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases), meta_dtype, x + t * K, uint32_t(n), K, N, group, ref);
            out[t * N + n] = round_out ? bf(v) : v;
        }
}

// Metal::gated_linear (metal.mm:845-880) for one record: h[n, F] from x rows.
void zco_expert(const Desc* d, const uint8_t* record, const float* x, uint32_t n, float* h, float* y) {
    for (uint32_t i = 0; i < n; ++i) expert_row(*d, record, x + size_t(i) * d->hidden, h + size_t(i) * d->ffn, y + size_t(i) * d->hidden);
}

// moe_sum, qwen.metal:804-816. expert_out [T,K,H], weights [T,K], shared [T,H] or null, gate [T] or null.
void zco_combine(const Desc* d, const float* expert_out, const float* weights, const float* shared,
                 const float* gate, uint32_t T, float* out) {
    const uint32_t H = d->hidden, K = d->top_k;
    const bool ref = d->arith == 1;
    #pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < int64_t(T); ++t)
        for (uint32_t c = 0; c < H; ++c) {
            float sum = combine_sum(expert_out + (size_t(t) * K) * H + c, H, weights + t * K, K);
            if (shared) {
                if (ref) { float m = bf(sigmoid_bf(gate[t])) * shared[t * H + c]; sum = bf(bf(sum) + bf(m)); }
                else { float m = sigmoid_f(gate[t]) * shared[t * H + c]; sum = sum + m; }
            } else if (ref) sum = bf(sum);
            out[t * H + c] = sum;
        }
}

// Model::moe (model.cpp:431-557) for one layer. `records` holds E pointers (one record each; a
// pointer may be null when that expert is known not to be selected — selecting it returns -2).
// x is fp32 [T,H]. Outputs: out [T,H] fp32; ids/weights [T,K]; logits [T,E] (optional);
// expert_out [T,K,H] (optional); shared_out [T,H] and gate_out [T] (optional).
int zco_moe_layer(const Desc* dp, const uint8_t* const* records, const void* router_w, const uint8_t* shared_record,
                  const void* shared_gate_w, const float* x, uint32_t T, float* out, int32_t* ids, float* weights,
                  float* logits_out, float* expert_out_opt, float* shared_out_opt, float* gate_out_opt) {
    const Desc& d = *dp;
    const uint32_t H = d.hidden, F = d.ffn, E = d.experts, K = d.top_k;
    std::vector<float> logits_store;
    float* logits = logits_out;
    if (!logits) { logits_store.resize(size_t(T) * E); logits = logits_store.data(); }
    zco_router_logits(x, router_w, d.router_dtype, T, H, E, logits);
    zco_route(logits, T, E, K, ids, weights);
    std::vector<int32_t> offsets(E + 1), perm(size_t(T) * K);
    if (zco_permute(ids, T, K, E, offsets.data(), perm.data())) return -1;
    std::vector<float> eo_store;
    float* eo = expert_out_opt;
    if (!eo) { eo_store.resize(size_t(T) * K * H); eo = eo_store.data(); }
    std::vector<float> h(F);
    for (uint32_t e = 0; e < E; ++e)
        for (int32_t i = offsets[e]; i < offsets[e + 1]; ++i) {
            if (!records[e]) return -2;
            const int32_t p = perm[i];
            expert_row(d, records[e], x + size_t(p / K) * H, h.data(), eo + size_t(p) * H);
        }
    std::vector<float> shared, gate;
    if (d.has_shared) {
        shared.resize(size_t(T) * H); gate.resize(T);
        for (uint32_t t = 0; t < T; ++t) {
            expert_row(d, shared_record, x + size_t(t) * H, h.data(), shared.data() + size_t(t) * H);
            // Gate scalar (model.cpp:485, plain_mm qwen.metal:499-506): accumulated here with the
            // router's partition order so that one definition serves both dot products.
            const float g = router_dot(x + size_t(t) * H, shared_gate_w, d.router_dtype, 0, H);
            gate[t] = d.arith == 1 ? bf(g) : g;
        }
        if (shared_out_opt) std::memcpy(shared_out_opt, shared.data(), shared.size() * 4);
        if (gate_out_opt) std::memcpy(gate_out_opt, gate.data(), gate.size() * 4);
    }
    zco_combine(dp, eo, weights, d.has_shared ? shared.data() : nullptr, d.has_shared ? gate.data() : nullptr, T, out);
    return 0;
}

}  // extern "C"
