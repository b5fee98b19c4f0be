// Seeded synthetic layer tensors written straight into HBM.
//
// Device twin of zerocool_b200/synth.py (the definition): every byte is a pure function of
// (seed, layer, expert, projection, tensor kind, element index) through a splitmix64 counter hash, so
// the CPU checker can rebuild any record a GPU run used. All floating-point steps are single,
// individually rounded operations (no contraction), which keeps host and device bit-identical.
#include "common.cuh"
#include <cmath>

namespace zc {
namespace {

constexpr uint64_t GOLD = 0x9E3779B97F4A7C15ull, M1 = 0xBF58476D1CE4E5B9ull, M2 = 0x94D049BB133111EBull;
constexpr uint32_t KIND_CODES = 0, KIND_SCALES = 1, KIND_ROUTER = 2, KIND_SHARED_GATE = 3;
constexpr uint64_t SHARED_EXPERT = 0xFFFFFF;

__host__ __device__ inline uint64_t splitmix(uint64_t z) {
    z += GOLD;
    z = (z ^ (z >> 30)) * M1;
    z = (z ^ (z >> 27)) * M2;
    return z ^ (z >> 31);
}
__host__ __device__ inline uint64_t stream_key(uint64_t seed, uint64_t layer, uint64_t expert, uint64_t projection, uint64_t kind) {
    const uint64_t stream = (layer << 32) | (expert << 8) | (projection << 4) | kind;
    return splitmix(seed ^ splitmix(stream));
}
__device__ __forceinline__ uint32_t rand32(uint64_t key, uint64_t index) { return uint32_t(splitmix(key + index * GOLD) >> 32); }

struct SynthArgs {
    uint8_t* records; uint8_t* shared_record;
    uint64_t record_stride, seed;
    uint32_t layer, first_expert, local_experts, group;
    Projection proj[3], shared_proj[3];
    uint8_t meta_f16, q8_signed, has_shared;
};

// grid: (x, local_experts + has_shared, 3)
__global__ void fill_records_kernel(SynthArgs a) {
    const uint32_t slot = blockIdx.y, p = blockIdx.z;
    const bool shared = slot >= a.local_experts;
    uint8_t* record = shared ? a.shared_record : a.records + size_t(slot) * a.record_stride;
    const uint64_t expert = shared ? SHARED_EXPERT : uint64_t(a.first_expert + slot);
    const Projection pr = shared ? a.shared_proj[p] : a.proj[p];
    const uint64_t ck = stream_key(a.seed, a.layer, expert, p, KIND_CODES), sk = stream_key(a.seed, a.layer, expert, p, KIND_SCALES);
    const uint64_t stride = uint64_t(gridDim.x) * blockDim.x, first = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (pr.bits == 4) {
        uint32_t* words = reinterpret_cast<uint32_t*>(record + pr.codes);
        const uint64_t n = uint64_t(pr.N) * pr.K / 8;
        for (uint64_t i = first; i < n; i += stride) words[i] = rand32(ck, i);
    } else {
        uint8_t* codes = record + pr.codes;
        const uint64_t n = uint64_t(pr.N) * pr.K;
        for (uint64_t i = first; i < n; i += stride) {
            const uint32_t r = rand32(ck, i);
            codes[i] = a.q8_signed ? uint8_t(int8_t(int(r % 255u) - 127)) : uint8_t(r & 255u);
        }
    }
    uint16_t* s = reinterpret_cast<uint16_t*>(record + pr.scales);
    uint16_t* b = reinterpret_cast<uint16_t*>(record + pr.biases);
    const uint64_t nm = uint64_t(pr.N) * (pr.K / a.group);
    for (uint64_t i = first; i < nm; i += stride) {
        const float frac = __fmul_rn(float(rand32(sk, i) >> 8), 1.0f / 16777216.0f);
        const float scale = __fadd_rn(0.004f, __fmul_rn(0.016f, frac));
        if (a.meta_f16) {
            const __half h = __float2half_rn(scale);
            s[i] = __half_as_ushort(h);
            b[i] = __half_as_ushort(__float2half_rn(__fmul_rn(-8.0f, __half2float(h))));
        } else {
            const uint16_t sb = bf_bits(scale);
            s[i] = sb;
            b[i] = bf_bits(__fmul_rn(-8.0f, bf_to_float(sb)));
        }
    }
}

__global__ void fill_normal_kernel(void* dst, int dtype, uint64_t key, uint64_t n, float scale) {
    const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        int total = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) { const uint32_t r = rand32(key, i * 4 + j); total += int(r & 0xffffu) + int(r >> 16); }
        const float v = __fmul_rn(float(total - 262140), scale);
        if (dtype == ZC_F32) static_cast<float*>(dst)[i] = v;
        else static_cast<uint16_t*>(dst)[i] = bf_bits(v);
    }
}

}  // namespace

int launch_synth_layer(zc_moe* m, uint32_t layer, uint64_t seed, cudaStream_t s) {
    const zc_moe_desc& d = m->d;
    const LayerMem& L = m->layers[layer];
    SynthArgs a{};
    a.records = L.records; a.shared_record = L.shared_record;
    a.record_stride = d.record_stride; a.seed = seed; a.layer = layer;
    a.first_expert = d.first_expert; a.local_experts = d.local_experts; a.group = d.group;
    const zc_moe_desc sd = shared_desc_of(d);
    for (int p = 0; p < 3; ++p) { a.proj[p] = projection_of(d, p); a.shared_proj[p] = projection_of(sd, p); }
    a.meta_f16 = d.meta_dtype == ZC_F16; a.q8_signed = d.q8_signed; a.has_shared = d.has_shared;
    int launched = 0;
    fill_records_kernel<<<dim3(32, d.local_experts + (d.has_shared ? 1 : 0), 3), 256, 0, s>>>(a);
    int rc = check_launch(m, "synth records");
    if (rc < 0) return rc;
    ++launched;
    // sigma / std of a sum of eight 16-bit uniforms, computed in double and rounded once (as numpy does)
    const float scale = float(0.02 / (65536.0 * std::sqrt(8.0 / 12.0)));
    fill_normal_kernel<<<256, 256, 0, s>>>(L.router_w, d.router_dtype, stream_key(seed, layer, 0, 0, KIND_ROUTER), uint64_t(d.experts) * d.hidden, scale);
    rc = check_launch(m, "synth router");
    if (rc < 0) return rc;
    ++launched;
    if (d.has_shared) {
        fill_normal_kernel<<<8, 256, 0, s>>>(L.shared_gate_w, d.router_dtype, stream_key(seed, layer, 0, 0, KIND_SHARED_GATE), d.hidden, scale);
        rc = check_launch(m, "synth shared gate");
        if (rc < 0) return rc;
        ++launched;
    }
    return launched;
}

}  // namespace zc
