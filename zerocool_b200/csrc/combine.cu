// Weighted combine of the routed experts plus the gated shared expert, and the inter-layer glue of
// the chained-stack measurement.
//
// combine_kernel replaces moe_sum (kernels/metal/qwen.metal:804-816, dispatched at
// src/engine/model.cpp:553-555). The reduction order is part of the reference's contract (its test
// "expert reduction preserves the reference BF16 midpoint decision"): products j and j+8 are added
// first, then the eight partials in order, without fused multiply-add contraction. For a top_k other
// than 10 the same rule reads: partial_i = sum over j = i, i+8, ...; (partial_0 + partial_1), then
// + partial_2 ... + partial_7.
#include "common.cuh"

namespace zc {
namespace {

constexpr int COMBINE_THREADS = 256;
constexpr int MAX_K = 32;

__device__ __forceinline__ float4 slot_product(const Call& c, uint32_t t, uint32_t j, uint32_t col, const float* w, const int* valid) {
    float4 y = make_float4(0, 0, 0, 0);
    if (valid[j]) y = *reinterpret_cast<const float4*>(c.expert_out + (size_t(t) * c.K + j) * c.H + col);
    return make_float4(__fmul_rn(y.x, w[j]), __fmul_rn(y.y, w[j]), __fmul_rn(y.z, w[j]), __fmul_rn(y.w, w[j]));
}
__device__ __forceinline__ float4 add4(float4 a, float4 b) {
    return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}

// Combined value of four consecutive columns of token t (before the output rounding).
__device__ __forceinline__ void combine_columns(const Call& c, uint32_t t, uint32_t col, const float* w, const int* valid, float (&r)[4]) {
    const uint32_t n = c.K < 8 ? c.K : 8;
    float4 partial[8];
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        if (i < n) {
            float4 p = slot_product(c, t, i, col, w, valid);
            for (uint32_t j = i + 8; j < c.K; j += 8) p = add4(p, slot_product(c, t, j, col, w, valid));
            partial[i] = p;
        }
    }
    float4 total = n > 1 ? add4(partial[0], partial[1]) : partial[0];
#pragma unroll
    for (uint32_t i = 2; i < 8; ++i) if (i < n) total = add4(total, partial[i]);
    r[0] = total.x; r[1] = total.y; r[2] = total.z; r[3] = total.w;
    if (c.has_shared) {
        const float4 sh = *reinterpret_cast<const float4*>(c.shared_out + size_t(t) * c.H + col);
        const float s[4] = {sh.x, sh.y, sh.z, sh.w};
        if (c.ref) {
            const float gate = bf_round(sigmoid_bf(bf_round(c.gate_logit[t])));
#pragma unroll
            for (int i = 0; i < 4; ++i) r[i] = bf_round(__fadd_rn(bf_round(r[i]), bf_round(__fmul_rn(gate, s[i]))));
        } else {
            const float gate = sigmoid_f(c.gate_logit[t]);
#pragma unroll
            for (int i = 0; i < 4; ++i) r[i] = __fadd_rn(r[i], __fmul_rn(gate, s[i]));
        }
    } else if (c.ref) {
#pragma unroll
        for (int i = 0; i < 4; ++i) r[i] = bf_round(r[i]);
    }
}
__device__ __forceinline__ void store4(void* base, int dtype, size_t index, const float (&r)[4]) {
    if (dtype == ZC_F32) {
        *reinterpret_cast<float4*>(static_cast<float*>(base) + index) = make_float4(r[0], r[1], r[2], r[3]);
    } else {
        const uint32_t lo = uint32_t(bf_bits(r[0])) | (uint32_t(bf_bits(r[1])) << 16);
        const uint32_t hi = uint32_t(bf_bits(r[2])) | (uint32_t(bf_bits(r[3])) << 16);
        *reinterpret_cast<uint2*>(static_cast<uint16_t*>(base) + index) = make_uint2(lo, hi);
    }
}

__global__ void __launch_bounds__(COMBINE_THREADS) combine_kernel(Call c) {
    const uint32_t t = blockIdx.y;
    const uint32_t col = (blockIdx.x * COMBINE_THREADS + threadIdx.x) * 4;
    __shared__ float w[MAX_K];
    __shared__ int valid[MAX_K];
    if (threadIdx.x < c.K) {
        w[threadIdx.x] = c.weights[size_t(t) * c.K + threadIdx.x];
        valid[threadIdx.x] = c.ids[size_t(t) * c.K + threadIdx.x] >= 0;
    }
    __syncthreads();
    if (col >= c.H) return;
    float r[4];
    combine_columns(c, t, col, w, valid, r);
    store4(c.out, c.out_dtype, size_t(t) * c.H + col, r);
}

// combine + the inter-layer stand-in of the chained stack in one launch: one CTA per token computes the
// layer output (rounded to the output dtype, as a separate combine launch would have stored it), keeps it
// in shared memory, and writes next[t, :] = act_dtype((out - mean) / std). See norm_act_kernel.
constexpr int CN_THREADS = 512;
__global__ void __launch_bounds__(CN_THREADS) combine_norm_kernel(Call c, void* next, int next_dtype) {
    extern __shared__ float row[];          // [H]
    __shared__ float w[MAX_K];
    __shared__ int valid[MAX_K];
    __shared__ float partial[CN_THREADS / 32];
    const uint32_t t = blockIdx.x;
    if (threadIdx.x < c.K) {
        w[threadIdx.x] = c.weights[size_t(t) * c.K + threadIdx.x];
        valid[threadIdx.x] = c.ids[size_t(t) * c.K + threadIdx.x] >= 0;
    }
    __syncthreads();
    float sum = 0.0f;
    for (uint32_t col = threadIdx.x * 4; col < c.H; col += CN_THREADS * 4) {
        float r[4];
        combine_columns(c, t, col, w, valid, r);
#pragma unroll
        for (int i = 0; i < 4; ++i) { if (c.out_dtype != ZC_F32) r[i] = bf_round(r[i]); row[col + i] = r[i]; sum += r[i]; }
    }
    auto block_total = [&](float v) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        __syncthreads();
        if (threadIdx.x % 32 == 0) partial[threadIdx.x / 32] = v;
        __syncthreads();
        float total = 0.0f;
        for (int i = 0; i < CN_THREADS / 32; ++i) total += partial[i];
        return total;
    };
    const float mean = block_total(sum) / float(c.H);
    float sq = 0.0f;
    for (uint32_t col = threadIdx.x * 4; col < c.H; col += CN_THREADS * 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float d = row[col + i] - mean; sq = __fmaf_rn(d, d, sq); }
    }
    const float var = block_total(sq) / float(c.H);
    const float scale = var > 0.0f ? __fdiv_rn(1.0f, sqrtf(var)) : 0.0f;
    for (uint32_t col = threadIdx.x * 4; col < c.H; col += CN_THREADS * 4) {
        float r[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) r[i] = __fmul_rn(row[col + i] - mean, scale);
        store4(next, next_dtype, size_t(t) * c.H + col, r);
    }
}

// x_next[t, :] = act_dtype((in[t, :] - mean) / std): the stand-in for the residual + norm between MoE
// layers used when the stack is timed as one dependent chain. The mean is removed because the synthetic
// weights have a non-zero mean (codes 0..15 with bias -8 scale): without centring, that common component
// is amplified layer after layer until every token carries the same vector and routes to the same ten
// experts, which a real model's hidden states do not do. One CTA per token.
constexpr int RMS_THREADS = 256;
__device__ __forceinline__ float block_sum(float v, float* partial) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();
    if (threadIdx.x % 32 == 0) partial[threadIdx.x / 32] = v;
    __syncthreads();
    float total = 0.0f;
    for (int i = 0; i < RMS_THREADS / 32; ++i) total += partial[i];
    return total;
}
__device__ __forceinline__ float load_as_float(const void* in, int dtype, size_t i) {
    return dtype == ZC_F32 ? static_cast<const float*>(in)[i] : bf_to_float(static_cast<const uint16_t*>(in)[i]);
}
__global__ void __launch_bounds__(RMS_THREADS) norm_act_kernel(const void* in, int in_dtype, void* out, int out_dtype, uint32_t H) {
    const uint32_t t = blockIdx.x;
    __shared__ float partial[RMS_THREADS / 32];
    float sum = 0.0f;
    for (uint32_t k = threadIdx.x; k < H; k += RMS_THREADS) sum += load_as_float(in, in_dtype, size_t(t) * H + k);
    const float mean = block_sum(sum, partial) / float(H);
    float sq = 0.0f;
    for (uint32_t k = threadIdx.x; k < H; k += RMS_THREADS) {
        const float d = load_as_float(in, in_dtype, size_t(t) * H + k) - mean;
        sq = __fmaf_rn(d, d, sq);
    }
    const float var = block_sum(sq, partial) / float(H);
    const float scale = var > 0.0f ? __fdiv_rn(1.0f, sqrtf(var)) : 0.0f;
    for (uint32_t k = threadIdx.x; k < H; k += RMS_THREADS) {
        const float r = __fmul_rn(load_as_float(in, in_dtype, size_t(t) * H + k) - mean, scale);
        if (out_dtype == ZC_F32) static_cast<float*>(out)[size_t(t) * H + k] = r;
        else static_cast<uint16_t*>(out)[size_t(t) * H + k] = bf_bits(r);
    }
}

}  // namespace

int launch_combine(zc_moe* m, const Call& c, cudaStream_t s) {
    if (c.K > MAX_K) return fail(m, ZC_EINVAL, "top_k above 32");
    const dim3 grid((c.H / 4 + COMBINE_THREADS - 1) / COMBINE_THREADS, c.T);
    int rc;
    { Timed t(m, s, KERNEL_COMBINE); combine_kernel<<<grid, COMBINE_THREADS, 0, s>>>(c); rc = check_launch(m, "combine"); }
    return rc < 0 ? rc : 1;
}

int launch_combine_norm(zc_moe* m, const Call& c, void* next, int next_dtype, cudaStream_t s) {
    if (c.K > MAX_K) return fail(m, ZC_EINVAL, "top_k above 32");
    int rc;
    { Timed t(m, s, KERNEL_COMBINE); combine_norm_kernel<<<c.T, CN_THREADS, c.H * sizeof(float), s>>>(c, next, next_dtype); rc = check_launch(m, "combine_norm"); }
    return rc < 0 ? rc : 1;
}

int launch_norm_act(zc_moe* m, const void* in, int in_dtype, void* out, int out_dtype, uint32_t T, uint32_t H, cudaStream_t s) {
    int rc;
    { Timed t(m, s, KERNEL_NORM_ACT); norm_act_kernel<<<T, RMS_THREADS, 0, s>>>(in, in_dtype, out, out_dtype, H); rc = check_launch(m, "norm_act"); }
    return rc < 0 ? rc : 1;
}

}  // namespace zc
