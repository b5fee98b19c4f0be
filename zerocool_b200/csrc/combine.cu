// Weighted combine of the routed experts plus the gated shared expert, and the inter-layer glue of
// the chained-stack measurement.
//
// combine_kernel replaces moe_sum (kernels/metal/qwen.metal:804-816, dispatched at
// src/engine/model.cpp:553-555). The reduction order is part of the reference's contract (its test
// "expert reduction preserves the reference BF16 midpoint decision"): products j and j+8 are added
// first, then the eight partials in order, without fused multiply-add contraction. For a top_k other
// than 10 the same rule reads: partial_i = sum over j = i, i+8, ...; (partial_0 + partial_1), then
// + partial_2 ... + partial_7.
#include <algorithm>

#include "common.cuh"

namespace zc {
namespace {

constexpr int COMBINE_THREADS = 256;
constexpr int MAX_K = 32;

__device__ __forceinline__ float4 mul4(float4 y, float w) { return make_float4(__fmul_rn(y.x, w), __fmul_rn(y.y, w), __fmul_rn(y.z, w), __fmul_rn(y.w, w)); }
__device__ __forceinline__ float4 add4(float4 a, float4 b) {
    return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}

// Combined value of four consecutive columns of token t (before the output rounding). KMAX >= top_k is the
// compile-time slot count: every slot's 16 bytes (and the shared expert's) are requested before the first is
// used, so that a thread waits for one memory round trip, not one per slot. A slot whose id is invalid is read
// too (the buffer always holds T x K rows) and replaced by zero.
// NV: four-column vectors per thread, at col and col + vstride (a long batch takes two, so that twice the bytes are in
// flight per thread and the slot weights, ids and the gate are fetched once for both); a vector past the row's end is
// skipped. The arithmetic of every element is the same for any NV.
template <int KMAX, int NV>
__device__ __forceinline__ void combine_columns_n(const Call& c, uint32_t t, uint32_t col, uint32_t vstride, float (&r)[NV][4]) {
    const uint32_t stride = c.H / 4;
    float4 y[NV][KMAX];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const bool on = col + v * vstride < c.H;
        const float4* base = reinterpret_cast<const float4*>(c.expert_out + size_t(t) * c.K * c.H + col + v * vstride);
#pragma unroll
        for (int j = 0; j < KMAX; ++j) {
            y[v][j] = make_float4(0, 0, 0, 0);
            if (on && uint32_t(j) < c.K) y[v][j] = __ldcg(base + size_t(j) * stride);
        }
    }
    // Router weight and validity of every slot: the same addresses for the whole CTA (one broadcast transaction
    // per warp), requested together with the rows instead of through a staged copy and a barrier.
    float w[KMAX];
    int id[KMAX];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
        w[j] = 0.0f; id[j] = -1;
        if (uint32_t(j) < c.K) { w[j] = __ldcg(c.weights + size_t(t) * c.K + j); id[j] = __ldcg(c.ids + size_t(t) * c.K + j); }
    }
    float4 sh[NV];
    float gate_logit = 0.0f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        sh[v] = make_float4(0, 0, 0, 0);
        if (c.has_shared && col + v * vstride < c.H) sh[v] = __ldcg(reinterpret_cast<const float4*>(c.shared_out + size_t(t) * c.H + col + v * vstride));
    }
    if (c.has_shared) gate_logit = __ldcg(c.gate_logit + t);
    float gate = 0.0f;
    if (c.has_shared) gate = c.ref ? bf_round(sigmoid_bf(bf_round(gate_logit))) : sigmoid_f(gate_logit);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
#pragma unroll
        for (int j = 0; j < KMAX; ++j) {
            if (uint32_t(j) < c.K) y[v][j] = mul4(id[j] >= 0 ? y[v][j] : make_float4(0, 0, 0, 0), w[j]);
        }
        // partial_i = sum over j = i, i+8, ... in ascending j; then (partial_0 + partial_1) + partial_2 ...
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int j = i + 8; j < KMAX; j += 8) if (uint32_t(j) < c.K) y[v][i] = add4(y[v][i], y[v][j]);
        }
        float4 total = y[v][0];
#pragma unroll
        for (int i = 1; i < 8; ++i) if (uint32_t(i) < c.K) total = add4(total, y[v][i]);
        r[v][0] = total.x; r[v][1] = total.y; r[v][2] = total.z; r[v][3] = total.w;
        if (c.has_shared) {
            const float s4[4] = {sh[v].x, sh[v].y, sh[v].z, sh[v].w};
            if (c.ref) {
#pragma unroll
                for (int i = 0; i < 4; ++i) r[v][i] = bf_round(__fadd_rn(bf_round(r[v][i]), bf_round(__fmul_rn(gate, s4[i]))));
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) r[v][i] = __fadd_rn(r[v][i], __fmul_rn(gate, s4[i]));
            }
        } else if (c.ref) {
#pragma unroll
            for (int i = 0; i < 4; ++i) r[v][i] = bf_round(r[v][i]);
        }
    }
}
template <int KMAX>
__device__ __forceinline__ void combine_columns(const Call& c, uint32_t t, uint32_t col, float (&r)[4]) {
    float one[1][4];
    combine_columns_n<KMAX, 1>(c, t, col, 0, one);
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = one[0][i];
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

// Grid: (column blocks, tokens or fewer); a CTA walks the tokens blockIdx.y, blockIdx.y + gridDim.y, ... so that a long
// batch runs as a few resident waves instead of thousands of one-shot CTAs.
template <int KMAX>
__global__ void __launch_bounds__(COMBINE_THREADS) combine_kernel(Call c) {
    const uint32_t col = (blockIdx.x * COMBINE_THREADS + threadIdx.x) * 4;
    pdl_wait();
    pdl_launch_dependents();
    ep_wait_results(c);
    if (col >= c.H) return;
    for (uint32_t t = blockIdx.y; t < c.T; t += gridDim.y) {
        float r[4];
        combine_columns<KMAX>(c, t, col, r);
        store4(c.out, c.out_dtype, size_t(t) * c.H + col, r);
    }
}

// The same for a long batch: every thread takes two vectors of a token row, COMBINE_THREADS x 4 columns apart, and a
// CTA walks the tokens blockIdx.x, blockIdx.x + gridDim.x, ... (the grid is one resident wave).
template <int KMAX>
__global__ void __launch_bounds__(COMBINE_THREADS, 2) combine_long_kernel(Call c) {
    pdl_wait();
    pdl_launch_dependents();
    ep_wait_results(c);
    for (uint32_t t = blockIdx.x; t < c.T; t += gridDim.x) {
        for (uint32_t col = threadIdx.x * 4; col < c.H; col += COMBINE_THREADS * 8) {
            float r[2][4];
            combine_columns_n<KMAX, 2>(c, t, col, COMBINE_THREADS * 4, r);
            store4(c.out, c.out_dtype, size_t(t) * c.H + col, r[0]);
            if (col + COMBINE_THREADS * 4 < c.H) store4(c.out, c.out_dtype, size_t(t) * c.H + col + COMBINE_THREADS * 4, r[1]);
        }
    }
}

// combine + the inter-layer stand-in of the chained stack in one launch: one CTA per token computes the
// layer output (rounded to the output dtype, as a separate combine launch would have stored it), keeps it
// in shared memory, and writes next[t, :] = act_dtype((out - mean) / std): the stand-in for the residual + norm
// between MoE layers used when the stack is timed as one dependent chain. The mean is removed because the
// synthetic weights have a non-zero mean (codes 0..15 with bias -8 scale): without centring, that common
// component is amplified layer after layer until every token carries the same vector and routes to the same
// ten experts, which a real model's hidden states do not do.
// CN_THREADS: 512 for short batches (one pass over a 2048-wide row, the latency of a decode step), 256 for long ones
// (several CTAs per SM, so that the loads of one overlap the reductions of another); a CTA walks the tokens
// blockIdx.x, blockIdx.x + gridDim.x, ...
template <int KMAX, int CN_THREADS>
__global__ void __launch_bounds__(CN_THREADS) combine_norm_kernel(Call c, void* next, int next_dtype) {
    extern __shared__ float row[];          // [H]
    __shared__ float partial[CN_THREADS / 32];
    pdl_wait();
    pdl_launch_dependents();
    ep_wait_results(c);
    for (uint32_t t = blockIdx.x; t < c.T; t += gridDim.x) {
    float sum = 0.0f;
    constexpr int NV = CN_THREADS == 256 ? 2 : 1;          // the long-batch form keeps two vectors per thread in flight
    for (uint32_t col = threadIdx.x * 4; col < c.H; col += CN_THREADS * 4 * NV) {
        float r[NV][4];
        combine_columns_n<KMAX, NV>(c, t, col, CN_THREADS * 4, r);
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const uint32_t cv = col + v * CN_THREADS * 4;
            if (cv >= c.H) break;
#pragma unroll
            for (int i = 0; i < 4; ++i) { if (c.out_dtype != ZC_F32) r[v][i] = bf_round(r[v][i]); row[cv + i] = r[v][i]; sum += r[v][i]; }
        }
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
    __syncthreads();                        // the row is rewritten for the CTA's next token
    }
}

// Hyper-connection glue either side of the layer (the reference keeps four residual streams of width H).
// hc_mix_kernel replaces hc_mix (kernels/metal/qwen.metal:582-588, dispatched by Model::hyper, src/engine/model.cpp:343):
//   x[t, d] = bf( bf(bf(bf(p0 + p1) + p2) + p3) / 4 ),  p_h = bf(n[t, h, d] * mix[t, h, d])
// - the layer's input, written in the activation dtype the router and the expert kernels read (a BF16 value either way).
constexpr int HC_STREAMS = 4;
__global__ void __launch_bounds__(256) hc_mix_kernel(const float* __restrict__ n, const float* __restrict__ mix, uint32_t H, void* __restrict__ x, int x_dtype) {
    const uint32_t t = blockIdx.y, d = (blockIdx.x * 256 + threadIdx.x) * 4;
    if (d >= H) return;
    float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int h = 0; h < HC_STREAMS; ++h) {
        const size_t k = (size_t(t) * HC_STREAMS + h) * H + d;
        const float4 a = __ldcg(reinterpret_cast<const float4*>(n + k)), b = __ldcg(reinterpret_cast<const float4*>(mix + k));
        sum[0] = bf_round(__fadd_rn(sum[0], bf_round(__fmul_rn(a.x, b.x))));
        sum[1] = bf_round(__fadd_rn(sum[1], bf_round(__fmul_rn(a.y, b.y))));
        sum[2] = bf_round(__fadd_rn(sum[2], bf_round(__fmul_rn(a.z, b.z))));
        sum[3] = bf_round(__fadd_rn(sum[3], bf_round(__fmul_rn(a.w, b.w))));
    }
    float r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = bf_round(__fmul_rn(sum[i], 0.25f));
    store4(x, x_dtype, size_t(t) * H + d, r);
}

// combine_hc_kernel: the combine with hc_add (qwen.metal:589-595, dispatched at src/engine/model.cpp:660-662) as its
// epilogue: the layer output m[t, :] never goes to memory, the four residual streams are updated directly,
//   out[t, h, d] = bf( hyper[t, h, d] + bf( m[t, d] * inject[t, h] ) )
// (without the roundings outside the reference arithmetic; m is first rounded as the handle's output dtype would have stored it).
template <int KMAX>
__global__ void __launch_bounds__(COMBINE_THREADS) combine_hc_kernel(Call c, const float* __restrict__ hyper, const float* __restrict__ inject, float* __restrict__ out) {
    const uint32_t t = blockIdx.y;
    const uint32_t col = (blockIdx.x * COMBINE_THREADS + threadIdx.x) * 4;
    pdl_wait();
    pdl_launch_dependents();
    ep_wait_results(c);
    if (col >= c.H) return;
    float m[4];
    combine_columns<KMAX>(c, t, col, m);
    if (c.out_dtype != ZC_F32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) m[i] = bf_round(m[i]);
    }
#pragma unroll
    for (int h = 0; h < HC_STREAMS; ++h) {
        const size_t k = (size_t(t) * HC_STREAMS + h) * c.H + col;
        const float4 o = __ldcg(reinterpret_cast<const float4*>(hyper + k));
        const float inj = __ldcg(inject + size_t(t) * HC_STREAMS + h);
        const float base[4] = {o.x, o.y, o.z, o.w};
        float r[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float p = __fmul_rn(m[i], inj);
            r[i] = c.ref ? bf_round(__fadd_rn(base[i], bf_round(p))) : __fadd_rn(base[i], p);
        }
        *reinterpret_cast<float4*>(out + k) = make_float4(r[0], r[1], r[2], r[3]);
    }
}

// The BF16-staged activations of the reference arithmetic, element by element (parity hook).
__global__ void activation_table_kernel(const float* __restrict__ x, uint32_t n, float* __restrict__ sigmoid_out, float* __restrict__ silu_out) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i], sg = sigmoid_bf(v);
    if (sigmoid_out) sigmoid_out[i] = bf_round(sg);
    if (silu_out) silu_out[i] = bf_round(__fmul_rn(v, sg));
}

}  // namespace

int launch_activation_table(const float* x, uint32_t n, float* sigmoid_out, float* silu_out, cudaStream_t s) {
    activation_table_kernel<<<(n + 127) / 128, 128, 0, s>>>(x, n, sigmoid_out, silu_out);
    return check_launch(nullptr, "activation table");
}

int launch_hc_mix(zc_moe* m, const float* n, const float* mix, uint32_t T, uint32_t H, void* x, int x_dtype, cudaStream_t s) {
    Timed t(m, s, KERNEL_COMBINE);
    hc_mix_kernel<<<dim3((H / 4 + 255) / 256, T), 256, 0, s>>>(n, mix, H, x, x_dtype);
    const int rc = check_launch(m, "hc_mix");
    return rc < 0 ? rc : 1;
}

int launch_combine_hc(zc_moe* m, const Call& c, const float* hyper, const float* inject, float* out, cudaStream_t s) {
    if (c.K > MAX_K) return fail(m, ZC_EINVAL, "top_k above 32");
    const dim3 grid((c.H / 4 + COMBINE_THREADS - 1) / COMBINE_THREADS, c.T);
    int rc;
    { Timed t(m, s, KERNEL_COMBINE); auto k = c.K <= 8 ? combine_hc_kernel<8> : c.K <= 16 ? combine_hc_kernel<16> : combine_hc_kernel<32>;
      launch_chained(m, KERNEL_COMBINE, k, grid, dim3(COMBINE_THREADS), 0, s, nullptr, 0, c, hyper, inject, out);
      rc = check_launch(m, "combine + hc_add"); }
    return rc < 0 ? rc : 1;
}

int launch_combine(zc_moe* m, const Call& c, cudaStream_t s) {
    if (c.K > MAX_K) return fail(m, ZC_EINVAL, "top_k above 32");
    int rc;
    { Timed t(m, s, KERNEL_COMBINE);
      if (c.T > 128 && c.K <= 10) {          // two vectors of sixteen slots per thread do not fit the registers of two CTAs per SM
          auto k = c.K <= 8 ? combine_long_kernel<8> : combine_long_kernel<10>;
          launch_chained(m, KERNEL_COMBINE, k, dim3(std::min<uint32_t>(c.T, 2 * sm_count(m))), dim3(COMBINE_THREADS), 0, s, nullptr, 0, c);
      } else {
          const dim3 grid((c.H / 4 + COMBINE_THREADS - 1) / COMBINE_THREADS, c.T);
          auto k = c.K <= 8 ? combine_kernel<8> : c.K <= 10 ? combine_kernel<10> : c.K <= 16 ? combine_kernel<16> : combine_kernel<32>;
          launch_chained(m, KERNEL_COMBINE, k, grid, dim3(COMBINE_THREADS), 0, s, nullptr, 0, c);
      }
      rc = check_launch(m, "combine"); }
    return rc < 0 ? rc : 1;
}

int launch_combine_norm(zc_moe* m, const Call& c, void* next, int next_dtype, cudaStream_t s) {
    if (c.K > MAX_K) return fail(m, ZC_EINVAL, "top_k above 32");
    int rc;
    { Timed t(m, s, KERNEL_COMBINE); const size_t smem = c.H * sizeof(float);
      if (c.T <= 128 || c.K > 10) {
          auto k = c.K <= 8 ? combine_norm_kernel<8, 512> : c.K <= 10 ? combine_norm_kernel<10, 512> : c.K <= 16 ? combine_norm_kernel<16, 512> : combine_norm_kernel<32, 512>;
          launch_chained(m, KERNEL_COMBINE, k, dim3(c.T), dim3(512), smem, s, nullptr, 0, c, next, next_dtype);
      } else {
          auto k = c.K <= 8 ? combine_norm_kernel<8, 256> : combine_norm_kernel<10, 256>;
          launch_chained(m, KERNEL_COMBINE, k, dim3(std::min<uint32_t>(c.T, 2 * sm_count(m))), dim3(256), smem, s, nullptr, 0, c, next, next_dtype);
      }
      rc = check_launch(m, "combine_norm"); }
    return rc < 0 ? rc : 1;
}

}  // namespace zc
