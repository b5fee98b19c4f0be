// Router logits (and the shared-expert gate scalar) in fp32 with a pinned accumulation order.
//
// Replaces router_mm + router_accumulate (kernels/metal/qwen.metal:512-534, launched from
// src/engine/metal.mm:818-822). The order is part of the contract because one last-bit change in a
// logit can flip a top-k decision: K is cut into sixteen contiguous partitions, each partition is a
// k-ascending chain of fused multiply-adds, and the sixteen partials are added in order 0..15.
//
// Mapping: a CTA owns ER consecutive router rows, staged once in shared memory, and walks the token
// batch in chunks of TT tokens. A thread owns one (row, partition) chain for TT/TG tokens; the
// sixteen partition owners of a row sit in one half-warp, so the ordered final sum is sixteen
// shuffles. Rows are padded by four floats so that the sixteen partitions of a row start in
// different banks for 128-bit reads.
#include "common.cuh"

namespace zc {
namespace {

constexpr int ER = 4;      // router rows per CTA
constexpr int TG = 2;      // token groups per chunk
constexpr int ROUTER_THREADS = ER * 16 * TG;

template <int TT>
__global__ void __launch_bounds__(ROUTER_THREADS) router_kernel(Call c, uint32_t chunks_per_block) {
    extern __shared__ __align__(16) float smem[];
    constexpr int TPT = TT / TG;
    const uint32_t H = c.H, part = H / 16, PS = part + 4;
    float* Ws = smem;                       // [ER][16][PS]
    float* Xs = smem + ER * 16 * PS;        // [TT][16][PS]
    const uint32_t rows_total = c.E + (c.has_shared ? 1u : 0u);
    const uint32_t e0 = blockIdx.x * ER;
    const uint32_t tid = threadIdx.x;

    // Stage this CTA's rows as fp32.
    const uint32_t quads = H / 4;
    for (uint32_t idx = tid; idx < ER * quads; idx += ROUTER_THREADS) {
        const uint32_t r = idx / quads, k = (idx % quads) * 4, e = e0 + r;
        float4 v = make_float4(0, 0, 0, 0);
        if (e < rows_total) {
            const void* base = e < c.E ? c.router_w : c.shared_gate_w;
            const size_t row = e < c.E ? e : 0;
            if (c.router_dtype == ZC_F32) {
                v = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(base) + row * H + k));
            } else {
                const uint2 raw = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(base) + row * H + k));
                v = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
            }
        }
        *reinterpret_cast<float4*>(Ws + (r * 16 + k / part) * PS + k % part) = v;
    }

    const uint32_t p = tid & 15, el = (tid >> 4) % ER, tg = tid / (16 * ER);
    const uint32_t lane = tid & 31;
    const uint32_t e = e0 + el;
    const float* wrow = Ws + (el * 16 + p) * PS;

    const uint32_t first_chunk = blockIdx.y * chunks_per_block;
    for (uint32_t ch = first_chunk; ch < first_chunk + chunks_per_block; ++ch) {
        const uint32_t t0 = ch * TT;
        if (t0 >= c.T) break;
        __syncthreads();   // previous chunk fully consumed (and Ws visible on the first pass)
        for (uint32_t idx = tid; idx < TT * quads; idx += ROUTER_THREADS) {
            const uint32_t tt = idx / quads, k = (idx % quads) * 4, t = t0 + tt;
            float4 v = make_float4(0, 0, 0, 0);
            if (t < c.T) {
                if (c.act_dtype == ZC_F32) {
                    v = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(c.x) + size_t(t) * H + k));
                } else {
                    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(c.x) + size_t(t) * H + k));
                    v = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                    __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
                }
            }
            *reinterpret_cast<float4*>(Xs + (tt * 16 + k / part) * PS + k % part) = v;
        }
        __syncthreads();

        float acc[TPT];
#pragma unroll
        for (int j = 0; j < TPT; ++j) acc[j] = 0.0f;
        for (uint32_t kk = 0; kk < part; kk += 4) {
            const float4 w = *reinterpret_cast<const float4*>(wrow + kk);
#pragma unroll
            for (int j = 0; j < TPT; ++j) {
                const float4 xv = *reinterpret_cast<const float4*>(Xs + ((tg * TPT + j) * 16 + p) * PS + kk);
                acc[j] = __fmaf_rn(xv.x, w.x, acc[j]);
                acc[j] = __fmaf_rn(xv.y, w.y, acc[j]);
                acc[j] = __fmaf_rn(xv.z, w.z, acc[j]);
                acc[j] = __fmaf_rn(xv.w, w.w, acc[j]);
            }
        }
        // Ordered sum of the sixteen partials; every lane of the half-warp computes it.
#pragma unroll
        for (int j = 0; j < TPT; ++j) {
            float sum = 0.0f;
#pragma unroll
            for (int q = 0; q < 16; ++q) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, acc[j], (lane & 16) + q));
            const uint32_t t = t0 + tg * TPT + j;
            if (p == 0 && t < c.T) {
                if (e < c.E) c.logits[size_t(t) * c.E + e] = sum;
                else if (e == c.E && c.has_shared) c.gate_logit[t] = sum;
            }
        }
    }
}

}  // namespace

int launch_router(zc_moe* m, const Call& c, cudaStream_t s) {
    constexpr int TT = 8;
    const uint32_t PS = c.H / 16 + 4;
    const size_t smem = size_t(ER + TT) * 16 * PS * sizeof(float);
    if (smem > 227 * 1024) return fail(m, ZC_EINVAL, "hidden too large for the router kernel");
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(router_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        configured = true;
    }
    const uint32_t rows = c.E + (c.has_shared ? 1 : 0);
    const uint32_t chunks = (c.T + TT - 1) / TT;
    const uint32_t gx = (rows + ER - 1) / ER;
    // One chunk of tokens per block while that keeps the grid within a few thousand blocks (the rows are
    // re-read from L2); longer batches walk several chunks per block.
    uint32_t gy = chunks < 32 ? chunks : 32;
    const uint32_t per = (chunks + gy - 1) / gy;
    gy = (chunks + per - 1) / per;
    int rc;
    { Timed t(m, s, KERNEL_ROUTER); router_kernel<TT><<<dim3(gx, gy), ROUTER_THREADS, smem, s>>>(c, per); rc = check_launch(m, "router"); }
    return rc < 0 ? rc : 1;
}

}  // namespace zc
