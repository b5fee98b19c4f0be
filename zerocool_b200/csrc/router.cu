// Router logits (and the shared-expert gate scalar) in fp32 with a pinned accumulation order.
//
// Replaces router_mm + router_accumulate (kernels/metal/qwen.metal:512-534, launched from
// src/engine/metal.mm:818-822) and keeps their structure: K is cut into sixteen contiguous partitions,
// each partition is a k-ascending chain of fused multiply-adds that one thread owns, the sixteen
// partials go to memory as [16, T, rows], and they are added in order 0..15 by the last of the sixteen
// partition CTAs of a tile to finish. The order is part of the contract
// because one last-bit change in a logit can flip a top-k decision; it reproduces the MLX bit patterns
// the reference's own test holds (tests/test_qwen.cpp:798-826).
//
// router_partial_kernel: grid (row tiles of 32, 16 partitions, token tiles). A CTA stages its slice of
// x (k-major) and of the router rows (k-major) in shared memory, then every thread runs its chains:
// TT = 64: 4 tokens x 2 rows per thread; TT = 8: one (token, row) per thread.
#include "common.cuh"
#include <cooperative_groups.h>

namespace zc {
namespace {

constexpr int ROUTER_THREADS = 256;
constexpr int ROW_TILE_PAD = 64;      // rows are padded to a multiple of this in the partials buffer

// TT tokens x ROW_TILE rows per CTA: TT = 8 -> 32 rows (one output per thread), TT = 16 -> 32 rows (two),
// TT = 32 -> 64 rows (four tokens x two rows per thread: eight chains share two shared-memory reads per k).
template <int TT>
__global__ void __launch_bounds__(ROUTER_THREADS) router_partial_kernel(Call c, float* __restrict__ partial, uint32_t rows_padded,
                                                                         uint32_t* __restrict__ tile_done, uint32_t reduce) {
    constexpr int ROW_TILE = TT == 32 ? 64 : 32;
    extern __shared__ __align__(16) float smem[];
    const uint32_t H = c.H, part = H / 16;
    float* xs = smem;                    // [part][TT]
    float* ws = smem + part * TT;        // [part][ROW_TILE]
    const uint32_t e0 = blockIdx.x * ROW_TILE, p = blockIdx.y, t0 = blockIdx.z * TT;
    const uint32_t rows_total = c.E + (c.has_shared ? 1u : 0u);
    const uint32_t tid = threadIdx.x;
    const uint32_t k0 = p * part;
    pdl_wait();

    // x slice -> xs[k][t]
    for (uint32_t task = tid; task < TT * (part / 8); task += ROUTER_THREADS) {
        const uint32_t tt = task % TT, kb = task / TT, t = t0 + tt;
        float v[8];
        if (t < c.T) {
            if (c.act_dtype == ZC_F32) {
                const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(c.x) + size_t(t) * H + k0 + kb * 8);
                const float4 a = __ldg(src), b = __ldg(src + 1);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            } else {
                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(c.x) + size_t(t) * H + k0 + kb * 8));
                const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(r[i] << 16); v[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u); }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) xs[(kb * 8 + i) * TT + tt] = v[i];
    }
    // router rows -> ws[k][e]; four loads are issued before their stores so that a thread pays the memory
    // latency once per batch, not once per 16 bytes
    const uint32_t wtasks = ROW_TILE * (part / 4);
    for (uint32_t first = tid; first < wtasks; first += 4 * ROUTER_THREADS) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t task = first + u * ROUTER_THREADS;
            v[u] = make_float4(0, 0, 0, 0);
            if (task < wtasks) {
                const uint32_t el = task % ROW_TILE, kq = task / ROW_TILE, e = e0 + el;
                if (e < rows_total) {
                    const void* base = e < c.E ? c.router_w : c.shared_gate_w;
                    const size_t row = e < c.E ? e : 0;
                    if (c.router_dtype == ZC_F32) {
                        v[u] = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(base) + row * H + k0 + kq * 4));
                    } else {
                        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(base) + row * H + k0 + kq * 4));
                        v[u] = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                           __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t task = first + u * ROUTER_THREADS;
            if (task < wtasks) {
                const uint32_t el = task % ROW_TILE, kq = task / ROW_TILE;
                ws[(kq * 4 + 0) * ROW_TILE + el] = v[u].x;
                ws[(kq * 4 + 1) * ROW_TILE + el] = v[u].y;
                ws[(kq * 4 + 2) * ROW_TILE + el] = v[u].z;
                ws[(kq * 4 + 3) * ROW_TILE + el] = v[u].w;
            }
        }
    }
    __syncthreads();

    if constexpr (TT == 64) {
        const uint32_t tx = tid % 16, ty = tid / 16;        // rows 2tx, 2tx+1; tokens 4ty .. 4ty+3
        float acc[4][2];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = 0.0f;
#pragma unroll 4
        for (uint32_t k = 0; k < part; ++k) {
            const float4 xv = *reinterpret_cast<const float4*>(xs + k * TT + ty * 4);
            const float2 wv = *reinterpret_cast<const float2*>(ws + k * ROW_TILE + tx * 2);
            acc[0][0] = __fmaf_rn(xv.x, wv.x, acc[0][0]); acc[0][1] = __fmaf_rn(xv.x, wv.y, acc[0][1]);
            acc[1][0] = __fmaf_rn(xv.y, wv.x, acc[1][0]); acc[1][1] = __fmaf_rn(xv.y, wv.y, acc[1][1]);
            acc[2][0] = __fmaf_rn(xv.z, wv.x, acc[2][0]); acc[2][1] = __fmaf_rn(xv.z, wv.y, acc[2][1]);
            acc[3][0] = __fmaf_rn(xv.w, wv.x, acc[3][0]); acc[3][1] = __fmaf_rn(xv.w, wv.y, acc[3][1]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t t = t0 + ty * 4 + i;
            if (t < c.T) *reinterpret_cast<float2*>(partial + (size_t(p) * c.T + t) * rows_padded + e0 + tx * 2) = make_float2(acc[i][0], acc[i][1]);
        }
    } else if constexpr (TT == 32) {
        const uint32_t tx = tid % 32, ty = tid / 32;        // rows 2tx, 2tx+1; tokens 4ty .. 4ty+3
        float acc[4][2];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = 0.0f;
#pragma unroll 4
        for (uint32_t k = 0; k < part; ++k) {
            const float4 xv = *reinterpret_cast<const float4*>(xs + k * TT + ty * 4);
            const float2 wv = *reinterpret_cast<const float2*>(ws + k * ROW_TILE + tx * 2);
            acc[0][0] = __fmaf_rn(xv.x, wv.x, acc[0][0]); acc[0][1] = __fmaf_rn(xv.x, wv.y, acc[0][1]);
            acc[1][0] = __fmaf_rn(xv.y, wv.x, acc[1][0]); acc[1][1] = __fmaf_rn(xv.y, wv.y, acc[1][1]);
            acc[2][0] = __fmaf_rn(xv.z, wv.x, acc[2][0]); acc[2][1] = __fmaf_rn(xv.z, wv.y, acc[2][1]);
            acc[3][0] = __fmaf_rn(xv.w, wv.x, acc[3][0]); acc[3][1] = __fmaf_rn(xv.w, wv.y, acc[3][1]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t t = t0 + ty * 4 + i;
            if (t < c.T) *reinterpret_cast<float2*>(partial + (size_t(p) * c.T + t) * rows_padded + e0 + tx * 2) = make_float2(acc[i][0], acc[i][1]);
        }
    } else if constexpr (TT == 16) {
        const uint32_t tx = tid % 16, ty = tid / 16;        // rows 2tx, 2tx+1; token ty
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll 8
        for (uint32_t k = 0; k < part; ++k) {
            const float xv = xs[k * TT + ty];
            const float2 wv = *reinterpret_cast<const float2*>(ws + k * ROW_TILE + tx * 2);
            a0 = __fmaf_rn(xv, wv.x, a0);
            a1 = __fmaf_rn(xv, wv.y, a1);
        }
        const uint32_t t = t0 + ty;
        if (t < c.T) *reinterpret_cast<float2*>(partial + (size_t(p) * c.T + t) * rows_padded + e0 + tx * 2) = make_float2(a0, a1);
    } else {
        const uint32_t el = tid % ROW_TILE, tt = tid / ROW_TILE;   // TT == 8
        float acc = 0.0f;
#pragma unroll 8
        for (uint32_t k = 0; k < part; ++k) acc = __fmaf_rn(xs[k * TT + tt], ws[k * ROW_TILE + el], acc);
        const uint32_t t = t0 + tt;
        if (t < c.T) partial[(size_t(p) * c.T + t) * rows_padded + e0 + el] = acc;
    }
    if (!reduce) return;
    // The last of the sixteen partition CTAs of this (row tile, token tile) adds the partials in order
    // 0..15, starting from zero like router_accumulate (qwen.metal:529-534).
    __shared__ bool last;
    __threadfence();
    __syncthreads();
    uint32_t* counter = tile_done + blockIdx.z * gridDim.x + blockIdx.x;
    if (tid == 0) last = atomicAdd(counter, 1u) == 15u;
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (tid == 0) *counter = 0;
    constexpr int PER = TT * ROW_TILE / ROUTER_THREADS;      // outputs per thread: 1, 2 or 8
    constexpr int BATCH = PER < 4 ? PER : 4;                 // outputs whose 16 loads are in flight together
#pragma unroll 1
    for (int b = 0; b < PER; b += BATCH) {
        float v[BATCH][16];
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            const uint32_t o = tid + (b + i) * ROUTER_THREADS, tt = o / ROW_TILE, el = o % ROW_TILE, t = t0 + tt, e = e0 + el;
            const bool live = t < c.T && e < rows_total;
#pragma unroll
            for (uint32_t q = 0; q < 16; ++q) v[i][q] = live ? __ldcg(partial + (size_t(q) * c.T + t) * rows_padded + e) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            const uint32_t o = tid + (b + i) * ROUTER_THREADS, tt = o / ROW_TILE, el = o % ROW_TILE, t = t0 + tt, e = e0 + el;
            if (t >= c.T || e >= rows_total) continue;
            float sum = 0.0f;
#pragma unroll
            for (uint32_t q = 0; q < 16; ++q) sum = __fadd_rn(sum, v[i][q]);
            if (e < c.E) c.logits[size_t(t) * c.E + e] = c.router_bias ? __fadd_rn(sum, c.router_bias[e]) : sum;
            else c.gate_logit[t] = sum;
        }
    }
}


// ---------------------------------------------------------------------------------------------------------
// Cluster form of the same computation, used whenever the device can host its clusters. A thread-block
// cluster of eight CTAs covers the sixteen partitions of one (row tile, token tile): CTA r computes
// partitions 2r and 2r+1. The partials never leave the chip: each CTA leaves its two [TT][rows] partial tiles in
// its shared memory, and after one cluster barrier every CTA adds, in order 0..15 from zero, the sixteen
// partials of its eighth of the outputs, read from its peers' shared memory. Compared with the global-memory
// form this removes the partial store, the fence, the arrival counter and the tail that one CTA ran alone.
//
// Staging: x and the router rows keep their row-major [row][k] layout in shared memory (leading dimension
// KC + 4 floats, which spreads eight consecutive rows over all banks for 16-byte reads), so fp32 rows are
// copied with 16-byte cp.async and everything is in flight at once: one memory round trip before the chains.
// Thread (tx = lane, ty = warp) owns rows tx (and tx + 32) x tokens ty*TPT.. x both partitions: up to 32
// independent chains, each still the k-ascending fused multiply-add chain of its partition.
namespace cg = cooperative_groups;
#ifndef ZC_ROUTER_SMALL_T
#define ZC_ROUTER_SMALL_T 128
#endif
constexpr int CLUSTER_PARTS = 2;                      // partitions per CTA
constexpr int CLUSTER_SIZE = 16 / CLUSTER_PARTS;

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(uint32_t(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}

template <int TT, int RPT>
__global__ void __launch_bounds__(ROUTER_THREADS) router_cluster_kernel(Call c) {
    constexpr int ROW_TILE = 32 * RPT, TPT = TT / 8;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ __align__(16) float smem[];
    const uint32_t H = c.H, part = H / 16, KC = CLUSTER_PARTS * part, LD = KC + 4;
    float* ws = smem;                         // [ROW_TILE][LD]
    float* xs = ws + ROW_TILE * LD;           // [TT][LD]
    float* ps = xs + TT * LD;                 // [2][TT][ROW_TILE]
    const uint32_t e0 = blockIdx.x * ROW_TILE, cr = blockIdx.y, t0 = blockIdx.z * TT;
    const uint32_t rows_total = c.E + (c.has_shared ? 1u : 0u);
    const uint32_t tid = threadIdx.x, k0 = cr * KC;

    // ---- stage: the rows first (weights), then x (registers when it needs a conversion) ----
    constexpr int XB = 4;                     // x tasks (8 values each) a thread keeps in flight
    const uint32_t xtasks = TT * (KC / 8);
    const bool x32 = c.act_dtype == ZC_F32, w32 = c.router_dtype == ZC_F32;
    auto stage_rows = [&]() {
        const uint32_t wtasks = ROW_TILE * (KC / 4);
        if (w32) {
            for (uint32_t task = tid; task < wtasks; task += ROUTER_THREADS) {
                const uint32_t el = task / (KC / 4), kq = task % (KC / 4), e = e0 + el;
                float* dst = ws + el * LD + kq * 4;
                if (e < rows_total) {
                    const float* base = e < c.E ? static_cast<const float*>(c.router_w) + size_t(e) * H : static_cast<const float*>(c.shared_gate_w);
                    cp_async16(dst, base + k0 + kq * 4);
                } else {
                    *reinterpret_cast<float4*>(dst) = make_float4(0, 0, 0, 0);
                }
            }
        } else {
            for (uint32_t first = tid; first < wtasks; first += 4 * ROUTER_THREADS) {
                uint2 raw[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t task = first + u * ROUTER_THREADS;
                    raw[u] = make_uint2(0, 0);
                    if (task < wtasks) {
                        const uint32_t el = task / (KC / 4), kq = task % (KC / 4), e = e0 + el;
                        if (e < rows_total) {
                            const uint16_t* base = e < c.E ? static_cast<const uint16_t*>(c.router_w) + size_t(e) * H : static_cast<const uint16_t*>(c.shared_gate_w);
                            raw[u] = __ldg(reinterpret_cast<const uint2*>(base + k0 + kq * 4));
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t task = first + u * ROUTER_THREADS;
                    if (task < wtasks) {
                        const uint32_t el = task / (KC / 4), kq = task % (KC / 4);
                        *reinterpret_cast<float4*>(ws + el * LD + kq * 4) =
                            make_float4(__uint_as_float(raw[u].x << 16), __uint_as_float(raw[u].x & 0xffff0000u),
                                        __uint_as_float(raw[u].y << 16), __uint_as_float(raw[u].y & 0xffff0000u));
                    }
                }
            }
        }
    };
    // The router rows are weights: their copies start before the previous kernel of the chain has finished.
    stage_rows();
    pdl_wait();
    pdl_launch_dependents();
    if (x32) {
        for (uint32_t task = tid; task < xtasks * 2; task += ROUTER_THREADS) {       // 16-byte pieces
            const uint32_t tt = task / (KC / 4), kq = task % (KC / 4), t = t0 + tt;
            float* dst = xs + tt * LD + kq * 4;
            if (t < c.T) cp_async16(dst, static_cast<const float*>(c.x) + size_t(t) * H + k0 + kq * 4);
            else *reinterpret_cast<float4*>(dst) = make_float4(0, 0, 0, 0);
        }
    } else {
        for (uint32_t first = tid; first < xtasks; first += XB * ROUTER_THREADS) {
            uint4 raw[XB];
#pragma unroll
            for (int u = 0; u < XB; ++u) {
                const uint32_t task = first + u * ROUTER_THREADS;
                raw[u] = make_uint4(0, 0, 0, 0);
                if (task < xtasks) {
                    const uint32_t tt = task / (KC / 8), kb = task % (KC / 8), t = t0 + tt;
                    if (t < c.T) raw[u] = __ldcg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(c.x) + size_t(t) * H + k0 + kb * 8));
                }
            }
#pragma unroll
            for (int u = 0; u < XB; ++u) {
                const uint32_t task = first + u * ROUTER_THREADS;
                if (task < xtasks) {
                    const uint32_t tt = task / (KC / 8), kb = task % (KC / 8);
                    const uint32_t r[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
                    float4* dst = reinterpret_cast<float4*>(xs + tt * LD + kb * 8);
                    dst[0] = make_float4(__uint_as_float(r[0] << 16), __uint_as_float(r[0] & 0xffff0000u), __uint_as_float(r[1] << 16), __uint_as_float(r[1] & 0xffff0000u));
                    dst[1] = make_float4(__uint_as_float(r[2] << 16), __uint_as_float(r[2] & 0xffff0000u), __uint_as_float(r[3] << 16), __uint_as_float(r[3] & 0xffff0000u));
                }
            }
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // ---- chains ----
    const uint32_t tx = tid % 32, ty = tid / 32;
    float acc[CLUSTER_PARTS][TPT][RPT];
#pragma unroll
    for (int pp = 0; pp < CLUSTER_PARTS; ++pp)
#pragma unroll
        for (int j = 0; j < TPT; ++j)
#pragma unroll
            for (int i = 0; i < RPT; ++i) acc[pp][j][i] = 0.0f;
    const float* wrow = ws + tx * LD;
    const float* xrow = xs + ty * TPT * LD;
#pragma unroll 2
    for (uint32_t k = 0; k < part; k += 4) {
#pragma unroll
        for (int pp = 0; pp < CLUSTER_PARTS; ++pp) {
            float4 wv[RPT], xv[TPT];
#pragma unroll
            for (int i = 0; i < RPT; ++i) wv[i] = *reinterpret_cast<const float4*>(wrow + i * 32 * LD + pp * part + k);
#pragma unroll
            for (int j = 0; j < TPT; ++j) xv[j] = *reinterpret_cast<const float4*>(xrow + j * LD + pp * part + k);
#pragma unroll
            for (int j = 0; j < TPT; ++j)
#pragma unroll
                for (int i = 0; i < RPT; ++i) {
                    float a = acc[pp][j][i];
                    a = __fmaf_rn(xv[j].x, wv[i].x, a);
                    a = __fmaf_rn(xv[j].y, wv[i].y, a);
                    a = __fmaf_rn(xv[j].z, wv[i].z, a);
                    a = __fmaf_rn(xv[j].w, wv[i].w, a);
                    acc[pp][j][i] = a;
                }
        }
    }
#pragma unroll
    for (int pp = 0; pp < CLUSTER_PARTS; ++pp)
#pragma unroll
        for (int j = 0; j < TPT; ++j)
#pragma unroll
            for (int i = 0; i < RPT; ++i) ps[(pp * TT + ty * TPT + j) * ROW_TILE + tx + 32 * i] = acc[pp][j][i];
    cluster.sync();

    // ---- ordered sum of the sixteen partials (router_accumulate, qwen.metal:529-534) for this CTA's outputs ----
    constexpr uint32_t OUT_PER_CTA = TT * ROW_TILE / CLUSTER_SIZE;
    for (uint32_t o = cr * OUT_PER_CTA + tid; o < (cr + 1) * OUT_PER_CTA; o += ROUTER_THREADS) {
        const uint32_t tt = o / ROW_TILE, el = o % ROW_TILE, t = t0 + tt, e = e0 + el;
        float v[16];
#pragma unroll
        for (uint32_t q = 0; q < 16; ++q) {
            const float* remote = cluster.map_shared_rank(ps + ((q % CLUSTER_PARTS) * TT + tt) * ROW_TILE + el, q / CLUSTER_PARTS);
            v[q] = *remote;
        }
        float sum = 0.0f;
#pragma unroll
        for (uint32_t q = 0; q < 16; ++q) sum = __fadd_rn(sum, v[q]);
        if (t < c.T && e < rows_total) {
            if (e < c.E) c.logits[size_t(t) * c.E + e] = c.router_bias ? __fadd_rn(sum, c.router_bias[e]) : sum;
            else c.gate_logit[t] = sum;
        }
    }
    cluster.sync();          // nobody leaves while a peer may still read its partials
}

template <int TT, int RPT>
int launch_router_cluster(zc_moe* m, const Call& c, cudaStream_t s) {
    constexpr int ROW_TILE = 32 * RPT;
    const uint32_t KC = CLUSTER_PARTS * (c.H / 16), LD = KC + 4;
    const size_t smem = (size_t(ROW_TILE + TT) * LD + size_t(CLUSTER_PARTS) * TT * ROW_TILE) * sizeof(float);
    const uint32_t rows_total = c.E + (c.has_shared ? 1 : 0);
    auto kernel = router_cluster_kernel<TT, RPT>;
    const dim3 grid((rows_total + ROW_TILE - 1) / ROW_TILE, CLUSTER_SIZE, (c.T + TT - 1) / TT);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = CLUSTER_SIZE; attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg{};           // for the occupancy query
    cfg.gridDim = grid; cfg.blockDim = dim3(ROUTER_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cfg.attrs = attr; cfg.numAttrs = 1;
    static SmemOptIn configured;        // per instantiation, per device
    static int8_t usable[MAX_DEVICES];  // per device: 0 unknown, 1 the device hosts a cluster of this shape, 2 it cannot
    if (smem > 224 * 1024 || m->device < 0 || m->device >= MAX_DEVICES) return 0;
    if (smem > configured.bytes[m->device]) {
        if (opt_in_smem(kernel, configured, m->device, smem) != cudaSuccess) { cudaGetLastError(); return 0; }
        usable[m->device] = 0;
    }
    if (usable[m->device] == 0) {
        int clusters = 0;
        const cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg);
        if (e != cudaSuccess) cudaGetLastError();
        usable[m->device] = (e == cudaSuccess && clusters > 0) ? 1 : 2;
    }
    if (usable[m->device] != 1) return 0;
    int rc;
    {
        Timed t(m, s, KERNEL_ROUTER);
        // Early launch pays for short batches (the row prefetch hides behind the previous kernel); from 64 tokens on
        // the prefetch of several token tiles competes with that kernel and measured 2 % slower per layer.
        const cudaError_t e = launch_chained(m, c.T <= 32 ? int(KERNEL_ROUTER) : -1, kernel, grid, dim3(ROUTER_THREADS), smem, s, attr, 1, c);
        if (e != cudaSuccess) return fail(m, ZC_EEXEC, std::string("router (cluster) launch: ") + cudaGetErrorString(e));
        rc = check_launch(m, "router");
    }
    return rc < 0 ? rc : 1;
}

// ---------------------------------------------------------------------------------------------------------
// Long batches: one CTA owns a 64-token x 64-row tile of the logits for the whole of K. It walks the sixteen
// partitions in order; inside a partition every (token, row) pair is the k-ascending chain of fused multiply-adds,
// and the finished partial is added to the pair's running total - the same additions in the same order as the
// partition kernels above ("partials added 0..15 starting from zero"), but nothing leaves the registers: no partial
// store, no arrival counter, no ordered re-read. Thread (tx, ty) holds rows tx + 16 i and tokens 4 ty + j (i, j < 4):
// sixteen independent chains, fed by four row reads and four broadcast token reads per four k, which keeps the
// kernel bound by the FP32 pipe and not by shared memory. Tiles keep the row-major [row][k] layout (leading
// dimension part + 4 floats), so FP32 router rows are copied with 16-byte cp.async.
constexpr int LONG_TT = 64, LONG_RT = 64;
#ifndef ZC_RL_ROWS
#define ZC_RL_ROWS 4          // rows x tokens per thread: 4 x 4 chains, 256 threads (8 x 4 with 128 threads measured 20 % slower)
#endif
#ifndef ZC_RL_UNROLL
#define ZC_RL_UNROLL 2
#endif
#ifndef ZC_RL_BLOCKS
#define ZC_RL_BLOCKS 2
#endif
#define ZC_PRAGMA(x) _Pragma(#x)
#define ZC_UNROLL(n) ZC_PRAGMA(unroll n)
constexpr int LONG_RI = ZC_RL_ROWS, LONG_TJ = 4;
constexpr int LONG_TXN = LONG_RT / LONG_RI, LONG_TYN = LONG_TT / LONG_TJ, LONG_THREADS = LONG_TXN * LONG_TYN;
// Thread (tx, ty) owns rows tx + TXN i and tokens ty + TYN j: the lanes of a warp read consecutive rows of either tile,
// which the row pitch of part + 4 floats spreads over all banks (one wavefront per 128 distinct bytes).
__global__ void __launch_bounds__(LONG_THREADS, ZC_RL_BLOCKS) router_long_kernel(Call c) {
    extern __shared__ __align__(16) float smem[];
    const uint32_t H = c.H, part = H / 16, LD = part + 4;
    float* ws = smem;                       // [LONG_RT][LD]
    float* xs = ws + LONG_RT * LD;          // [LONG_TT][LD]
    const uint32_t e0 = blockIdx.x * LONG_RT, t0 = blockIdx.y * LONG_TT;
    const uint32_t rows_total = c.E + (c.has_shared ? 1u : 0u);
    const uint32_t tid = threadIdx.x, tx = tid % LONG_TXN, ty = tid / LONG_TXN, warp = tid / 32, lane = tid % 32;
    const bool x32 = c.act_dtype == ZC_F32, w32 = c.router_dtype == ZC_F32;
    const uint32_t rows_here = min(uint32_t(LONG_RT), rows_total - e0);
    const bool narrow = rows_here <= LONG_THREADS / LONG_TT;
    float total[LONG_RI][LONG_TJ];
#pragma unroll
    for (int i = 0; i < LONG_RI; ++i)
#pragma unroll
        for (int j = 0; j < LONG_TJ; ++j) total[i][j] = 0.0f;
    pdl_wait();
    for (uint32_t p = 0; p < 16; ++p) {
        const uint32_t k0 = p * part;
        __syncthreads();                     // the previous partition's tiles have been consumed
        // Staging without divisions: warp w copies rows w, w + warps, ... of both tiles, its lanes walk the row.
        for (uint32_t el = warp; el < (narrow ? rows_here : uint32_t(LONG_RT)); el += LONG_THREADS / 32) {
            const uint32_t e = e0 + el;
            float* dst = ws + el * LD;
            if (e >= rows_total) {
                for (uint32_t kq = lane; kq < part / 4; kq += 32) *reinterpret_cast<float4*>(dst + kq * 4) = make_float4(0, 0, 0, 0);
            } else if (w32) {
                const float* base = (e < c.E ? static_cast<const float*>(c.router_w) + size_t(e) * H : static_cast<const float*>(c.shared_gate_w)) + k0;
                for (uint32_t kq = lane; kq < part / 4; kq += 32) cp_async16(dst + kq * 4, base + kq * 4);
            } else {
                const uint16_t* base = (e < c.E ? static_cast<const uint16_t*>(c.router_w) + size_t(e) * H : static_cast<const uint16_t*>(c.shared_gate_w)) + k0;
                for (uint32_t kq = lane; kq < part / 4; kq += 32) {
                    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(base + kq * 4));
                    *reinterpret_cast<float4*>(dst + kq * 4) = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                                                           __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
                }
            }
        }
        if (x32) {
            for (uint32_t tt = warp; tt < LONG_TT; tt += LONG_THREADS / 32) {
                const uint32_t t = t0 + tt;
                float* dst = xs + tt * LD;
                if (t < c.T) { const float* base = static_cast<const float*>(c.x) + size_t(t) * H + k0; for (uint32_t kq = lane; kq < part / 4; kq += 32) cp_async16(dst + kq * 4, base + kq * 4); }
                else for (uint32_t kq = lane; kq < part / 4; kq += 32) *reinterpret_cast<float4*>(dst + kq * 4) = make_float4(0, 0, 0, 0);
            }
        } else {
            // BF16 rows: 16 bytes = eight values per lane; a half-warp takes a row (two rows per pass of the warp)
            for (uint32_t tt = warp * 2 + lane / 16; tt < LONG_TT; tt += LONG_THREADS / 16) {
                const uint32_t t = t0 + tt;
                const uint16_t* base = static_cast<const uint16_t*>(c.x) + size_t(t) * H + k0;
                for (uint32_t kb = lane % 16; kb < part / 8; kb += 16) {
                    uint4 raw = make_uint4(0, 0, 0, 0);
                    if (t < c.T) raw = __ldcg(reinterpret_cast<const uint4*>(base + kb * 8));
                    float4* dst = reinterpret_cast<float4*>(xs + tt * LD + kb * 8);
                    dst[0] = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
                    dst[1] = make_float4(__uint_as_float(raw.z << 16), __uint_as_float(raw.z & 0xffff0000u), __uint_as_float(raw.w << 16), __uint_as_float(raw.w & 0xffff0000u));
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (narrow) {
            // A row tile with one or two rows (the shared gate's row after 512 experts): one chain per thread,
            // thread = (token, row), the same k-ascending chain and the same ordered sum of partials.
            const uint32_t tt = tid % LONG_TT, rr = tid / LONG_TT;
            float a = 0.0f;
            if (rr < rows_here) {
                const float* wr = ws + rr * LD;
                const float* xr = xs + tt * LD;
                for (uint32_t k = 0; k < part; k += 4) {
                    const float4 wv = *reinterpret_cast<const float4*>(wr + k), xv = *reinterpret_cast<const float4*>(xr + k);
                    a = __fmaf_rn(xv.x, wv.x, a);
                    a = __fmaf_rn(xv.y, wv.y, a);
                    a = __fmaf_rn(xv.z, wv.z, a);
                    a = __fmaf_rn(xv.w, wv.w, a);
                }
            }
            total[0][0] = __fadd_rn(total[0][0], a);
            continue;
        }
        float acc[LONG_RI][LONG_TJ];
#pragma unroll
        for (int i = 0; i < LONG_RI; ++i)
#pragma unroll
            for (int j = 0; j < LONG_TJ; ++j) acc[i][j] = 0.0f;
        const float* wrow = ws + tx * LD;
        const float* xrow = xs + ty * LD;
ZC_UNROLL(ZC_RL_UNROLL)
        for (uint32_t k = 0; k < part; k += 4) {
            float4 wv[LONG_RI], xv[LONG_TJ];
#pragma unroll
            for (int i = 0; i < LONG_RI; ++i) wv[i] = *reinterpret_cast<const float4*>(wrow + i * LONG_TXN * LD + k);
#pragma unroll
            for (int j = 0; j < LONG_TJ; ++j) xv[j] = *reinterpret_cast<const float4*>(xrow + j * LONG_TYN * LD + k);
#pragma unroll
            for (int i = 0; i < LONG_RI; ++i)
#pragma unroll
                for (int j = 0; j < LONG_TJ; ++j) {
                    float a = acc[i][j];
                    a = __fmaf_rn(xv[j].x, wv[i].x, a);
                    a = __fmaf_rn(xv[j].y, wv[i].y, a);
                    a = __fmaf_rn(xv[j].z, wv[i].z, a);
                    a = __fmaf_rn(xv[j].w, wv[i].w, a);
                    acc[i][j] = a;
                }
        }
#pragma unroll
        for (int i = 0; i < LONG_RI; ++i)
#pragma unroll
            for (int j = 0; j < LONG_TJ; ++j) total[i][j] = __fadd_rn(total[i][j], acc[i][j]);      // partial p joins the ordered sum
    }
    pdl_launch_dependents();
    if (narrow) {
        const uint32_t tt = tid % LONG_TT, rr = tid / LONG_TT, e = e0 + rr, t = t0 + tt;
        if (rr < rows_here && t < c.T) {
            if (e < c.E) c.logits[size_t(t) * c.E + e] = c.router_bias ? __fadd_rn(total[0][0], c.router_bias[e]) : total[0][0];
            else c.gate_logit[t] = total[0][0];
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < LONG_RI; ++i) {
        const uint32_t e = e0 + tx + LONG_TXN * i;
        if (e >= rows_total) continue;
#pragma unroll
        for (int j = 0; j < LONG_TJ; ++j) {
            const uint32_t t = t0 + ty + LONG_TYN * j;
            if (t >= c.T) continue;
            if (e < c.E) c.logits[size_t(t) * c.E + e] = c.router_bias ? __fadd_rn(total[i][j], c.router_bias[e]) : total[i][j];
            else c.gate_logit[t] = total[i][j];
        }
    }
}

// The same whole-K tile for the common format - FP32 router rows, BF16 activations - with the two tiles double-buffered:
// the activations stay BF16 in shared memory (they become FP32 in registers, the same values), so both tiles are plain
// 16-byte cp.async copies, and partition p + 1 is fetched while partition p is multiplied. With one buffer the two CTAs
// of an SM start together and stay in step, so the FMA pipe idles through every staging phase (ncu: FMA pipe 41 %).
__global__ void __launch_bounds__(LONG_THREADS, 2) router_long_db_kernel(Call c) {
    extern __shared__ __align__(16) float smem[];
    const uint32_t H = c.H, part = H / 16, LD = part + 4, LDH = part + 8;
    const uint32_t w_floats = LONG_RT * LD, stage_bytes = w_floats * 4 + LONG_TT * LDH * 2;       // one stage: [64][LD] floats, then [64][LDH] halves
    const uint32_t e0 = blockIdx.x * LONG_RT, t0 = blockIdx.y * LONG_TT;
    const uint32_t rows_total = c.E + (c.has_shared ? 1u : 0u);
    const uint32_t tid = threadIdx.x, tx = tid % LONG_TXN, ty = tid / LONG_TXN, warp = tid / 32, lane = tid % 32;
    const uint32_t rows_here = min(uint32_t(LONG_RT), rows_total - e0);
    const bool narrow = rows_here <= LONG_THREADS / LONG_TT;
    auto ws_of = [&](uint32_t stage) { return reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(smem) + stage * stage_bytes); };
    auto xh_of = [&](uint32_t stage) { return reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(smem) + stage * stage_bytes + w_floats * 4); };
    auto issue = [&](uint32_t p) {
        const uint32_t k0 = p * part;
        float* ws = ws_of(p & 1);
        uint16_t* xh = xh_of(p & 1);
        for (uint32_t el = warp; el < (narrow ? rows_here : uint32_t(LONG_RT)); el += LONG_THREADS / 32) {
            const uint32_t e = e0 + el;
            float* dst = ws + el * LD;
            if (e >= rows_total) {
                for (uint32_t kq = lane; kq < part / 4; kq += 32) *reinterpret_cast<float4*>(dst + kq * 4) = make_float4(0, 0, 0, 0);
            } else {
                const float* base = (e < c.E ? static_cast<const float*>(c.router_w) + size_t(e) * H : static_cast<const float*>(c.shared_gate_w)) + k0;
                for (uint32_t kq = lane; kq < part / 4; kq += 32) cp_async16(dst + kq * 4, base + kq * 4);
            }
        }
        for (uint32_t tt = warp * 2 + lane / 16; tt < LONG_TT; tt += LONG_THREADS / 16) {      // a half-warp takes a row of 16-byte pieces
            const uint32_t t = t0 + tt;
            const uint16_t* base = static_cast<const uint16_t*>(c.x) + size_t(t) * H + k0;
            for (uint32_t kb = lane % 16; kb < part / 8; kb += 16) {
                if (t < c.T) cp_async16(xh + tt * LDH + kb * 8, base + kb * 8);
                else *reinterpret_cast<uint4*>(xh + tt * LDH + kb * 8) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto x4 = [](uint2 raw) { return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u)); };
    float total[LONG_RI][LONG_TJ];
#pragma unroll
    for (int i = 0; i < LONG_RI; ++i)
#pragma unroll
        for (int j = 0; j < LONG_TJ; ++j) total[i][j] = 0.0f;
    pdl_wait();
    issue(0);
    for (uint32_t p = 0; p < 16; ++p) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                     // partition p has landed for everyone, and partition p - 1 has been consumed
        if (p + 1 < 16) issue(p + 1);        // into the buffer partition p - 1 used
        const float* ws = ws_of(p & 1);
        const uint16_t* xh = xh_of(p & 1);
        if (narrow) {
            const uint32_t tt = tid % LONG_TT, rr = tid / LONG_TT;
            float a = 0.0f;
            if (rr < rows_here) {
                const float* wr = ws + rr * LD;
                for (uint32_t k = 0; k < part; k += 4) {
                    const float4 wv = *reinterpret_cast<const float4*>(wr + k), xv = x4(*reinterpret_cast<const uint2*>(xh + tt * LDH + k));
                    a = __fmaf_rn(xv.x, wv.x, a);
                    a = __fmaf_rn(xv.y, wv.y, a);
                    a = __fmaf_rn(xv.z, wv.z, a);
                    a = __fmaf_rn(xv.w, wv.w, a);
                }
            }
            total[0][0] = __fadd_rn(total[0][0], a);
            continue;
        }
        float acc[LONG_RI][LONG_TJ];
#pragma unroll
        for (int i = 0; i < LONG_RI; ++i)
#pragma unroll
            for (int j = 0; j < LONG_TJ; ++j) acc[i][j] = 0.0f;
        const float* wrow = ws + tx * LD;
#pragma unroll 2
        for (uint32_t k = 0; k < part; k += 4) {
            float4 wv[LONG_RI], xv[LONG_TJ];
#pragma unroll
            for (int i = 0; i < LONG_RI; ++i) wv[i] = *reinterpret_cast<const float4*>(wrow + i * LONG_TXN * LD + k);
#pragma unroll
            for (int j = 0; j < LONG_TJ; ++j) xv[j] = x4(*reinterpret_cast<const uint2*>(xh + (ty + j * LONG_TYN) * LDH + k));
#pragma unroll
            for (int i = 0; i < LONG_RI; ++i)
#pragma unroll
                for (int j = 0; j < LONG_TJ; ++j) {
                    float a = acc[i][j];
                    a = __fmaf_rn(xv[j].x, wv[i].x, a);
                    a = __fmaf_rn(xv[j].y, wv[i].y, a);
                    a = __fmaf_rn(xv[j].z, wv[i].z, a);
                    a = __fmaf_rn(xv[j].w, wv[i].w, a);
                    acc[i][j] = a;
                }
        }
#pragma unroll
        for (int i = 0; i < LONG_RI; ++i)
#pragma unroll
            for (int j = 0; j < LONG_TJ; ++j) total[i][j] = __fadd_rn(total[i][j], acc[i][j]);      // partial p joins the ordered sum
    }
    pdl_launch_dependents();
    if (narrow) {
        const uint32_t tt = tid % LONG_TT, rr = tid / LONG_TT, e = e0 + rr, t = t0 + tt;
        if (rr < rows_here && t < c.T) {
            if (e < c.E) c.logits[size_t(t) * c.E + e] = c.router_bias ? __fadd_rn(total[0][0], c.router_bias[e]) : total[0][0];
            else c.gate_logit[t] = total[0][0];
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < LONG_RI; ++i) {
        const uint32_t e = e0 + tx + LONG_TXN * i;
        if (e >= rows_total) continue;
#pragma unroll
        for (int j = 0; j < LONG_TJ; ++j) {
            const uint32_t t = t0 + ty + LONG_TYN * j;
            if (t >= c.T) continue;
            if (e < c.E) c.logits[size_t(t) * c.E + e] = c.router_bias ? __fadd_rn(total[i][j], c.router_bias[e]) : total[i][j];
            else c.gate_logit[t] = total[i][j];
        }
    }
}

int launch_router_long(zc_moe* m, const Call& c, cudaStream_t s) {
    if (c.router_dtype == ZC_F32 && c.act_dtype != ZC_F32 && m->router_db) {       // the double-buffered form
        const uint32_t partd = c.H / 16;
        const size_t bytes = 2 * (size_t(LONG_RT) * (partd + 4) * 4 + size_t(LONG_TT) * (partd + 8) * 2);
        static SmemOptIn configured_db;
        if (bytes <= 110 * 1024 && opt_in_smem(router_long_db_kernel, configured_db, m->device, bytes) == cudaSuccess) {
            const uint32_t rows = c.E + (c.has_shared ? 1 : 0);
            int rcd;
            {
                Timed t(m, s, KERNEL_ROUTER);
                const cudaError_t e = launch_chained(m, -1, router_long_db_kernel, dim3((rows + LONG_RT - 1) / LONG_RT, (c.T + LONG_TT - 1) / LONG_TT), dim3(LONG_THREADS), bytes, s, nullptr, 0, c);
                if (e != cudaSuccess) return fail(m, ZC_EEXEC, std::string("router (long, double-buffered) launch: ") + cudaGetErrorString(e));
                rcd = check_launch(m, "router");
            }
            return rcd < 0 ? rcd : 1;
        }
        cudaGetLastError();
    }
    const uint32_t part = c.H / 16, LD = part + 4;
    const size_t smem = size_t(LONG_RT + LONG_TT) * LD * sizeof(float);
    if (smem > 200 * 1024) return 0;
    static SmemOptIn configured;
    if (opt_in_smem(router_long_kernel, configured, m->device, smem) != cudaSuccess) { cudaGetLastError(); return 0; }
    const uint32_t rows_total = c.E + (c.has_shared ? 1 : 0);
    const dim3 grid((rows_total + LONG_RT - 1) / LONG_RT, (c.T + LONG_TT - 1) / LONG_TT);
    int rc;
    {
        Timed t(m, s, KERNEL_ROUTER);
        const cudaError_t e = launch_chained(m, -1, router_long_kernel, grid, dim3(LONG_THREADS), smem, s, nullptr, 0, c);
        if (e != cudaSuccess) return fail(m, ZC_EEXEC, std::string("router (long) launch: ") + cudaGetErrorString(e));
        rc = check_launch(m, "router");
    }
    return rc < 0 ? rc : 1;
}

}  // namespace

uint32_t router_rows_padded(const zc_moe_desc& d) { return (d.experts + (d.has_shared ? 1 : 0) + ROW_TILE_PAD - 1) / ROW_TILE_PAD * ROW_TILE_PAD; }

int launch_router_partial(zc_moe* m, const Call& c, cudaStream_t s) {
    // Cluster form for short batches, whole-K tiles for long ones (2048 tokens: 178 us against 237 us for the
    // global-memory form; 8192: 650 against 893), the global-memory form in between (256 tokens at hidden 4096: 77 us
    // against 205 us for 36 whole-K tiles) and whenever the device cannot host the others.
    {
        int n = 0;
        // Up to 128 tokens small tiles win on latency: at 64 tokens, 544 CTAs of 16 tokens x 32 rows measured 19 us
        // against 21 us (32 x 32) and 25 us (32 x 64, whose 144 large CTAs do not all find a cluster slot in the first wave).
        if (c.T <= 8) n = launch_router_cluster<8, 1>(m, c, s);
        else if (c.T <= ZC_ROUTER_SMALL_T) n = launch_router_cluster<16, 1>(m, c, s);
        else if (size_t((c.T + 63) / 64) * ((c.E + 64) / 64) >= 144) n = launch_router_long(m, c, s);      // enough whole-K tiles to fill the SMs
        if (n != 0) return n;
    }
    const uint32_t part = c.H / 16;
    const uint32_t rows_padded = router_rows_padded(m->d);
    // Token tile: 8 tokens x 32 rows for single-digit batches, 32 tokens x 64 rows beyond (eight chains per
    // thread share two shared-memory reads per k); long batches use the 64-token tile, which re-reads the
    // router rows least often.
    const int which = c.T <= 8 ? 0 : c.T <= 512 ? 1 : 2;
    const uint32_t TT = which == 0 ? 8 : which == 1 ? 32 : 64;
    const uint32_t row_tile = which == 1 ? 64 : 32;
    const size_t smem = size_t(part) * (TT + row_tile) * sizeof(float);
    static SmemOptIn configured[3];
    {
        const cudaError_t e = which == 0 ? opt_in_smem(router_partial_kernel<8>, configured[0], m->device, smem)
                            : which == 1 ? opt_in_smem(router_partial_kernel<32>, configured[1], m->device, smem)
                                         : opt_in_smem(router_partial_kernel<64>, configured[2], m->device, smem);
        if (e != cudaSuccess) return check_launch(m, "router attribute");
    }
    const uint32_t rows_total = c.E + (c.has_shared ? 1 : 0);
    const dim3 grid((rows_total + row_tile - 1) / row_tile, 16, (c.T + TT - 1) / TT);
    int rc;
    {
        Timed t(m, s, KERNEL_ROUTER);
        if (which == 0) router_partial_kernel<8><<<grid, ROUTER_THREADS, smem, s>>>(c, m->router_partial, rows_padded, m->router_done, 1);
        else if (which == 1) router_partial_kernel<32><<<grid, ROUTER_THREADS, smem, s>>>(c, m->router_partial, rows_padded, m->router_done, 1);
        else router_partial_kernel<64><<<grid, ROUTER_THREADS, smem, s>>>(c, m->router_partial, rows_padded, m->router_done, 1);
        rc = check_launch(m, "router");
    }
    return rc < 0 ? rc : 1;
}

// The router operator: one launch (partials, then the ordered sum by the last partition CTA of each tile).
int launch_router(zc_moe* m, const Call& c, cudaStream_t s) { return launch_router_partial(m, c, s); }

}  // namespace zc

// ---------------------------------------------------------------------------------------------
// Router logits for callers that must not allocate device memory.
//
// Some hosts of this library run inside a region where cudaMalloc is forbidden or would deadlock: a
// plugin called while the engine's own caching allocator holds all of HBM, a callback that runs while
// another thread is capturing a CUDA graph (allocation calls are illegal then), or a real-time loop
// that may not take the allocator's lock. zc_moe_create allocates, so those callers cannot own a
// handle. This entry point needs none: the router kernel's scratch — the [16, tokens, experts]
// partition sums and the tile arrival counters — lives in a fixed array inside the library image.
// ---------------------------------------------------------------------------------------------
namespace zc {
namespace {
constexpr uint32_t NOALLOC_MAX_TOKENS = 64, NOALLOC_MAX_EXPERTS = 512, NOALLOC_MAX_HIDDEN = 3072;
constexpr size_t NOALLOC_PARTIAL_BYTES = size_t(16) * NOALLOC_MAX_TOKENS * NOALLOC_MAX_EXPERTS * sizeof(float);   // 2 MiB
constexpr size_t NOALLOC_COUNTER_BYTES = 4096;       // (experts / 32) x (tokens / 8) counters at most = 128 words
// Held by every GPU that loads the library until the process exits: 2 MiB + 4 KiB.
static __device__ __align__(256) unsigned char noalloc_scratch[NOALLOC_PARTIAL_BYTES + NOALLOC_COUNTER_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
unsigned char* noalloc_address[NOALLOC_MAX_DEVICES] = {};   // device address of the array, per device
}  // namespace
}  // namespace zc

extern "C" int zc_router_logits_noalloc(const void* x, int act_dtype, const void* router_w, int router_dtype,
                                        uint32_t tokens, uint32_t hidden, uint32_t experts, float* logits, void* stream) {
    using namespace zc;
    if (!x || !router_w || !logits) return fail(nullptr, ZC_EINVAL, "linear input shape");
    if (!tokens || tokens > NOALLOC_MAX_TOKENS)
        return fail(nullptr, ZC_EINVAL, "zc_router_logits_noalloc: tokens must be 1..64 (the built-in scratch is sized for 64)");
    if (!experts || experts % 32 || experts > NOALLOC_MAX_EXPERTS)
        return fail(nullptr, ZC_EINVAL, "zc_router_logits_noalloc: experts must be a multiple of 32, at most 512");
    if (!hidden || hidden % 128 || hidden > NOALLOC_MAX_HIDDEN)
        return fail(nullptr, ZC_EINVAL, "zc_router_logits_noalloc: hidden must be a multiple of 128, at most 3072");
    if ((act_dtype != ZC_BF16 && act_dtype != ZC_F32) || (router_dtype != ZC_BF16 && router_dtype != ZC_F32))
        return fail(nullptr, ZC_EINVAL, "zc_router_logits_noalloc: dtypes must be BF16 or F32");
    // The kernel reads x and router_w and writes logits with 16-byte accesses: a misaligned or aliased buffer is an
    // argument error here, not a device fault.
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(router_w) | reinterpret_cast<uintptr_t>(logits)) & 15)
        return fail(nullptr, ZC_EINVAL, "zc_router_logits_noalloc: x, router_w and logits must be 16-byte aligned");
    {
        const size_t xb = size_t(tokens) * hidden * (act_dtype == ZC_F32 ? 4 : 2), wb = size_t(experts) * hidden * (router_dtype == ZC_F32 ? 4 : 2);
        const size_t lb = size_t(tokens) * experts * 4;
        const char* lo = reinterpret_cast<const char*>(logits);
        const char* xa = static_cast<const char*>(x); const char* wa = static_cast<const char*>(router_w);
        if ((lo < xa + xb && xa < lo + lb) || (lo < wa + wb && wa < lo + lb))
            return fail(nullptr, ZC_EINVAL, "zc_router_logits_noalloc: logits overlaps an input");
    }
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(nullptr, ZC_EEXEC, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (device < 0 || device >= NOALLOC_MAX_DEVICES) return fail(nullptr, ZC_EINVAL, "zc_router_logits_noalloc: device index above 63");
    if (!noalloc_address[device]) {
        // Set-up, once per device, with that device current: in host code the array's name is only a
        // stand-in, the kernel needs the address the runtime gives for it on this device.
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, noalloc_scratch);
        if (e != cudaSuccess || !p) return fail(nullptr, ZC_EEXEC, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        noalloc_address[device] = static_cast<unsigned char*>(p);
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* partial = reinterpret_cast<float*>(noalloc_address[device]);
    uint32_t* counters = reinterpret_cast<uint32_t*>(noalloc_address[device] + NOALLOC_PARTIAL_BYTES);
    // The counters must start at zero (a call cut short by an error would leave them dirty); the partial
    // sums are fully rewritten for the (tokens, experts) of this call before they are read.
    if ((e = cudaMemsetAsync(counters, 0, NOALLOC_COUNTER_BYTES, s)) != cudaSuccess)
        return fail(nullptr, ZC_EEXEC, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
    Call c{};
    c.x = x; c.router_w = router_w; c.logits = logits;
    c.T = tokens; c.H = hidden; c.E = experts; c.act_dtype = uint8_t(act_dtype); c.router_dtype = uint8_t(router_dtype); c.has_shared = 0;
    const uint32_t part = hidden / 16, rows_padded = experts;      // a multiple of the 32-row tile already
    const bool tiny = tokens <= 8;
    const uint32_t TT = tiny ? 8 : 16;
    const size_t smem = size_t(part) * (TT + 32) * sizeof(float);   // at most 36 KiB: no opt-in attribute needed
    const dim3 grid(rows_padded / 32, 16, (tokens + TT - 1) / TT);
    if (tiny) router_partial_kernel<8><<<grid, ROUTER_THREADS, smem, s>>>(c, partial, rows_padded, counters, 1);
    else router_partial_kernel<16><<<grid, ROUTER_THREADS, smem, s>>>(c, partial, rows_padded, counters, 1);
    return check_launch(nullptr, "router (no-alloc)");
}
