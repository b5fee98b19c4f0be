// Prefill family: grouped GEMM over all experts' row groups on the 5th-generation tensor cores.
//
// Replaces the reference's prefill branch of encode_expert_rows (src/engine/pipeline.cpp:18-30: per expert
// and per microbatch a gathered q4_gate_up, a q4_mm and a scatter_experts launch, kernels/metal/qwen.metal
// :71-81, :63-70, :800-803) with two launches per layer over a tile list that covers every expert.
//
// Formulation ("weights as M"): for one expert, D[weight row, token] = W[rows, K] . X^T[K, tokens]. The
// 128-row weight tile is the M of tcgen05.mma, the expert's tokens are the N (padded to 16, at most 128
// per tile), so a ragged or skewed expert load costs at most 15 padded columns instead of a padded
// 128-row token tile, and every weight is fetched and dequantised once per 128 tokens of its expert.
//   NMAT = 2: gate and up tiles of the same 128 rows accumulate side by side in TMEM (columns [0,N) and
//             [N,2N)); the epilogue reads both, applies SwiGLU and stores h as FP16 in the k order the
//             second launch consumes.
//   NMAT = 1: the down projection; the epilogue writes FP32 rows at the slots' router positions.
//
// Roles in a CTA of 160 threads: warps 0-3 are producers, then the epilogue; warp 4 owns TMEM
// (tcgen05.alloc / dealloc) and one of its lanes issues the MMAs.
//   producer thread r: dequantises weight row r of the tile for one 64-wide quantisation group per stage
//     (w = s*q + b in FP16, one rounding; eight codes -> one 16-byte store). The packed codes reach it
//     through a thread-private cp.async ring three stages ahead; the token rows (already FP16, in the
//     matching k order) are copied by cp.async straight into the B tile two stages ahead. Stage buffers
//     use the no-swizzle K-major core-matrix layout ([rows/8][8 k-chunks][8 rows][16 bytes]; LBO = 128,
//     SBO = 1024).
//   a stage is handed over with fence.proxy.async + mbarrier arrive; the MMA lane waits, issues
//     4 (k steps of 16) x NMAT x 2 (hi, lo weight terms) tcgen05.mma, and frees the stage with tcgen05.commit.
// Precision: an FP16 weight s*q+b rounded once costs ~2e-4 relative rms per projection, and three projections
// plus the FP16 intermediate put the layer's max-abs error at ~2.5e-3 x RMS, above the 2e-3 bound. The weights
// are therefore fed as two exact-product FP16 terms (see pf_dequant_word); what remains is the single FP16
// rounding of the intermediate h (~1.4e-3 x RMS max-abs at a few hundred thousand outputs).
// Every wait is bounded: after ~2^22 polls a role sets ZC_STATUS_TIMEOUT, raises the CTA's abort flag and
// leaves its loop; the CTA then frees its TMEM and exits.
#include "common.cuh"

namespace zc {
namespace {

constexpr int PF_THREADS = 160;
constexpr int PF_M = 128;
constexpr int PF_NMAX = 128;          // tokens per tile (the N of the MMA, padded to 16)
constexpr uint32_t PF_A_BYTES = PF_M * 128;          // one matrix, one stage: 128 rows x 64 halves
constexpr uint32_t PF_B_BYTES = PF_NMAX * 128;
constexpr uint32_t PF_POLL_LIMIT = 1u << 22;

struct PfTile { int32_t expert, row0, rows, shared; };

__device__ __forceinline__ uint32_t pf_smem(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pf_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pf_smem(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(pf_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait. Returns false (and raises the abort flag) when the phase did not complete in time or
// another role has already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* status) {
    for (uint32_t i = 0; i < PF_POLL_LIMIT; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (*abort_flag) return false;
        if (i > 64) __nanosleep(40);
    }
    *abort_flag = 1;
    atomicOr(status, ZC_STATUS_TIMEOUT);
    return false;
}

// K-major, no swizzle: start address, LBO = 128 B (next k chunk), SBO = 1024 B (next 8 rows), version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(128 >> 4) << 16) | (uint64_t(1024 >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(pf_smem(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}

// Position inside a block of eight k values at which value k%8 = i is stored: blocks hold
// (k0,k4,k1,k5,k2,k6,k3,k7), the order the Q4 extraction below produces.
__device__ __forceinline__ uint32_t pf_pos8(uint32_t i) { return (i & 3) * 2 + (i >> 2); }

__device__ __forceinline__ uint32_t pf_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Eight Q4 codes of one word -> the weights s*q + b as two FP16 terms whose sum has (almost) no rounding:
//   hi = s_hi * (q - 8)            exact: s_hi keeps 6 significant bits of the scale, q - 8 has 4
//   lo = s_lo * (q - 8) + (b + 8s) s_lo * (q - 8) is exact too; the only rounding is at the size of the
//                                  residual bias b + 8s, which is zero for symmetric codes (b = -8 s)
// Both come out as (k0,k4) (k1,k5) (k2,k6) (k3,k7). The tensor cores add hi.x + lo.x in FP32.
__device__ __forceinline__ void pf_dequant_word(uint32_t w, __half2 s_hi, __half2 s_lo, __half2 resid, uint4& hi, uint4& lo) {
    const uint32_t mlo = 0x000f000fu, mhi = 0x00f000f0u, magic = 0x64006400u;
    const __half2 k1032 = __floats2half2_rn(1032.0f, 1032.0f), k16 = __floats2half2_rn(0.0625f, 0.0625f), k72 = __floats2half2_rn(-72.0f, -72.0f);
    const uint32_t w8 = w >> 8;
    uint32_t p[4] = {pf_and_or(w, mlo, magic), pf_and_or(w, mhi, magic), pf_and_or(w8, mlo, magic), pf_and_or(w8, mhi, magic)};
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 q = *reinterpret_cast<__half2*>(&p[i]);
        q = (i & 1) ? __hfma2(q, k16, k72) : __hsub2(q, k1032);      // exact integer q - 8
        const __half2 a = __hmul2(q, s_hi), b = __hfma2(q, s_lo, resid);
        h[i] = *reinterpret_cast<const uint32_t*>(&a);
        l[i] = *reinterpret_cast<const uint32_t*>(&b);
    }
    hi = make_uint4(h[0], h[1], h[2], h[3]);
    lo = make_uint4(l[0], l[1], l[2], l[3]);
}

// Tile list: one entry per (expert with work, block of PF_NMAX of its rows), the shared expert's token
// blocks first. One CTA of 1024 threads; experts <= 1024.
__global__ void __launch_bounds__(1024) pf_tiles_kernel(const int32_t* __restrict__ offsets, uint32_t E, uint32_t first_expert, uint32_t local_experts,
                                                        uint32_t T, uint32_t has_shared, uint32_t nmax, PfTile* __restrict__ tiles, int32_t* __restrict__ ntiles) {
    __shared__ int warp_totals[33];
    const uint32_t e = threadIdx.x, lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const uint32_t shared_tiles = has_shared ? (T + nmax - 1) / nmax : 0;
    int rows = 0;
    if (e < E && e >= first_expert && e < first_expert + local_experts) rows = offsets[e + 1] - offsets[e];
    const int mine = (rows + int(nmax) - 1) / int(nmax);
    int inclusive = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) { const int n = __shfl_up_sync(0xffffffffu, inclusive, off); if (lane >= uint32_t(off)) inclusive += n; }
    if (lane == 31) warp_totals[warp] = inclusive;
    __syncthreads();
    if (warp == 0) {
        int w = warp_totals[lane], inc = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) { const int n = __shfl_up_sync(0xffffffffu, inc, off); if (lane >= uint32_t(off)) inc += n; }
        warp_totals[lane] = inc - w;
        if (lane == 31) warp_totals[32] = inc;
    }
    __syncthreads();
    const int first = int(shared_tiles) + warp_totals[warp] + inclusive - mine;
    for (int i = 0; i < mine; ++i) tiles[first + i] = PfTile{int32_t(e), int32_t(i * nmax), min(int(nmax), rows - i * int(nmax)), 0};
    if (threadIdx.x < shared_tiles) tiles[threadIdx.x] = PfTile{int32_t(E), int32_t(threadIdx.x * nmax), int32_t(min(nmax, T - threadIdx.x * nmax)), 1};
    if (threadIdx.x == 0) *ntiles = int(shared_tiles) + warp_totals[32];
}

// x [T, H] (bf16 or fp32) -> FP16 [T, H] with every block of eight k values stored in pf_pos8 order: the
// B operand of the gate/up launch, copied into shared memory with plain 16-byte cp.async.
__global__ void pf_prepare_x_kernel(const void* __restrict__ x, int act_dtype, __half* __restrict__ xp, size_t blocks) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= blocks) return;
    float v[8];
    if (act_dtype == ZC_F32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(x) + i * 8);
        const float4 a = p[0], b = p[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + i * 8);
        const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { v[2 * j] = __uint_as_float(r[j] << 16); v[2 * j + 1] = __uint_as_float(r[j] & 0xffff0000u); }
    }
    __half h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) h[pf_pos8(j)] = __float2half_rn(v[j]);
    *reinterpret_cast<uint4*>(xp + i * 8) = *reinterpret_cast<uint4*>(h);
}

__device__ __forceinline__ void pf_cp16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void pf_cp4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

constexpr int PF_RAW = 4;      // depth of the per-thread ring of packed codes

// Shared memory of one CTA (dynamic, 1024-byte aligned for the tile buffers): a ring of A stages (each
// matrix as a hi and a lo tile), a ring of B stages, and the per-thread rings of packed codes and metadata.
template <int NMAT>
struct PfSmem {
    static constexpr uint32_t SA = NMAT == 2 ? 2 : 3;                 // A ring depth
    static constexpr uint32_t SB = 3;                                 // B ring depth
    static constexpr uint32_t A_STAGE = NMAT * 2 * PF_A_BYTES;        // [matrix][hi, lo]
    static constexpr uint32_t A_RING = SA * A_STAGE;
    static constexpr uint32_t B_RING = SB * PF_B_BYTES;
    static constexpr uint32_t RAW = PF_RAW * NMAT * 128 * 32;         // [slot][matrix][thread][32 B]
    static constexpr uint32_t META = PF_RAW * NMAT * 128 * 8;         // [slot][matrix][thread][s0 s1 b0 b1]
    static constexpr uint32_t TOTAL = A_RING + B_RING + RAW + META + 1024;   // + alignment slack
};

// Grid: (weight-row tiles of 128, tiles of the list). See the file header for the roles.
template <int NMAT, bool META_F16>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_kernel(Call c, const PfTile* __restrict__ tiles, const int32_t* __restrict__ ntiles,
                                                                 const __half* __restrict__ bsrc, __half* __restrict__ hdst) {
    using S = PfSmem<NMAT>;
    extern __shared__ uint8_t pf_raw_smem[];
    __shared__ __align__(8) uint64_t full_bar[3], done_bar[3], accum_bar;     // indexed by stage % 3
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile uint32_t abort_flag;
    __shared__ const __half* brow[PF_NMAX];       // source row of each token row of the tile
    __shared__ long long drow[PF_NMAX];           // destination element offset of each token row
    if (blockIdx.y >= uint32_t(*ntiles)) return;
    const PfTile tile = tiles[blockIdx.y];
    const uint32_t K = NMAT == 2 ? c.H : c.F, G = K / 64, nst = G;
    const uint32_t N = uint32_t(tile.rows), Npad = (N + 15) & ~15u;
    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t r0 = blockIdx.x * PF_M;
    const uint32_t base = (pf_smem(pf_raw_smem) + 1023) & ~1023u;
    const uint32_t b_ring = base + S::A_RING, raw_base = b_ring + S::B_RING, meta_base = raw_base + S::RAW;
    const uint8_t* record = tile.shared ? c.shared_record : c.records + size_t(uint32_t(tile.expert) - c.first_expert) * c.record_stride;

    // ---- set-up ----------------------------------------------------------------------------------
    if (tid == 0) {
        for (int i = 0; i < 3; ++i) { mbar_init(&full_bar[i], 128); mbar_init(&done_bar[i], 1); }
        mbar_init(&accum_bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < N) {
        const uint32_t i = uint32_t(tile.row0) + tid;
        if (tile.shared) {
            brow[tid] = bsrc + (NMAT == 2 ? size_t(i) * K : (size_t(c.T) * c.K + i) * K);
            drow[tid] = NMAT == 2 ? (long long)(size_t(c.T) * c.K + i) * c.F : (long long)i * c.H;
        } else {
            const uint32_t pos = uint32_t(c.offsets[tile.expert]) + i, slot = uint32_t(c.perm[pos]);
            brow[tid] = bsrc + (NMAT == 2 ? size_t(slot / c.K) * K : size_t(pos) * K);
            drow[tid] = NMAT == 2 ? (long long)pos * c.F : (long long)slot * c.H;
        }
    }
    uint32_t ncols = 32;
    while (ncols < NMAT * Npad) ncols <<= 1;
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pf_smem(&tmem_base_s)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    uint32_t* status = c.status;

    if (warp < 4) {
        // ---- producers -----------------------------------------------------------------------------
        const uint32_t r = tid;                                   // weight row of the tile
        const Projection pr[2] = {NMAT == 2 ? c.gate : c.down, c.up};
        const uint8_t* codes[NMAT]; const uint8_t* scales[NMAT]; const uint8_t* biases[NMAT];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
            codes[m] = record + pr[m].codes + size_t(r0 + r) * (K / 2);
            scales[m] = record + pr[m].scales + size_t(r0 + r) * G * 2;
            biases[m] = record + pr[m].biases + size_t(r0 + r) * G * 2;
        }
        auto issue_raw = [&](uint32_t ks) {          // packed codes (and, for even groups, metadata of two groups)
            if (ks >= nst) return;
            const uint32_t slot = ks % PF_RAW;
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                const uint32_t dst = raw_base + ((slot * NMAT + m) * 128 + r) * 32;
                pf_cp16(dst, codes[m] + ks * 32);
                pf_cp16(dst + 16, codes[m] + ks * 32 + 16);
                if ((ks & 1) == 0) {
                    const uint32_t md = meta_base + (((ks / 2) % PF_RAW * NMAT + m) * 128 + r) * 8;
                    pf_cp4(md, scales[m] + ks * 2);
                    pf_cp4(md + 4, biases[m] + ks * 2);
                }
            }
        };
        auto issue_b = [&](uint32_t ks) {            // token rows of stage ks, 16-byte pieces straight into the tile
            if (ks >= nst) return;
            const uint32_t bs = b_ring + (ks % S::SB) * PF_B_BYTES;
            for (uint32_t q = tid; q < N * 8; q += 128) {
                const uint32_t j = q / 8, kc = q % 8;
                pf_cp16(bs + (j / 8) * 1024 + kc * 128 + (j % 8) * 16, brow[j] + ks * 64 + kc * 8);
            }
        };
        bool ok = true;
        issue_b(0); issue_raw(0); issue_raw(1); issue_raw(2);
        asm volatile("cp.async.commit_group;" ::: "memory");
        issue_b(1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        // done_bar[j % 3] completes phase j / 3 when the MMAs of stage j have drained.
        auto stage_done = [&](uint32_t j) { return mbar_wait(&done_bar[j % 3], (j / 3) & 1, &abort_flag, status); };
        for (uint32_t ks = 0; ks < nst && ok; ++ks) {
            // codes and token rows of stage ks were committed at least two groups ago
            asm volatile("cp.async.wait_group 1;" ::: "memory");
            // the A buffer of this stage was last read by stage ks - SA
            if (ks >= S::SA) ok = stage_done(ks - S::SA);
            if (!ok) break;
            const uint32_t as = base + (ks % S::SA) * S::A_STAGE;
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                const uint32_t src = raw_base + (((ks % PF_RAW) * NMAT + m) * 128 + r) * 32;
                const uint32_t md = meta_base + (((ks / 2) % PF_RAW * NMAT + m) * 128 + r) * 8 + (ks & 1) * 2;
                uint4 w0, w1;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w0.x), "=r"(w0.y), "=r"(w0.z), "=r"(w0.w) : "r"(src));
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w1.x), "=r"(w1.y), "=r"(w1.z), "=r"(w1.w) : "r"(src + 16));
                uint16_t sb, bb;
                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sb) : "r"(md));
                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(bb) : "r"(md + 4));
                __half sh, bh;
                if (META_F16) { sh = __ushort_as_half(sb); bh = __ushort_as_half(bb); }
                else { sh = __float2half_rn(bf_to_float(sb)); bh = __float2half_rn(bf_to_float(bb)); }
                const __half shi = __ushort_as_half(uint16_t(__half_as_ushort(sh) & 0xffe0u));     // top 6 significant bits
                const __half slo = __hsub(sh, shi);                                                 // exact
                const __half res = __hfma(sh, __float2half_rn(8.0f), bh);                           // b + 8 s
                const __half2 s_hi = __half2half2(shi), s_lo = __half2half2(slo), resid = __half2half2(res);
                const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                const uint32_t dst = as + m * 2 * PF_A_BYTES + (r / 8) * 1024 + (r % 8) * 16;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    uint4 hi, lo;
                    pf_dequant_word(words[i], s_hi, s_lo, resid, hi, lo);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + i * 128), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w) : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + PF_A_BYTES + i * 128), "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w) : "memory");
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&full_bar[ks % 3]);
            // The B buffer of stage ks+2 was last read by stage ks-1, whose MMAs ran while this stage was
            // being dequantised: wait for them, then start the copies of stage ks+2 and the codes of ks+3.
            if (ks >= 1 && ks + 2 < nst) ok = stage_done(ks - 1);
            if (!ok) break;
            issue_b(ks + 2);
            issue_raw(ks + 3);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");

        // ---- epilogue: TMEM lane 32*warp + lane is weight row r; columns are the tile's tokens --------
        if (ok) ok = mbar_wait(&accum_bar, 0, &abort_flag, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const uint32_t lane_addr = tmem_base + ((warp * 32) << 16);
            const uint32_t row = r0 + r;
            float* out_base = tile.shared ? c.shared_out : c.expert_out;
            for (uint32_t c0 = 0; c0 < Npad; c0 += 16) {
                uint32_t a[16], b[16];
                tmem_ld16(lane_addr + c0, a);
                if constexpr (NMAT == 2) tmem_ld16(lane_addr + Npad + c0, b);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const uint32_t t = c0 + j;
                    if (t < N) {
                        const float g = __uint_as_float(a[j]);
                        if constexpr (NMAT == 2) {
                            const float u = __uint_as_float(b[j]);
                            const float h = (g * sigmoid_f(g)) * u;
                            hdst[drow[t] + (row & ~7u) + pf_pos8(row & 7)] = __float2half_rn(h);
                        } else {
                            out_base[drow[t] + row] = g;
                        }
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    } else {
        // ---- MMA issue: one lane of warp 4 ------------------------------------------------------------
        if (lane == 0) {
            // instruction descriptor: D = F32, A = B = F16, both K-major, N = Npad, M = 128
            const uint32_t idesc = (1u << 4) | ((Npad >> 3) << 17) | ((PF_M >> 4) << 24);
            bool ok = true;
            for (uint32_t ks = 0; ks < nst; ++ks) {
                ok = mbar_wait(&full_bar[ks % 3], (ks / 3) & 1, &abort_flag, status);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t as = base + (ks % S::SA) * S::A_STAGE, bs = b_ring + (ks % S::SB) * PF_B_BYTES;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t bdesc = umma_desc(bs + kk * 256);
#pragma unroll
                    for (int m = 0; m < NMAT; ++m) {
                        umma_f16(tmem_base + m * Npad, umma_desc(as + (m * 2 + 0) * PF_A_BYTES + kk * 256), bdesc, idesc, (ks | kk) != 0);
                        umma_f16(tmem_base + m * Npad, umma_desc(as + (m * 2 + 1) * PF_A_BYTES + kk * 256), bdesc, idesc, 1);
                    }
                }
                umma_commit(&done_bar[ks % 3]);
            }
            if (ok) umma_commit(&accum_bar);
        }
        __syncwarp();
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 4) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ncols) : "memory");
    }
}

template <int NMAT, bool META_F16>
int launch_prefill(zc_moe* m, const Call& c, const __half* bsrc, cudaStream_t s) {
    const uint32_t N = NMAT == 2 ? c.F : c.H;
    if (N % PF_M) return fail(m, ZC_EINVAL, "prefill kernel: rows not a multiple of 128");
    auto kernel = prefill_kernel<NMAT, META_F16>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(PfSmem<NMAT>::TOTAL)) != cudaSuccess)
            return check_launch(m, "prefill kernel attribute");
        configured = true;
    }
    Timed t(m, s, NMAT == 2 ? KERNEL_PREFILL_GATE_UP : KERNEL_PREFILL_DOWN);
    kernel<<<dim3(N / PF_M, m->pf_max_tiles), PF_THREADS, PfSmem<NMAT>::TOTAL, s>>>(c, static_cast<const PfTile*>(m->pf_tiles), m->pf_ntiles, bsrc, m->hbuf16);
    return check_launch(m, NMAT == 2 ? "prefill gate_up" : "prefill down");
}

}  // namespace

size_t prefill_tile_capacity(const zc_moe_desc& d) {
    const size_t local = d.local_experts ? d.local_experts : d.experts;
    return local + (size_t(d.max_tokens) * d.top_k + d.max_tokens) / PF_NMAX + 2;
}
size_t prefill_tile_bytes() { return sizeof(PfTile); }

bool prefill_supported(const zc_moe_desc& d) {
    // BF16 activations convert to FP16 exactly; an FP32 activation would need a second FP16 term.
    return d.gate_bits == 4 && d.up_bits == 4 && d.down_bits == 4 && d.arith == ZC_ARITH_FP32 && d.act_dtype == ZC_BF16 &&
           d.ffn % 128 == 0 && d.hidden % 128 == 0;
}

// tile list -> FP16 activations -> gate/up (+SwiGLU) -> down. Routing must already be in place.
int launch_experts_prefill(zc_moe* m, const Call& c, cudaStream_t s) {
    int rc;
    {
        Timed t(m, s, KERNEL_PREFILL_PREP);
        pf_tiles_kernel<<<1, 1024, 0, s>>>(c.offsets, c.E, c.first_expert, c.local_experts, c.T, c.has_shared, PF_NMAX,
                                           static_cast<PfTile*>(m->pf_tiles), m->pf_ntiles);
        if ((rc = check_launch(m, "prefill tiles")) < 0) return rc;
    }
    {
        Timed t(m, s, KERNEL_PREFILL_PREP);
        const size_t blocks = size_t(c.T) * c.H / 8;
        pf_prepare_x_kernel<<<unsigned((blocks + 255) / 256), 256, 0, s>>>(c.x, c.act_dtype, m->xp, blocks);
        if ((rc = check_launch(m, "prefill activations")) < 0) return rc;
    }
    rc = c.meta_f16 ? launch_prefill<2, true>(m, c, m->xp, s) : launch_prefill<2, false>(m, c, m->xp, s);
    if (rc < 0) return rc;
    rc = c.meta_f16 ? launch_prefill<1, true>(m, c, m->hbuf16, s) : launch_prefill<1, false>(m, c, m->hbuf16, s);
    if (rc < 0) return rc;
    return 4;
}

}  // namespace zc
