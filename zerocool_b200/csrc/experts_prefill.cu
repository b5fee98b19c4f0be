// Prefill family: grouped GEMM over all experts' row groups on the 5th-generation tensor cores.
//
// Replaces the reference's prefill branch of encode_expert_rows (src/engine/pipeline.cpp:18-30: per expert
// and per microbatch a gathered q4_gate_up, a q4_mm and a scatter_experts launch, kernels/metal/qwen.metal
// :71-81, :63-70, :800-803) with two launches per layer over a tile list that covers every expert.
//
// Formulation ("weights as M"): for one expert, D[weight row, token] = W[rows, K] . X^T[K, tokens]. The
// 128-row weight tile is the M of tcgen05.mma, the expert's tokens are the N (padded to 16, at most 64
// per tile), so a ragged or skewed expert load costs at most 15 padded columns instead of a padded
// 128-row token tile. At 2048 tokens over 512 experts (40 tokens per expert) the launch moves 0.56 bytes per
// 80 flops: it is bound by the weight stream from HBM, not by the tensor cores, so the kernel is built to keep
// the dequantisation cheap and many bytes in flight.
//
// Arithmetic (the reference's affine form, qwen.metal:46-62, regrouped):
//     sum_k (s_g q_k + b_g) x_k  =  s_g * sum_k q_k x_k  +  b_g * sum_k x_k      per 64-wide group g
//   * the tensor cores multiply the exact integer codes q (FP16) with the FP16 activations, one fresh TMEM
//     accumulator per group (four buffers rotate);
//   * the epilogue warps read each group's accumulator (tcgen05.ld) and add it into FP32 registers scaled by
//     s_g - the scale never enters an FP16 product, so no weight is rounded;
//   * the second term is itself a small product over the groups: A' = [s_0..s_G-1 | b_0..b_G-1] (the record's
//     own FP16 metadata) times B' = [0 .. | S_0..] with S_g = sum of the token's activations in group g,
//     carried as two FP16 terms (hi, lo); the zero half meets the scales, so the tile is used as it lies in the record. It runs as extra stages after the K loop (K' in blocks of 64, hi then lo)
//     and is added with scale 1.
//   8-bit codes (u8 as in the reference's affine8_dot, qwen.metal:112-125, or int8) take the same path: two byte
//   permutes bring them into the k order the token rows are stored in.
//   NMAT = 2: gate and up tiles of the same 128 rows sit side by side in TMEM; the final epilogue applies
//             SwiGLU and stores h as FP16 in the k order the second launch consumes.
//   NMAT = 1: the down projection; the final epilogue writes FP32 rows at the slots' router positions.
//
// Roles in a CTA of 416 threads: warps 0-3 producers, warp 4 owns TMEM (alloc / dealloc) and one of its lanes
// issues the MMAs, warps 5-12 are the epilogue (warp w reads TMEM lanes 32 (w mod 4) ..; two warps share a lane
// quadrant and split the token columns).
//   producer thread r: turns the packed codes of weight row r for one group per stage into 64 FP16 integers
//     (one lop3 per two codes + one FP16 add or fma, eight 16-byte stores). The packed codes reach it through a
//     thread-private cp.async ring several stages ahead; the token rows (already FP16, in the matching k order)
//     are copied by cp.async straight into the B tile. Stage buffers use the no-swizzle K-major core-matrix
//     layout ([rows/8][k chunks][8 rows][16 bytes]; LBO = 128, SBO = 128 x chunks).
//   a stage is handed over with fence.proxy.async + mbarrier arrive; the MMA lane waits for the stage and for the
//     accumulator buffer to be drained, issues 4 (k steps of 16) x NMAT tcgen05.mma and signals with tcgen05.commit
//     both "stage buffers free" and "accumulator full".
// Every wait is bounded: after ~2^22 polls a role sets ZC_STATUS_TIMEOUT, raises the CTA's abort flag and
// leaves its loop; the CTA then frees its TMEM and exits.
#include "common.cuh"
#include <type_traits>

namespace zc {
namespace {

constexpr int PF_THREADS = 416;        // 4 producer warps, 1 MMA / TMEM warp, 8 epilogue warps
constexpr uint32_t PF_ACC = 4;         // TMEM accumulator buffers (one 64-wide group each)
constexpr int PF_M = 128;
constexpr int PF_NMAX = 64;           // tokens per tile (the N of the MMA, padded to 16)
constexpr uint32_t PF_A_BYTES = PF_M * 128;          // one matrix, one stage: 128 rows x 64 halves
constexpr uint32_t PF_B_BYTES = PF_NMAX * 128;
constexpr uint32_t PF_POLL_LIMIT = 1u << 20;     // attempts of a bounded wait (each suspends for at most ~1 us: about one second in all)

struct PfTile { int32_t expert, row0, rows, shared; };

__device__ __forceinline__ uint32_t pf_smem(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pf_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pf_smem(bar)) : "memory");
}
// One attempt: mbarrier.try_wait suspends the thread until the phase completes or the time hint (1 us) passes
// (it wakes as soon as the barrier flips, unlike a poll followed by a sleep).
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(pf_smem(bar)), "r"(parity), "r"(1000u) : "memory");       // suspend for at most ~1 us per attempt
    return ok != 0;
}
// Bounded wait. Returns false (and raises the abort flag) when the phase did not complete in time or
// another role has already given up.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {       // non-blocking probe
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(pf_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* status, uint32_t limit = PF_POLL_LIMIT) {
    if (mbar_test(bar, parity)) return true;          // the common case in a pipeline that runs ahead
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicOr(status, ZC_STATUS_TIMEOUT);
    return false;
}

// The same for the lane that feeds the tensor cores: it has nothing else to do, and the wake-up of a suspended wait
// (a few hundred clocks) is idle tensor time, so it polls without suspending. Still bounded.
__device__ __forceinline__ bool mbar_spin(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* status, uint32_t limit = PF_POLL_LIMIT) {
    for (uint32_t i = 0; i < (limit << 4); ++i) {
        if (mbar_test(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicOr(status, ZC_STATUS_TIMEOUT);
    return false;
}

// K-major, no swizzle: start address, LBO = 128 B (next k chunk), SBO = sbo bytes (next 8 rows), version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t sbo = 1024) {
    return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(128 >> 4) << 16) | (uint64_t(sbo >> 4) << 32) | (1ull << 46);
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
// Eight Q4 codes of one word -> the integers q as FP16, in the order (k0,k4) (k1,k5) (k2,k6) (k3,k7).
// (w & 0x000f000f) | 0x6400 is the half2 (1024 + q, 1024 + q'); the nibbles one position up give 1024 + 16 q.
__device__ __forceinline__ uint4 pf_dequant_word(uint32_t w) {
    const uint32_t mlo = 0x000f000fu, mhi = 0x00f000f0u, magic = 0x64006400u;
    const __half2 k1024 = __floats2half2_rn(1024.0f, 1024.0f), k16 = __floats2half2_rn(0.0625f, 0.0625f), k64 = __floats2half2_rn(-64.0f, -64.0f);
    const uint32_t w8 = w >> 8;
    uint32_t p[4] = {pf_and_or(w, mlo, magic), pf_and_or(w, mhi, magic), pf_and_or(w8, mlo, magic), pf_and_or(w8, mhi, magic)};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 q = *reinterpret_cast<__half2*>(&p[i]);
        q = (i & 1) ? __hfma2(q, k16, k64) : __hsub2(q, k1024);      // exact
        p[i] = *reinterpret_cast<const uint32_t*>(&q);
    }
    return make_uint4(p[0], p[1], p[2], p[3]);
}

// Four 8-bit codes of one word -> two half2 (k0,k1) (k2,k3) holding the integers exactly: the byte b next to 0x64 is
// the FP16 value 1024 + b; int8 codes are biased by 128 first (b ^ 0x80) and lose 1152.
__device__ __forceinline__ uint2 pf_dequant_q8_word(uint32_t w, bool is_signed) {
    if (is_signed) w ^= 0x80808080u;
    const __half2 off = is_signed ? __floats2half2_rn(1152.0f, 1152.0f) : __floats2half2_rn(1024.0f, 1024.0f);
    uint32_t lo = __byte_perm(w, 0x64646464u, 0x4140), hi = __byte_perm(w, 0x64646464u, 0x4342);
    __half2 a = __hsub2(*reinterpret_cast<__half2*>(&lo), off), b = __hsub2(*reinterpret_cast<__half2*>(&hi), off);
    return make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}

// Eight 8-bit codes (two words, k0..k3 and k4..k7) -> four half2 in the order every B tile of this file uses:
// (k0,k4) (k1,k5) (k2,k6) (k3,k7). Two byte permutes interleave the words first.
__device__ __forceinline__ uint4 pf_dequant_q8_block(uint32_t lo, uint32_t hi, bool is_signed) {
    const uint2 a = pf_dequant_q8_word(__byte_perm(lo, hi, 0x5140), is_signed);      // bytes k0, k4, k1, k5
    const uint2 b = pf_dequant_q8_word(__byte_perm(lo, hi, 0x7362), is_signed);      // bytes k2, k6, k3, k7
    return make_uint4(a.x, a.y, b.x, b.y);
}

// Tile list: one entry per (expert with work, block of PF_NMAX of its rows), the shared expert's token
// blocks first. One CTA of 1024 threads; experts <= 1024.
__global__ void __launch_bounds__(1024) pf_tiles_kernel(const int32_t* __restrict__ offsets, uint32_t E, uint32_t first_expert, uint32_t local_experts,
                                                        uint32_t T, uint32_t has_shared, uint32_t nmax, uint32_t skip_rows_upto,
                                                        PfTile* __restrict__ tiles, int32_t* __restrict__ ntiles) {
    __shared__ int warp_totals[33];
    const uint32_t e = threadIdx.x, lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const uint32_t shared_tiles = has_shared ? (T + nmax - 1) / nmax : 0;
    int rows = 0;
    if (e < E && e >= first_expert && e < first_expert + local_experts) rows = offsets[e + 1] - offsets[e];
    if (uint32_t(rows) <= skip_rows_upto) rows = 0;          // few rows: the streaming kernels take this expert
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

// Per row of an FP16 matrix [rows, K] and per 64-wide group g: S_g = sum of the row's values in the group (FP32 sum),
// stored as the B' operand of the correction stages, [0 .. | hi_0.. | 0 .. | lo_0..] with hi = fp16(S),
// lo = fp16(S - hi): 4 Gp halves per row, Gp = the group count rounded up to a multiple of eight (entries past G are
// zero); the zeros of the first half meet the scale half of the metadata tile. One warp per row.
__host__ __device__ inline uint32_t pf_padded_groups(uint32_t K) { return (K / 64 + 7) & ~7u; }
__global__ void pf_sums_kernel(const __half* __restrict__ src, uint32_t rows, uint32_t K, __half* __restrict__ sums, uint32_t* __restrict__ status) {
    const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) / 32, lane = threadIdx.x % 32;
    if (row >= rows) return;
    const uint32_t G = K / 64, Gp = pf_padded_groups(K);
    for (uint32_t g0 = 0; g0 < Gp; g0 += 4) {            // a lane adds one 16-byte piece; eight lanes cover a group
        const uint32_t g = g0 + lane / 8;
        float sum = 0.0f;
        if (g < G) {
            const uint4 raw = *reinterpret_cast<const uint4*>(src + size_t(row) * K + g * 64 + (lane % 8) * 8);
            const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); sum += f.x; sum += f.y; }
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if (g < Gp && lane % 8 == 0) {
            if (!(fabsf(sum) <= 65504.0f)) atomicOr(status, ZC_STATUS_RANGE);      // S (or an infinite input) leaves FP16
            const __half hi = __float2half_rn(sum), lo = __float2half_rn(sum - __half2float(hi));      // both zero for a padding group
            __half* dst = sums + size_t(row) * 4 * Gp;
            const __half zero = __float2half_rn(0.0f);
            dst[g] = zero; dst[Gp + g] = hi;
            dst[2 * Gp + g] = zero; dst[3 * Gp + g] = lo;
        }
    }
}

// The layer's input x [T, H] (bf16 or fp32) -> FP16 [T, H] with every block of eight k values stored in pf_pos8 order
// (the B operand of the gate/up launch, copied into shared memory with plain 16-byte cp.async), and its group sums in
// the same pass: one warp per token row, the same piece per lane and the same order of additions as pf_sums_kernel.
__global__ void pf_prepare_x_sums_kernel(const void* __restrict__ x, int act_dtype, __half* __restrict__ xp, uint32_t rows, uint32_t K,
                                         __half* __restrict__ sums, uint32_t* __restrict__ status) {
    const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) / 32, lane = threadIdx.x % 32;
    if (row >= rows) return;
    const uint32_t G = K / 64, Gp = pf_padded_groups(K);
    bool out_of_range = false;
    for (uint32_t g0 = 0; g0 < Gp; g0 += 4) {
        const uint32_t g = g0 + lane / 8;
        float sum = 0.0f;
        if (g < G) {
            const size_t at = size_t(row) * K + g * 64 + (lane % 8) * 8;
            float v[8];
            if (act_dtype == ZC_F32) {
                const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(x) + at);
                const float4 a = p[0], b = p[1];
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            } else {
                const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + at);
                const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) { v[2 * j] = __uint_as_float(r[j] << 16); v[2 * j + 1] = __uint_as_float(r[j] & 0xffff0000u); }
            }
            __half h[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { out_of_range |= fabsf(v[j]) > 65504.0f; h[pf_pos8(j)] = __float2half_rn(v[j]); }
            *reinterpret_cast<uint4*>(xp + at) = *reinterpret_cast<uint4*>(h);
#pragma unroll
            for (int j = 0; j < 8; ++j) sum += __half2float(h[j]);
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if (g < Gp && lane % 8 == 0) {
            if (!(fabsf(sum) <= 65504.0f)) out_of_range = true;
            const __half hi = __float2half_rn(sum), lo = __float2half_rn(sum - __half2float(hi));
            __half* dst = sums + size_t(row) * 4 * Gp;
            const __half zero = __float2half_rn(0.0f);
            dst[g] = zero; dst[Gp + g] = hi;
            dst[2 * Gp + g] = zero; dst[3 * Gp + g] = lo;
        }
    }
    if (out_of_range) atomicOr(status, ZC_STATUS_RANGE);
}

__device__ __forceinline__ void pf_cp16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

constexpr uint32_t PF_STAGES = 3;      // A stage buffers (written by the producers, read by the MMAs): the producers may run two stages ahead
// Prefetch distance D (template parameter of the kernel): the packed codes and the token rows of stage ks + D are
// requested while stage ks is dequantised, so that D stages of work (a few thousand cycles) cover the memory
// latency. Token-row (B) ring: D + PF_STAGES slots; per-thread ring of packed codes: D + 1 slots.

// Shared memory of one CTA (dynamic, 1024-byte aligned for the tile buffers).
template <int NMAT, int BITS>
struct PfSmem {
    static constexpr uint32_t A_STAGE = NMAT * PF_A_BYTES;
    static constexpr uint32_t A_RING = PF_STAGES * A_STAGE;
    static constexpr uint32_t RAWB = BITS * 8;                 // packed code bytes of one weight row of one group
    __host__ __device__ static uint32_t b_ring(uint32_t D) { return (D + PF_STAGES) * PF_B_BYTES; }
    __host__ __device__ static uint32_t raw_bytes(uint32_t D) { return (D + 1) * NMAT * 128 * RAWB; }       // [slot][matrix][thread][RAWB]
    // metadata tiles: per matrix 128 rows x 2 G halves in the A' layout (16 x 2 G / 8 core matrices of 128 B)
    static uint32_t meta_bytes(uint32_t G) { return NMAT * 128 * 2 * G * 2; }
    static uint32_t total(uint32_t G, uint32_t D) { return A_RING + b_ring(D) + raw_bytes(D) + meta_bytes(G) + 1024; }   // + alignment slack
};

// Grid: (weight-row tiles of 128, tiles of the list). See the file header for the roles.
// bsrc: FP16 token rows [.., K]; bsum: their group sums [.., 4 G] (pf_sums_kernel).
template <int NMAT, int BITS, bool META_F16, int D>
__global__ void __launch_bounds__(PF_THREADS, NMAT == 1 ? 2 : 1) prefill_kernel(Call c, const PfTile* __restrict__ tiles, const int32_t* __restrict__ ntiles,
                                                                 const __half* __restrict__ bsrc, const __half* __restrict__ bsum,
                                                                 __half* __restrict__ hdst, uint32_t tile_filter) {
    using S = PfSmem<NMAT, BITS>;
    constexpr uint32_t PF_RAW = D + 1, PF_BS = D + PF_STAGES;
    extern __shared__ uint8_t pf_raw_smem[];
    __shared__ __align__(8) uint64_t full_bar[PF_STAGES], done_bar[PF_STAGES], acc_full[PF_ACC], acc_free[PF_ACC], meta_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile uint32_t abort_flag;
    __shared__ uint32_t brow[PF_NMAX];            // source row index of each token row of the tile
    __shared__ long long drow[PF_NMAX];           // destination element offset of each token row
    if (blockIdx.y >= uint32_t(*ntiles)) return;
    const PfTile tile = tiles[blockIdx.y];
    if ((tile_filter == 1 && tile.shared) || (tile_filter == 2 && !tile.shared)) return;
    const uint32_t K = NMAT == 2 ? c.H : c.F, G = K / 64;
    // K stages, then the correction stages: K' = 2 G in blocks of at most 64, each as a hi and a lo term
    const uint32_t kb = 2 * G < 64 ? 2 * G : 64, nblk = 2 * G / kb, nst = G + 2 * nblk;
    const uint32_t N = uint32_t(tile.rows), Npad = (N + 15) & ~15u;
    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t r0 = blockIdx.x * PF_M;
    const uint32_t base = (pf_smem(pf_raw_smem) + 1023) & ~1023u;
    uint8_t* const sm = pf_raw_smem + (base - pf_smem(pf_raw_smem));       // the same place as a generic pointer
    auto at = [&](uint32_t shared_addr) { return sm + (shared_addr - base); };
    const uint32_t b_ring = base + S::A_RING, raw_base = b_ring + S::b_ring(D), meta_base = raw_base + S::raw_bytes(D);
    const uint32_t meta_sbo = (2 * G / 8) * 128, meta_tile = 128 * 2 * G * 2;      // A' tile of one matrix
    const uint8_t* record = tile.shared ? c.shared_record : c.records + size_t(uint32_t(tile.expert) - c.first_expert) * c.record_stride;

    // ---- set-up ----------------------------------------------------------------------------------
    if (tid == 0) {
        for (uint32_t i = 0; i < PF_STAGES; ++i) { mbar_init(&full_bar[i], 4); mbar_init(&done_bar[i], 1); }
        for (uint32_t i = 0; i < PF_ACC; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_free[i], 8); }
        mbar_init(&meta_bar, 4);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < N) {
        const uint32_t i = uint32_t(tile.row0) + tid;
        if (tile.shared) {
            brow[tid] = NMAT == 2 ? i : c.T * c.K + i;
            drow[tid] = NMAT == 2 ? (long long)(size_t(c.T) * c.K + i) * c.F : (long long)i * c.H;
        } else {
            const uint32_t pos = uint32_t(c.offsets[tile.expert]) + i, slot = uint32_t(c.perm[pos]);
            brow[tid] = NMAT == 2 ? slot / c.K : pos;
            drow[tid] = NMAT == 2 ? (long long)pos * c.F : (long long)slot * c.H;
        }
    }
    uint32_t ncols = 32;
    while (ncols < PF_ACC * NMAT * Npad) ncols <<= 1;     // PF_ACC accumulator buffers of NMAT x Npad columns
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pf_smem(&tmem_base_s)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    uint32_t* status = c.status;
    const Projection pr[2] = {NMAT == 2 ? c.gate : c.down, c.up};

    if (warp < 4) {
        // ---- producers -----------------------------------------------------------------------------
        const uint32_t r = tid;                                   // weight row of the tile
        const uint8_t* codes[NMAT];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) codes[m] = record + pr[m].codes + size_t(r0 + r) * (K * BITS / 8);
        // metadata of row r -> A' tiles [s_0..s_G-1 | b_0..b_G-1] as FP16, core-matrix layout
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
            const uint8_t* sc = record + pr[m].scales + size_t(r0 + r) * G * 2;
            const uint8_t* bi = record + pr[m].biases + size_t(r0 + r) * G * 2;
            const uint32_t dst = meta_base + m * meta_tile + (r / 8) * meta_sbo + (r % 8) * 16;
            for (uint32_t ch = 0; ch < G / 8; ++ch) {
                if (META_F16) {
                    pf_cp16(dst + ch * 128, sc + ch * 16);
                    pf_cp16(dst + (G / 8 + ch) * 128, bi + ch * 16);
                } else {
                    const uint4 a = *reinterpret_cast<const uint4*>(sc + ch * 16), b = *reinterpret_cast<const uint4*>(bi + ch * 16);
                    const uint32_t ra[4] = {a.x, a.y, a.z, a.w}, rb[4] = {b.x, b.y, b.z, b.w};
                    uint32_t ha[4], hb[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const __half2 x = __floats2half2_rn(__uint_as_float(ra[i] << 16), __uint_as_float(ra[i] & 0xffff0000u));
                        const __half2 y = __floats2half2_rn(__uint_as_float(rb[i] << 16), __uint_as_float(rb[i] & 0xffff0000u));
                        ha[i] = *reinterpret_cast<const uint32_t*>(&x); hb[i] = *reinterpret_cast<const uint32_t*>(&y);
                    }
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + ch * 128), "r"(ha[0]), "r"(ha[1]), "r"(ha[2]), "r"(ha[3]) : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + (G / 8 + ch) * 128), "r"(hb[0]), "r"(hb[1]), "r"(hb[2]), "r"(hb[3]) : "memory");
                }
            }
        }
        // K stages: this thread's pieces of the token rows, addresses prepared once (q = tid + 128 i: row q / 8, chunk q % 8)
        const __half* bsrc_i[PF_NMAX * 8 / 128];
        uint32_t bdst_i[PF_NMAX * 8 / 128];
#pragma unroll
        for (int i = 0; i < PF_NMAX * 8 / 128; ++i) {
            const uint32_t q = tid + 128 * i, j = q / 8, kc = q % 8;
            bsrc_i[i] = j < N ? bsrc + size_t(brow[j]) * K + kc * 8 : nullptr;
            bdst_i[i] = (j / 8) * 1024 + kc * 128 + (j % 8) * 16;
        }
        auto issue_raw = [&](uint32_t ks) {          // packed codes of group ks
            if (ks >= G) return;
            const uint32_t slot = ks % PF_RAW;
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                const uint32_t dst = raw_base + ((slot * NMAT + m) * 128 + r) * S::RAWB;
#pragma unroll
                for (uint32_t piece = 0; piece < S::RAWB; piece += 16) pf_cp16(dst + piece, codes[m] + ks * S::RAWB + piece);
            }
        };
        // token rows of stage ks, 16-byte pieces straight into the tile: 64 k of the rows for a K stage, the 2 G
        // group sums (hi for stage G, lo for stage G+1) for a correction stage
        auto issue_b = [&](uint32_t ks) {
            if (ks >= nst) return;
            const uint32_t bs = b_ring + (ks % PF_BS) * PF_B_BYTES;
            const bool main = ks < G;
            if (main) {
#pragma unroll
                for (int i = 0; i < PF_NMAX * 8 / 128; ++i) if (bsrc_i[i]) pf_cp16(bs + bdst_i[i], bsrc_i[i] + ks * 64);
                return;
            }
            const uint32_t chunks = kb / 8;
            const uint32_t term = main ? 0 : (ks - G) / nblk, blk = main ? 0 : (ks - G) % nblk;     // hi / lo, block of K'
            for (uint32_t q = tid; q < N * chunks; q += 128) {
                const uint32_t j = q / chunks, kc = q % chunks;
                const __half* src = main ? bsrc + size_t(brow[j]) * K + ks * 64 + kc * 8
                                         : bsum + size_t(brow[j]) * 4 * G + term * 2 * G + blk * kb + kc * 8;
                pf_cp16(bs + (j / 8) * (chunks * 128) + kc * 128 + (j % 8) * 16, src);
            }
        };
        bool ok = true;
        // prologue: copy group j holds the token rows and the codes of stage j (group 0 also the metadata)
#pragma unroll 1
        for (uint32_t j = 0; j < uint32_t(D); ++j) {
            issue_b(j); issue_raw(j);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        // done_bar[j % PF_STAGES] completes phase j / PF_STAGES when the MMAs of stage j have drained.
        auto stage_done = [&](uint32_t j) { return mbar_wait(&done_bar[j % PF_STAGES], (j / PF_STAGES) & 1, &abort_flag, status); };
        for (uint32_t ks = 0; ks < nst && ok; ++ks) {
            // group ks (token rows and codes of this stage) is complete when at most D - 1 later groups are pending
            asm volatile("cp.async.wait_group %0;" ::"n"(D - 1) : "memory");
            // the A buffer of this stage was last read by stage ks - PF_STAGES; MMAs complete in order, so every
            // earlier stage has drained too and the B slot of stage ks + D (last used by stage ks - PF_STAGES) is free
            if (ks >= PF_STAGES) ok = stage_done(ks - PF_STAGES);
            ok = __all_sync(0xffffffffu, ok);          // warp-uniform: the hand-over below synchronises the warp
            if (!ok) break;
            issue_b(ks + D);
            issue_raw(ks + D);
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (ks < G) {
                const uint32_t as = base + (ks % PF_STAGES) * S::A_STAGE;
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                    const uint32_t src = raw_base + (((ks % PF_RAW) * NMAT + m) * 128 + r) * S::RAWB;
                    const uint32_t dst = as + m * PF_A_BYTES + (r / 8) * 1024 + (r % 8) * 16;
                    if constexpr (BITS == 4) {
                        const uint4 w0 = *reinterpret_cast<const uint4*>(at(src)), w1 = *reinterpret_cast<const uint4*>(at(src + 16));
                        const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const uint4 v = pf_dequant_word(words[i]);
                            *reinterpret_cast<uint4*>(at(dst + i * 128)) = v;
                        }
                    } else {
                        const bool q8s = c.q8_signed;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {             // 16 bytes = 16 codes = two k chunks of eight
                            const uint4 w = *reinterpret_cast<const uint4*>(at(src + i * 16));
                            *reinterpret_cast<uint4*>(at(dst + (2 * i) * 128)) = pf_dequant_q8_block(w.x, w.y, q8s);
                            *reinterpret_cast<uint4*>(at(dst + (2 * i + 1) * 128)) = pf_dequant_q8_block(w.z, w.w, q8s);
                        }
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            // one arrival per warp: 128 arrivals on one barrier would serialise in shared memory
            __syncwarp();
            if (lane == 0) {
                if (ks == 0) mbar_arrive(&meta_bar);      // one-shot: the metadata tiles (first copy group) are in place
                mbar_arrive(&full_bar[ks % PF_STAGES]);
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else if (warp == 4) {
        // ---- MMA issue: the whole warp runs the loop (waits and addresses stay warp-uniform), one lane issues ----
        {
            // instruction descriptor: D = F32, A = B = F16, both K-major, N = Npad, M = 128
            const uint32_t idesc = (1u << 4) | ((Npad >> 3) << 17) | ((PF_M >> 4) << 24);
            const uint64_t desc0 = umma_desc(base);
            bool ok = true;
            for (uint32_t ks = 0; ks < nst; ++ks) {
                ok = mbar_wait(&full_bar[ks % PF_STAGES], (ks / PF_STAGES) & 1, &abort_flag, status);
                if (ok && ks >= PF_ACC) ok = mbar_wait(&acc_free[ks % PF_ACC], ((ks / PF_ACC) - 1) & 1, &abort_flag, status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t bs = b_ring + (ks % PF_BS) * PF_B_BYTES;
                const uint32_t acc = tmem_base + (ks % PF_ACC) * NMAT * Npad;
                // descriptors differ from desc0 only in the start address field (bits 0-13, units of 16 bytes)
                const uint64_t adesc = desc0 + (((ks % PF_STAGES) * S::A_STAGE) >> 4), bdesc = desc0 + ((S::A_RING + (ks % PF_BS) * PF_B_BYTES) >> 4);
                if (lane == 0) {
                    if (ks < G) {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                            for (int m = 0; m < NMAT; ++m) umma_f16(acc + m * Npad, adesc + ((m * PF_A_BYTES + kk * 256) >> 4), bdesc + ((kk * 256) >> 4), idesc, kk != 0);
                        }
                    } else {
                        const uint32_t blk = (ks - G) % nblk;
                        for (uint32_t kk = 0; kk < kb / 16; ++kk) {
                            const uint64_t bd = umma_desc(bs + kk * 256, (kb / 8) * 128);
#pragma unroll
                            for (int m = 0; m < NMAT; ++m)
                                umma_f16(acc + m * Npad, umma_desc(meta_base + m * meta_tile + blk * (kb / 8) * 128 + kk * 256, meta_sbo), bd, idesc, kk != 0);
                        }
                    }
                    umma_commit(&done_bar[ks % PF_STAGES]);
                    umma_commit(&acc_full[ks % PF_ACC]);
                }
                __syncwarp();
            }
        }
        __syncwarp();
    } else {
        // ---- epilogue: TMEM lane 32 * (warp mod 4) + lane is weight row r; columns are the tile's tokens. Two
        // warps share a lane quadrant: set 0 takes the 16-column chunks 0 and 2, set 1 the chunks 1 and 3. ----
        const uint32_t r = (warp % 4) * 32 + lane, set = (warp - 5) / 4;
        const uint32_t lane_addr = tmem_base + (((warp % 4) * 32) << 16);
        float acc[NMAT][2][16];
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[m][h][j] = 0.0f;
        bool ok = true;
        // the metadata tiles are written by the producers (cp.async): wait for their one-shot barrier
        ok = __all_sync(0xffffffffu, mbar_wait(&meta_bar, 0, &abort_flag, status));
        for (uint32_t ks = 0; ks < nst && ok; ++ks) {
            float scale[NMAT];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                scale[m] = 1.0f;
                if (ks < G) {
                    scale[m] = __half2float(*reinterpret_cast<const __half*>(at(meta_base + m * meta_tile + (r / 8) * meta_sbo + (ks / 8) * 128 + (r % 8) * 16 + (ks % 8) * 2)));
                }
            }
            ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[ks % PF_ACC], (ks / PF_ACC) & 1, &abort_flag, status));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t buf = lane_addr + (ks % PF_ACC) * NMAT * Npad;
            uint32_t d[NMAT][2][16];
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t c0 = (2 * h + set) * 16;
                    if (c0 < Npad) tmem_ld16(buf + m * Npad + c0, d[m][h]);
                }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_free[ks % PF_ACC]);
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if ((2 * h + set) * 16 < Npad) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[m][h][j] = __fmaf_rn(scale[m], __uint_as_float(d[m][h][j]), acc[m][h][j]);
                    }
                }
        }
        if (ok) {
            const uint32_t row = r0 + r;
            float* out_base = tile.shared ? c.shared_out : c.expert_out;
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const uint32_t t = (2 * h + set) * 16 + j;
                    if (t < N) {
                        const float g = acc[0][h][j];
                        if constexpr (NMAT == 2) {
                            const float u = acc[NMAT - 1][h][j];
                            const float hv = (g * sigmoid_f(g)) * u;
                            hdst[drow[t] + (row & ~7u) + pf_pos8(row & 7)] = __float2half_rn(hv);
                        } else {
                            out_base[drow[t] + row] = g;
                        }
                    }
                }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 4) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ncols) : "memory");
    }
}

// =================================================================================================
// Wide-tile kernel: accumulators that stay in TMEM for the whole K, weights fed to the tensor cores from TMEM.
//
// The kernel above hands every 64-wide group from the tensor cores to the epilogue warps (one TMEM drain per
// group), and its token tile is at most 64 columns: per stage it offers 128-256 cycles of tensor work against a
// hand-over chain of well over a thousand. This kernel removes the per-group drain. The per-group scale rides in
// the A operand instead, without rounding any weight: the product s_g * q of an FP16 scale (11 significant bits) and
// an integer code needs up to 19 bits, so it is written as two FP16 terms, hi = fl(s q) and lo = s q - hi (the error
// of a rounded product is itself representable: one fused multiply-add gives it exactly), and both terms are
// multiplied into the same accumulator. Every product the tensor cores form is then exact and they accumulate in
// FP32, as before; the bias term b_g * sum_k x_k still runs as correction stages after the K loop.
//   tile   : 128 weight rows x up to 128 tokens (N padded to 16) x two matrices - gate and up of the same rows
//            (NMAT = 2, SwiGLU in the final epilogue) or two 128-row blocks of the down projection (NMAT = 1) -
//            so each staged token tile meets 256 weight rows; two FP32 accumulators of N columns in TMEM.
//   A      : the dequantised weights never touch shared memory. A first version staged them there (two terms x two
//            matrices = 32 KB written and read per 32 k) and measured shared-memory bound: 112 KB per stage through a
//            128 B/clock pipe is 860 clocks against 512 of tensor work. Producer thread r now writes its row's FP16
//            pairs straight into TMEM lane r (tcgen05.st, eight 32-bit columns per 16 k) and the MMAs take A from
//            tensor memory; a ring of two or three stages (128 columns each) sits beside the accumulators.
//   B      : [N x 64] FP16 per stage in shared memory (K-major core-matrix layout without swizzle: LBO 128 B, SBO 1024 B).
//   stage  : one 64-wide quantisation group = 16 MMAs (4 k steps x 2 matrices x 2 terms). Clock stamps showed the MMAs
//            issuing at the tensor rate (64 clocks each at N = 128) and every wait, fence and commit of the issuing
//            warp as idle tensor time, so a stage carries as much tensor work as TMEM allows and costs that warp one
//            wait and one commit.
//   roles  : warps 0-7 producers (warp w: matrix w / 4, TMEM lane quadrant w mod 4). Packed codes (whole 128-byte lines
//            of the warp's 32 rows, double-buffered) and token rows (DR stages ahead) both arrive through the producers'
//            cp.async stream: the token-row ring has DR + NA slots, so
//            the slot a producer refills was released by the same completed-stage barrier it waits on for its TMEM
//            columns. The same warps then run the final epilogue on their quadrant. One lane each of warps 8 and 9 issue
//            the MMAs of alternate stages and release a stage with one tcgen05.commit.
// Every wait is bounded as above.
constexpr int PW_NMAX = 128;
constexpr uint32_t PW_K = 64;
constexpr uint32_t PW_B_STAGE = PW_NMAX * PW_K * 2;       // 16 KB
constexpr uint32_t PW_A_COLS = 128;                       // TMEM columns of one A stage: [matrix][term][16-k block][8]
constexpr uint32_t PW_TMEM_COLS = 512;
constexpr uint32_t PW_NA_MAX = 3;
constexpr int PW_THREADS = 320;                           // producers / epilogue 0-7, MMA issue 8-9

// Development aid (build with -DZC_PW_STAMPS): the first CTA of a launch records clock64() at fixed points of each
// role's loop, read back through zc_dbg_prefill_stamps. Compiled out otherwise.
#ifdef ZC_PW_STAMPS
__device__ unsigned long long pw_stamps[4][96][8];
#define PW_STAMP(role, stage, slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (stage) < 96 && lane == 0 && (warp == 0 || warp >= 8)) pw_stamps[role][stage][slot] = clock64(); } while (0)
#else
#define PW_STAMP(role, stage, slot) do {} while (0)
#endif

// A BF16 scale or bias must survive the conversion to FP16 (the A' operand of the correction stages and the factor of the
// two-term weights): zero, or a magnitude in [2^-14, 65504]. Anything else is reported, not silently rounded.
__device__ __forceinline__ bool pw_meta_fits_f16(float v) { const float a = fabsf(v); return a == 0.0f || (a >= 6.103515625e-5f && a <= 65504.0f); }

struct PwSmem {
    uint32_t b_ring, raw, meta, total;
    __host__ __device__ PwSmem(uint32_t G, uint32_t DR, uint32_t bits) {
        b_ring = 0;
        raw = b_ring + (DR + PW_NA_MAX) * PW_B_STAGE;
        meta = raw + 2 * 8 * 32 * 128;                    // packed codes: [slot 0..1][producer warp][row of the warp][128 B]
        total = meta + 2 * 128 * 2 * G * 2 + 1024;        // two metadata tiles [128 x 2 G] FP16, + alignment slack
        if (total < 116 * 1024) total = 116 * 1024;       // one CTA per SM: a CTA takes all 512 TMEM columns
    }
};

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
// D (TMEM) += A (TMEM, lane = row, two FP16 per 32-bit column) * B (shared memory descriptor).
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

template <int NMAT, int BITS, int DR>
__global__ void __launch_bounds__(PW_THREADS, 1) prefill_wide_kernel(Call c, const PfTile* __restrict__ tiles, const int32_t* __restrict__ ntiles,
                                                                    const __half* __restrict__ bsrc, const __half* __restrict__ bsum,
                                                                    __half* __restrict__ hdst, uint32_t tile_filter) {
    constexpr uint32_t RAWB = BITS * 8;                   // packed bytes of one weight row of one stage
    constexpr uint32_t SUPER = 128 / RAWB;                // stages whose packed codes arrive in one 128-byte line per row: 4 (Q4), 2 (Q8)
    static_assert(DR <= int(SUPER), "the line of the next stages must have landed when its first stage begins");
    extern __shared__ uint8_t pf_raw_smem[];
    __shared__ __align__(8) uint64_t full[PW_NA_MAX], done[PW_NA_MAX], turn[2], meta_bar, acc_done, drain_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile uint32_t abort_flag;
    __shared__ uint32_t brow[PW_NMAX];
    __shared__ long long drow[PW_NMAX];
    if (blockIdx.y >= uint32_t(*ntiles)) return;
    const PfTile tile = tiles[blockIdx.y];
    if ((tile_filter == 1 && tile.shared) || (tile_filter == 2 && !tile.shared)) return;      // 1: routed tiles only, 2: shared tiles only
#ifdef ZC_PW_STAMPS
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) pw_stamps[1][2][0] = clock64();
#endif
    const uint32_t K = NMAT == 2 ? c.H : c.F, G = K / 64, Gp = pf_padded_groups(K);
    const uint32_t nmain = G;
    // correction stages: K' = 2 Gp metadata columns (scales, then biases, each padded to Gp) in blocks of kb
    const uint32_t kb = (2 * Gp) % 64 == 0 ? 64u : (2 * Gp) % 32 == 0 ? 32u : 16u, nblk = 2 * Gp / kb, ncorr = 2 * nblk, nst = nmain + ncorr;
    const uint32_t N = uint32_t(tile.rows), Npad = (N + 15) & ~15u;
    const uint32_t NA = Npad > 64 ? 2u : 3u;               // A stages beside two accumulators of Npad columns
    const uint32_t NB = DR + NA;                           // token-row slots
    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t r0 = blockIdx.x * (NMAT == 2 ? 128u : 256u);
    const PwSmem L(Gp, DR, BITS);
    const uint32_t base = (pf_smem(pf_raw_smem) + 1023) & ~1023u;
    uint8_t* const sm = pf_raw_smem + (base - pf_smem(pf_raw_smem));
    auto at = [&](uint32_t shared_addr) { return sm + (shared_addr - base); };
    const uint32_t b_ring = base + L.b_ring, raw_base = base + L.raw, meta_base = base + L.meta;
    const uint32_t meta_sbo = (2 * Gp / 8) * 128, meta_tile = 128 * 2 * Gp * 2;
    const uint8_t* record = tile.shared ? c.shared_record : c.records + size_t(uint32_t(tile.expert) - c.first_expert) * c.record_stride;
    uint32_t* status = c.status;

    if (tid == 0) {
        for (uint32_t i = 0; i < PW_NA_MAX; ++i) { mbar_init(&full[i], 8); mbar_init(&done[i], 1); }
        mbar_init(&meta_bar, 8); mbar_init(&acc_done, 1); mbar_init(&drain_bar, 2); mbar_init(&turn[0], 1); mbar_init(&turn[1], 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < N) {
        const uint32_t i = uint32_t(tile.row0) + tid;
        if (tile.shared) {
            brow[tid] = NMAT == 2 ? i : c.T * c.K + i;
            drow[tid] = NMAT == 2 ? (long long)(size_t(c.T) * c.K + i) * c.F : (long long)i * c.H;
        } else {
            const uint32_t pos = uint32_t(c.offsets[tile.expert]) + i, slot = uint32_t(c.perm[pos]);
            brow[tid] = NMAT == 2 ? slot / c.K : pos;
            drow[tid] = NMAT == 2 ? (long long)pos * c.F : (long long)slot * c.H;
        }
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pf_smem(&tmem_base_s)), "r"(PW_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
#ifdef ZC_PW_STAMPS
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) pw_stamps[1][2][1] = clock64();
#endif
    const uint32_t tmem_a = tmem_base + 2 * Npad;           // A ring: stage s at columns s * PW_A_COLS, then [matrix][term][block][8]

    if (warp < 8) {
        // ---- producers: thread (m, r) owns weight row r of matrix m ---------------------------------------
        PW_STAMP(1, 0, 0);
        const uint32_t m = warp / 4, quad = warp % 4, r = quad * 32 + lane;
        const Projection pr = NMAT == 2 ? (m == 0 ? c.gate : c.up) : c.down;
        const uint32_t mrow = r0 + (NMAT == 1 ? m * 128u : 0u) + r;
        const uint32_t row_bytes = K * BITS / 8;
        // Packed codes: the warp fetches the lines of its own 32 rows together - eight lanes take the eight 16-byte pieces
        // of one row's 128-byte line, four rows per instruction - so that every request is a whole line (one 16-byte piece
        // per thread from 32 different rows, as the first version had it, costs 32 tag look-ups per instruction and made
        // the issue of a stage take ~1,500 clocks). A line holds the codes of SUPER stages. In shared memory the pieces of a
        // row are xor-swizzled by the row so that the per-row reads below spread over the banks.
        const uint8_t* code_lines = record + pr.codes + size_t(mrow - lane + lane / 8) * row_bytes + (lane % 8) * 16;      // row (lane / 8) of the warp, piece lane % 8
        const uint32_t raw_warp = raw_base + warp * (32 * 128);
        const uint32_t lane_base = (quad * 32) << 16;
        // metadata of the row -> A' tile [s_0..s_G-1 | b_0..b_G-1] as FP16 (the correction stages' A operand, and where
        // this thread reads its scales)
        bool meta_bad = false;
        {
            const uint8_t* sc = record + pr.scales + size_t(mrow) * G * 2;
            const uint8_t* bi = record + pr.biases + size_t(mrow) * G * 2;
            const uint32_t dst = meta_base + m * meta_tile + (r / 8) * meta_sbo + (r % 8) * 16;
            if (G % 8 == 0) {
                for (uint32_t ch = 0; ch < G / 8; ++ch) {
                    if (c.meta_f16) {
                        pf_cp16(dst + ch * 128, sc + ch * 16);
                        pf_cp16(dst + (G / 8 + ch) * 128, bi + ch * 16);
                    } else {
                        const uint4 a = *reinterpret_cast<const uint4*>(sc + ch * 16), b = *reinterpret_cast<const uint4*>(bi + ch * 16);
                        const uint32_t ra[4] = {a.x, a.y, a.z, a.w}, rb[4] = {b.x, b.y, b.z, b.w};
                        uint32_t ha[4], hb[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float s0 = __uint_as_float(ra[i] << 16), s1 = __uint_as_float(ra[i] & 0xffff0000u);
                            const float b0 = __uint_as_float(rb[i] << 16), b1 = __uint_as_float(rb[i] & 0xffff0000u);
                            meta_bad |= !(pw_meta_fits_f16(s0) && pw_meta_fits_f16(s1) && pw_meta_fits_f16(b0) && pw_meta_fits_f16(b1));
                            const __half2 x = __floats2half2_rn(s0, s1);
                            const __half2 y = __floats2half2_rn(b0, b1);
                            ha[i] = *reinterpret_cast<const uint32_t*>(&x); hb[i] = *reinterpret_cast<const uint32_t*>(&y);
                        }
                        *reinterpret_cast<uint4*>(at(dst + ch * 128)) = make_uint4(ha[0], ha[1], ha[2], ha[3]);
                        *reinterpret_cast<uint4*>(at(dst + (G / 8 + ch) * 128)) = make_uint4(hb[0], hb[1], hb[2], hb[3]);
                    }
                }
            } else {
                // a group count that is not a multiple of eight (ffn 640: ten groups): the row's metadata is not 16-byte
                // aligned, so it is read value by value; the columns past G are zero
                for (uint32_t g = 0; g < Gp; ++g) {
                    __half sv = __float2half_rn(0.0f), bv = sv;
                    if (g < G) {
                        const uint16_t sr = *reinterpret_cast<const uint16_t*>(sc + g * 2), br = *reinterpret_cast<const uint16_t*>(bi + g * 2);
                        sv = c.meta_f16 ? __ushort_as_half(sr) : __float2half_rn(bf_to_float(sr));
                        bv = c.meta_f16 ? __ushort_as_half(br) : __float2half_rn(bf_to_float(br));
                        if (!c.meta_f16) meta_bad |= !(pw_meta_fits_f16(bf_to_float(sr)) && pw_meta_fits_f16(bf_to_float(br)));
                    }
                    *reinterpret_cast<__half*>(at(dst + (g / 8) * 128 + (g % 8) * 2)) = sv;
                    *reinterpret_cast<__half*>(at(dst + (Gp / 8 + g / 8) * 128 + (g % 8) * 2)) = bv;
                }
            }
        }
        if (meta_bad) atomicOr(status, ZC_STATUS_RANGE);
        PW_STAMP(1, 0, 1);
        // Token rows of a main stage: 128 bytes per row = 8 pieces; thread t copies piece (row t / 8 + 32 i, chunk t mod 8)
        // for i < 4. The row pointers are prepared once; a stage adds 128 bytes.
        const __half* src_i[PW_NMAX / 32];
#pragma unroll
        for (int i = 0; i < PW_NMAX / 32; ++i) {
            const uint32_t row = tid / 8 + 32 * i;
            src_i[i] = row < N ? bsrc + size_t(brow[row]) * K + (tid % 8) * 8 : nullptr;
        }
        const uint32_t dst_piece = (tid / 64) * 1024 + (tid % 8) * 128 + ((tid / 8) % 8) * 16;     // + i * 4096
        auto issue_codes = [&](uint32_t line) {          // the 128-byte lines holding stages line * SUPER .. of this warp's rows
            if (line * SUPER >= nmain) return;
            const uint32_t slot = raw_warp + (line & 1) * (8 * 32 * 128);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t row = uint32_t(i) * 4 + lane / 8;
                pf_cp16(slot + row * 128 + (((lane % 8) ^ (row & 7)) * 16), code_lines + size_t(i) * 4 * row_bytes + size_t(line) * 128);
            }
        };
        auto issue_stage = [&](uint32_t j) {             // the token rows (or group sums) of stage j, into slot j of their ring
            if (j >= nst) return;
            const uint32_t bs = b_ring + (j % NB) * PW_B_STAGE;
            if (j < nmain) {
#pragma unroll
                for (int i = 0; i < PW_NMAX / 32; ++i) if (src_i[i]) pf_cp16(bs + i * 4096 + dst_piece, src_i[i] + j * PW_K);
            } else {
                const uint32_t chunks = kb / 8, term = (j - nmain) / nblk, blk = (j - nmain) % nblk;
                for (uint32_t q = tid; q < N * chunks; q += 256) {
                    const uint32_t row = q / chunks, kc = q % chunks;
                    pf_cp16(bs + (row / 8) * (chunks * 128) + kc * 128 + (row % 8) * 16, bsum + size_t(brow[row]) * 4 * Gp + term * 2 * Gp + blk * kb + kc * 8);
                }
            }
        };
        PW_STAMP(1, 0, 2);
        issue_codes(0);
#pragma unroll 1
        for (uint32_t j = 0; j < uint32_t(DR); ++j) {
            issue_stage(j);
            asm volatile("cp.async.commit_group;" ::: "memory");
            PW_STAMP(1, 1, j);
        }
        bool ok = true;
        const bool q8s = c.q8_signed;
        const uint32_t scale_at = meta_base + m * meta_tile + (r / 8) * meta_sbo + (r % 8) * 16;
        for (uint32_t ks = 0; ks < nst && ok; ++ks) {
            PW_STAMP(0, ks, 0);
            asm volatile("cp.async.wait_group %0;" ::"n"(DR - 1) : "memory");       // this thread's copies for stage ks (and, at ks = 0, the metadata) have landed
            PW_STAMP(0, ks, 1);
            // stage ks - NA has drained: its TMEM columns, and the token-row slot that stage ks + DR will use, are free
            if (ks >= NA) ok = mbar_wait(&done[ks % NA], ((ks / NA) - 1) & 1, &abort_flag, status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            PW_STAMP(0, ks, 2);
            issue_stage(ks + DR);
            if (ks % SUPER == 0) issue_codes(ks / SUPER + 1);       // into the slot whose stages this warp finished reading an iteration ago
            asm volatile("cp.async.commit_group;" ::: "memory");
            __syncwarp();                                           // the other lanes' pieces of this row's line have landed too
            if (ks < nmain) {
                const __half sh = *reinterpret_cast<const __half*>(at(scale_at + (ks / 8) * 128 + (ks % 8) * 2));
                const __half2 s2 = __half2half2(sh);
                const uint32_t src = raw_warp + ((ks / SUPER) & 1) * (8 * 32 * 128) + lane * 128;      // this row's line
                const uint32_t sub = ks % SUPER;
                const uint32_t ta = tmem_a + lane_base + (ks % NA) * PW_A_COLS + m * 64;       // this row's columns: [term][block][8]
                auto two_terms = [&](uint32_t q_bits, uint32_t& hi, uint32_t& lo) {      // q exact -> fl(s q), s q - fl(s q)
                    const __half2 q = *reinterpret_cast<const __half2*>(&q_bits);
                    const __half2 h = __hmul2(q, s2);
                    const __half2 l = __hfma2(q, s2, __hneg2(h));
                    hi = *reinterpret_cast<const uint32_t*>(&h); lo = *reinterpret_cast<const uint32_t*>(&l);
                };
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");      // the MMAs that read these columns have completed
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) {                // 16 k per block: eight packed columns per term
                    uint32_t hi[8], lo[8];
                    if constexpr (BITS == 4) {
                        const uint32_t piece = sub * 2 + blk / 2;
                        const uint2 w = *reinterpret_cast<const uint2*>(at(src + ((piece ^ (lane & 7)) * 16) + (blk % 2) * 8));
                        const uint4 qa = pf_dequant_word(w.x), qb = pf_dequant_word(w.y);
                        two_terms(qa.x, hi[0], lo[0]); two_terms(qa.y, hi[1], lo[1]); two_terms(qa.z, hi[2], lo[2]); two_terms(qa.w, hi[3], lo[3]);
                        two_terms(qb.x, hi[4], lo[4]); two_terms(qb.y, hi[5], lo[5]); two_terms(qb.z, hi[6], lo[6]); two_terms(qb.w, hi[7], lo[7]);
                    } else {
                        const uint32_t piece = sub * 4 + blk;
                        const uint4 w = *reinterpret_cast<const uint4*>(at(src + ((piece ^ (lane & 7)) * 16)));
                        const uint4 qa = pf_dequant_q8_block(w.x, w.y, q8s), qb = pf_dequant_q8_block(w.z, w.w, q8s);
                        two_terms(qa.x, hi[0], lo[0]); two_terms(qa.y, hi[1], lo[1]); two_terms(qa.z, hi[2], lo[2]); two_terms(qa.w, hi[3], lo[3]);
                        two_terms(qb.x, hi[4], lo[4]); two_terms(qb.y, hi[5], lo[5]); two_terms(qb.z, hi[6], lo[6]); two_terms(qb.w, hi[7], lo[7]);
                    }
                    tmem_st8(ta + 0 * 32 + blk * 8, hi);
                    tmem_st8(ta + 1 * 32 + blk * 8, lo);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            PW_STAMP(0, ks, 3);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the token rows (and at ks = 0 the metadata tile) for the MMAs
            __syncwarp();
            if (lane == 0) {
                if (ks == 0) mbar_arrive(&meta_bar);      // one-shot: the metadata tiles are in place
                mbar_arrive(&full[ks % NA]);
            }
            PW_STAMP(0, ks, 4);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        // ---- final epilogue on this warp's lane quadrant: TMEM lane r is weight row r; the two warps of a quadrant
        // (m = 0, 1) take alternate 16-column chunks ---------------------------------------------------------
        PW_STAMP(3, 0, 0);
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&acc_done, 0, &abort_flag, status));
        PW_STAMP(3, 0, 1);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float* out_base = tile.shared ? c.shared_out : c.expert_out;
            const uint32_t row = r0 + r;
            for (uint32_t chunk = m; chunk * 16 < Npad; chunk += 2) {
                uint32_t d0[16], d1[16];
                tmem_ld16(tmem_base + lane_base + chunk * 16, d0);
                tmem_ld16(tmem_base + lane_base + Npad + chunk * 16, d1);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const uint32_t t = chunk * 16 + j;
                    if (t < N) {
                        const float a = __uint_as_float(d0[j]), b = __uint_as_float(d1[j]);
                        if constexpr (NMAT == 2) {
                            const float hv = (a * sigmoid_f(a)) * b;
                            hdst[drow[t] + (row & ~7u) + pf_pos8(row & 7)] = __float2half_rn(hv);
                        } else {
                            out_base[drow[t] + row] = a;
                            out_base[drow[t] + row + 128] = b;
                        }
                    }
                }
            }
        }
        PW_STAMP(3, 0, 2);
    } else {
        // ---- MMA issue (warps 8 and 9): whatever the issuing lane does besides issuing is idle tensor time - the MMAs
        // leave at the tensor rate, so the queue behind the lane is shallow. Two lanes therefore alternate: warp 8 takes
        // the even stages, warp 9 the odd ones; a lane waits for its stage's operands while the other one issues, takes
        // the turn (one mbarrier hand-over, ordered by the tcgen05 fences), issues, passes the turn on and only then
        // commits. All MMAs of the tile still reach the tensor pipe in stage order.
        const uint32_t idesc = (1u << 4) | ((Npad >> 3) << 17) | ((PF_M >> 4) << 24);       // D = F32, A = B = F16, K-major, N = Npad, M = 128
        const uint32_t me = warp - 8;
        if (lane == 0) {
            bool ok = true;
            for (uint32_t j = me; j < nst; j += 2) {
                const bool main = j < nmain;
                PW_STAMP(2, j, 0);
                if (j >= nmain) ok = mbar_spin(&meta_bar, 0, &abort_flag, status);
                if (ok) ok = mbar_spin(&full[j % NA], (j / NA) & 1, &abort_flag, status);
                if (ok && j > 0) ok = mbar_spin(&turn[(j - 1) & 1], ((j - 1) / 2) & 1, &abort_flag, status);      // stage j - 1 has been issued
                if (!ok) break;
                PW_STAMP(2, j, 1);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t bs = b_ring + (j % NB) * PW_B_STAGE;
                if (main) {
                    const uint32_t ta = tmem_a + (j % NA) * PW_A_COLS;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint64_t bd = umma_desc(bs + kk * 256, 1024);
#pragma unroll
                        for (int m = 0; m < 2; ++m)
#pragma unroll
                            for (int term = 0; term < 2; ++term)
                                umma_f16_ts(tmem_base + m * Npad, ta + m * 64 + term * 32 + kk * 8, bd, idesc, (j | kk | term) != 0);
                    }
                } else {
                    const uint32_t blk = (j - nmain) % nblk;
                    for (uint32_t kk = 0; kk < kb / 16; ++kk) {
                        const uint64_t bd = umma_desc(bs + kk * 256, (kb / 8) * 128);
#pragma unroll
                        for (int m = 0; m < 2; ++m)
                            umma_f16(tmem_base + m * Npad, umma_desc(meta_base + m * meta_tile + blk * (kb / 8) * 128 + kk * 256, meta_sbo), bd, idesc, 1);
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(&turn[j & 1]);
                PW_STAMP(2, j, 2);
                umma_commit(&done[j % NA]);
                if (j + 1 == nst) umma_commit(&acc_done);
                PW_STAMP(2, j, 3);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp >= 8) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // After an aborted run MMAs may still be in flight: both issuing lanes commit, and the columns are returned only
        // after everything issued has drained (bounded).
        if (abort_flag) {
            if (lane == 0) umma_commit(&drain_bar);
            __syncwarp();
            if (warp == 8) for (uint32_t i = 0; i < PF_POLL_LIMIT && !mbar_try(&drain_bar, 0); ++i) {}
            __syncwarp();
        }
        if (warp == 8) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(PW_TMEM_COLS) : "memory");
    }
}

template <int NMAT, int BITS, int DR>
int launch_prefill_wide_d(zc_moe* m, const Call& c, const __half* bsrc, const __half* bsum, size_t smem, uint32_t filter, cudaStream_t s) {
    auto kernel = prefill_wide_kernel<NMAT, BITS, DR>;
    static SmemOptIn configured;
    if (opt_in_smem(kernel, configured, m->device, smem) != cudaSuccess) return check_launch(m, "prefill kernel attribute");
    Timed t(m, s, NMAT == 2 ? KERNEL_PREFILL_GATE_UP : KERNEL_PREFILL_DOWN);
    const uint32_t row_tiles = NMAT == 2 ? c.F / 128 : c.H / 256;
    kernel<<<dim3(row_tiles, m->pf_max_tiles), PW_THREADS, smem, s>>>(c, static_cast<const PfTile*>(m->pf_tiles), m->pf_ntiles, bsrc, bsum, m->hbuf16, filter);
    return check_launch(m, NMAT == 2 ? "prefill gate_up" : "prefill down");
}

// Token-row prefetch depth: two stages ahead measured slightly faster than four (a shorter set-up per CTA: the first
// stages of a tile arrive at the SM's share of the memory bandwidth, about 25 bytes per clock).
template <int NMAT, int BITS>
int launch_prefill_wide(zc_moe* m, const Call& c, const __half* bsrc, const __half* bsum, uint32_t filter, cudaStream_t s) {
    const uint32_t K = NMAT == 2 ? c.H : c.F, G = pf_padded_groups(K);
    const size_t limit = 227 * 1024 - 2048;             // dynamic shared memory beside the kernel's static arrays
#ifndef ZC_PW_DR_GU
#define ZC_PW_DR_GU 2
#endif
#ifndef ZC_PW_DR_DN
#define ZC_PW_DR_DN 2
#endif
    if constexpr (BITS == 4 && (NMAT == 2 ? ZC_PW_DR_GU : ZC_PW_DR_DN) == 4) {
        if (PwSmem(G, 4, BITS).total <= limit) return launch_prefill_wide_d<NMAT, BITS, 4>(m, c, bsrc, bsum, PwSmem(G, 4, BITS).total, filter, s);
    }
    if (PwSmem(G, 2, BITS).total <= limit) return launch_prefill_wide_d<NMAT, BITS, 2>(m, c, bsrc, bsum, PwSmem(G, 2, BITS).total, filter, s);
    return fail(m, ZC_EINVAL, "prefill kernel: shape needs too much shared memory");
}

template <int NMAT, int BITS, bool META_F16, int D>
int launch_prefill_d(zc_moe* m, const Call& c, const __half* bsrc, const __half* bsum, size_t smem, uint32_t filter, cudaStream_t s) {
    const uint32_t N = NMAT == 2 ? c.F : c.H;
    auto kernel = prefill_kernel<NMAT, BITS, META_F16, D>;
    static SmemOptIn configured;
    if (opt_in_smem(kernel, configured, m->device, smem) != cudaSuccess) return check_launch(m, "prefill kernel attribute");
    Timed t(m, s, NMAT == 2 ? KERNEL_PREFILL_GATE_UP : KERNEL_PREFILL_DOWN);
    kernel<<<dim3(N / PF_M, m->pf_max_tiles), PF_THREADS, smem, s>>>(c, static_cast<const PfTile*>(m->pf_tiles), m->pf_ntiles, bsrc, bsum, m->hbuf16, filter);
    return check_launch(m, NMAT == 2 ? "prefill gate_up" : "prefill down");
}

template <int NMAT, int BITS, bool META_F16>
int launch_prefill(zc_moe* m, const Call& c, const __half* bsrc, const __half* bsum, uint32_t filter, cudaStream_t s) {
    using P = PfSmem<NMAT, BITS>;
    const uint32_t N = NMAT == 2 ? c.F : c.H, K = NMAT == 2 ? c.H : c.F, G = K / 64;
    if (N % PF_M) return fail(m, ZC_EINVAL, "prefill kernel: rows not a multiple of 128");
    if (G % 8) return fail(m, ZC_EINVAL, "prefill kernel: K must be a multiple of 512");
    const size_t limit = 227 * 1024;
    // down: its K is short (ten stages per CTA), so the fixed cost of a CTA matters: a shallower ring lets two CTAs
    // share an SM (shared memory and 256 TMEM columns each) and overlap one's set-up with the other's loop
    if (NMAT == 1 && 2 * (P::total(G, 2) + 1024) <= limit) return launch_prefill_d<NMAT, BITS, META_F16, 2>(m, c, bsrc, bsum, P::total(G, 2), filter, s);
    if (P::total(G, 4) <= limit) return launch_prefill_d<NMAT, BITS, META_F16, 4>(m, c, bsrc, bsum, P::total(G, 4), filter, s);
    if (P::total(G, 2) <= limit) return launch_prefill_d<NMAT, BITS, META_F16, 2>(m, c, bsrc, bsum, P::total(G, 2), filter, s);
    return fail(m, ZC_EINVAL, "prefill kernel: shape needs too much shared memory");
}

// The give-up path of the tensor-core kernels, run on its own: the roles of a CTA wait, with the kernels' own bounded
// waits, on an mbarrier that nothing ever arrives on. The suspending wait runs out after `polls` attempts (about a
// microsecond each), raises the abort flag and ZC_STATUS_TIMEOUT; the polling wait of the issuing role sees the flag (or
// runs out itself); then the CTA meets at its barrier and returns the tensor memory it had allocated, as the kernels do.
// report: {suspending wait returned, polling wait returned, abort flag, TMEM base} (a wait returns 0 when it gave up).
__global__ void __launch_bounds__(96) pf_wait_selftest_kernel(uint32_t polls, uint32_t* status, uint32_t* report) {
    __shared__ uint64_t never;
    __shared__ volatile uint32_t abort_flag;
    __shared__ uint32_t tmem_slot;
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) { mbar_init(&never, 1); abort_flag = 0; asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pf_smem(&tmem_slot)), "r"(32u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 1 && lane == 0) report[0] = mbar_wait(&never, 0, &abort_flag, status, polls) ? 1u : 0u;
    if (warp == 2 && lane == 0) report[1] = mbar_spin(&never, 0, &abort_flag, status, polls) ? 1u : 0u;
    __syncthreads();
    if (threadIdx.x == 0) { report[2] = abort_flag; report[3] = tmem_slot; }
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(32u) : "memory");
}

}  // namespace

int launch_wait_selftest(zc_moe* m, uint32_t polls, uint32_t* report, cudaStream_t s) {
    pf_wait_selftest_kernel<<<1, 96, 0, s>>>(polls, m->scratch.status, report);
    return check_launch(m, "wait self-test");
}

#ifdef ZC_PW_STAMPS
extern "C" int zc_dbg_prefill_stamps(void* host) { return cudaMemcpyFromSymbol(host, pw_stamps, sizeof(pw_stamps)) == cudaSuccess ? 0 : -1; }
#endif

size_t prefill_tile_capacity(const zc_moe_desc& d) {
    const size_t local = d.local_experts ? d.local_experts : d.experts;
    return local + (size_t(d.max_tokens) * d.top_k + d.max_tokens) / PF_NMAX + 2;
}
size_t prefill_tile_bytes() { return sizeof(PfTile); }

bool prefill_supported(const zc_moe_desc& d) {
    // BF16 activations convert to FP16 exactly; an FP32 activation would need a second FP16 term. Row tiles: 128 rows of
    // gate/up, 256 of down. (The per-group-drain kernel behind the prefill_wide = 0 option needs multiples of 512.)
    return d.arith == ZC_ARITH_FP32 && d.act_dtype == ZC_BF16 && d.ffn % 128 == 0 && d.hidden % 256 == 0 && d.hidden <= 4096;
}
size_t prefill_sum_halves(uint32_t K) { return size_t(4) * pf_padded_groups(K); }

// tile list -> FP16 activations -> gate/up (+SwiGLU) -> down. Routing must already be in place.
int launch_experts_prefill(zc_moe* m, const Call& c, cudaStream_t s, uint32_t skip_rows_upto) {
    int rc;
    const bool wide = m->prefill_wide;
    {
        Timed t(m, s, KERNEL_PREFILL_PREP);
        pf_tiles_kernel<<<1, 1024, 0, s>>>(c.offsets, c.E, c.first_expert, c.local_experts, c.T, c.has_shared, wide ? PW_NMAX : PF_NMAX, skip_rows_upto,
                                           static_cast<PfTile*>(m->pf_tiles), m->pf_ntiles);
        if ((rc = check_launch(m, "prefill tiles")) < 0) return rc;
    }
    {
        Timed t(m, s, KERNEL_PREFILL_PREP);
        pf_prepare_x_sums_kernel<<<(c.T * 32 + 255) / 256, 256, 0, s>>>(c.x, c.act_dtype, m->xp, c.T, c.H, m->xsum, c.status);
        if ((rc = check_launch(m, "prefill activations and sums")) < 0) return rc;
    }
    // The code width is a template parameter: a shared expert with other bit widths than the routed experts' takes the
    // shared tiles in launches of its own (filter 2) while the routed launch skips them (filter 1).
    auto gemm = [&](auto nmat_tag, const Call& q, uint32_t bits, const __half* bsrc, const __half* bsum, uint32_t filter) {
        constexpr int NM = decltype(nmat_tag)::value;
        if (wide) return bits == 4 ? launch_prefill_wide<NM, 4>(m, q, bsrc, bsum, filter, s) : launch_prefill_wide<NM, 8>(m, q, bsrc, bsum, filter, s);
        if (bits == 4) return q.meta_f16 ? launch_prefill<NM, 4, true>(m, q, bsrc, bsum, filter, s) : launch_prefill<NM, 4, false>(m, q, bsrc, bsum, filter, s);
        return q.meta_f16 ? launch_prefill<NM, 8, true>(m, q, bsrc, bsum, filter, s) : launch_prefill<NM, 8, false>(m, q, bsrc, bsum, filter, s);
    };
    const bool split = c.has_shared && c.shared_split;
    Call shared = c;
    shared.gate = c.sgate; shared.up = c.sup; shared.down = c.sdown;
    int extra = 0;
    rc = gemm(std::integral_constant<int, 2>{}, c, c.gate.bits, m->xp, m->xsum, split ? 1u : 0u);
    if (rc >= 0 && split) { rc = gemm(std::integral_constant<int, 2>{}, shared, shared.gate.bits, m->xp, m->xsum, 2u); ++extra; }
    if (rc < 0) return rc;
    {
        Timed t(m, s, KERNEL_PREFILL_PREP);
        const uint32_t rows = c.T * c.K + c.T;
        pf_sums_kernel<<<(rows * 32 + 255) / 256, 256, 0, s>>>(m->hbuf16, rows, c.F, m->hsum, c.status);
        if ((rc = check_launch(m, "prefill intermediate sums")) < 0) return rc;
    }
    rc = gemm(std::integral_constant<int, 1>{}, c, c.down.bits, m->hbuf16, m->hsum, split ? 1u : 0u);
    if (rc >= 0 && split) { rc = gemm(std::integral_constant<int, 1>{}, shared, shared.down.bits, m->hbuf16, m->hsum, 2u); ++extra; }
    if (rc < 0) return rc;
    return 5 + extra;
}

}  // namespace zc
