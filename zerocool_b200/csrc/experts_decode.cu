// Decode family: the routed and shared experts for short token batches.
//
// Replaces, for every expert that received work, the reference's per-expert launches
//   gated_linear -> q4_gate_mv_r2 / q4_gate_up (kernels/metal/qwen.metal:333-376, 71-81)
//   linear_into  -> q4_mv_r* / q4_mm           (qwen.metal:289-330, 63-70), scatter_experts :800-803
// issued by encode_expert_rows (src/engine/pipeline.cpp:7-31), and the shared expert of
// Model::moe (src/engine/model.cpp:482-484), with two grouped launches per layer:
//   gate_up_kernel: h[row, f]  = silu(gate_e . x_row) * (up_e . x_row)       for every (expert, row)
//   down_kernel:    y[slot, c] = down_e . h_row, written at the slot's router position
//
// Both stream each selected record exactly once per eight rows. The limiting resource at B200 rates
// is instruction issue, not arithmetic: 4-bit codes arrive at ~13 T weights/s, which leaves about
// three issue slots per weight per SM. So the multiply-accumulates run on the tensor cores as
// m16n8k16 BF16 MMAs with up to eight token rows in the N dimension: the integer codes 0..15 (or the
// 8-bit codes) are exact in BF16, a BF16 activation is used as it is (an FP32 activation is split into
// two BF16 terms), products are accumulated in FP32 per 64-wide quantisation group, and the group's
// scale and bias are applied to the FP32 accumulator in registers:
//     acc += scale[row, g] * sum_k(q * x) + bias[row, g] * sum_k(x)
// which is the reference's affine_dot form (qwen.metal:46-62) with an exact inner sum.
//
// Weight traffic: lane (g = lane/4, c = lane%4) of a warp loads 8 bytes (Q4) or 16 bytes (Q8) of rows
// g and g+8 for group `grp` — the 16 k values [16c, 16c+16) of that group — so the four lanes of a row
// stay inside one quantisation group, each 32-byte sector is fetched once, and loads for the next
// chunk of groups are issued before the current chunk is multiplied. Because a dot product does not
// care about the order of k, the MMA's k slots are bound to whatever k values fall out of the cheapest
// nibble extraction; the activations are staged in shared memory in the matching order.
#include "common.cuh"

namespace zc {
namespace {

constexpr int NTOK = 8;             // token rows per MMA pass (the N of m16n8k16)
constexpr int EXPERT_THREADS = 128; // 4 warps
constexpr int ROW_PAD = 8;          // bf16 elements added to each staged row (keeps 16-byte reads conflict free)

template <int BITS> struct Fmt;
template <> struct Fmt<4> { static constexpr int CH = 4, WORDS = 2; };   // groups per chunk, 32-bit words per row per group
template <> struct Fmt<8> { static constexpr int CH = 2, WORDS = 4; };

struct ItemInfo {
    const uint8_t* record;
    uint32_t count;     // rows of this item
    uint32_t pos0;      // routed: first position in perm; shared: 0
    uint32_t hrow0;     // first row in hbuf
    bool shared;
};

__device__ __forceinline__ bool decode_item(const Call& c, uint32_t item, ItemInfo& it) {
    if (c.has_shared) {
        if (item == 0) {
            it.record = c.shared_record; it.count = c.T; it.pos0 = 0; it.hrow0 = c.T * c.K; it.shared = true;
            return true;
        }
        --item;
    }
    if (item >= uint32_t(c.counters[0])) return false;
    const uint32_t e = uint32_t(c.active[item]);
    it.record = c.records + size_t(e - c.first_expert) * c.record_stride;
    it.pos0 = uint32_t(c.offsets[e]);
    it.count = uint32_t(c.offsets[e + 1]) - it.pos0;
    it.hrow0 = it.pos0;
    it.shared = false;
    return true;
}

// Stage up to NTOK source rows of K elements into shared memory as BF16 (hi, and lo when SPLIT), in
// the k order the MMA fragments expect, and the per-group input sums Sx[grp][n].
//   Q4 order inside each block of 8: (0,4,1,5,2,6,3,7); Q8 order: natural.
//   REF: Sx is the reference's BF16-rounded sum of four (qwen.metal:55); otherwise plain fp32.
template <bool Q4ORDER, bool SPLIT>
__device__ __forceinline__ void stage_rows(const void* src, bool src_f32, const int* rows /*[NTOK], -1 = none*/,
                                           uint32_t K, bool ref, uint16_t* hi, uint16_t* lo, float* Sx) {
    const uint32_t RS = K + ROW_PAD, blocks = K / 8;
    for (uint32_t idx = threadIdx.x; idx < NTOK * blocks; idx += EXPERT_THREADS) {
        const uint32_t n = idx / blocks, q = idx % blocks;
        const int row = rows[n];
        float v[8];
        if (row < 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        } else if (src_f32) {
            const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(src) + size_t(row) * K + q * 8);
            const float4 a = p[0], b = p[1];
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
            const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(src) + size_t(row) * K + q * 8);
            const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(r[i] << 16); v[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u); }
        }
        float sum;
        if (ref) sum = bf_round(bf_round(bf_round(v[0] + v[1]) + v[2]) + v[3]) + bf_round(bf_round(bf_round(v[4] + v[5]) + v[6]) + v[7]);
        else sum = (((v[0] + v[1]) + v[2]) + v[3]) + (((v[4] + v[5]) + v[6]) + v[7]);
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if ((q & 7) == 0) Sx[(q / 8) * NTOK + n] = sum;
        uint16_t h[8], l[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            h[i] = bf_bits(v[i]);
            if (SPLIT) l[i] = bf_bits(v[i] - bf_to_float(h[i]));
        }
        constexpr int order_q4[8] = {0, 4, 1, 5, 2, 6, 3, 7};
        uint32_t ph[4], pl[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int a = Q4ORDER ? order_q4[2 * i] : 2 * i, b = Q4ORDER ? order_q4[2 * i + 1] : 2 * i + 1;
            ph[i] = uint32_t(h[a]) | (uint32_t(h[b]) << 16);
            if (SPLIT) pl[i] = uint32_t(l[a]) | (uint32_t(l[b]) << 16);
        }
        *reinterpret_cast<uint4*>(hi + n * RS + q * 8) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
        if (SPLIT) *reinterpret_cast<uint4*>(lo + n * RS + q * 8) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
    }
}

// One chunk (CH groups) of one matrix for the lane's two rows (g and g+8): codes and metadata.
template <int BITS>
struct Chunk {
    uint32_t w[2][Fmt<BITS>::CH][Fmt<BITS>::WORDS];
    uint16_t s[2][Fmt<BITS>::CH], b[2][Fmt<BITS>::CH];
};

template <int BITS>
__device__ __forceinline__ void load_chunk(Chunk<BITS>& ch, const uint8_t* codes, const uint16_t* scales, const uint16_t* biases,
                                           uint32_t row0, uint32_t K, uint32_t G, uint32_t grp0, uint32_t valid, uint32_t cq) {
    constexpr int CH = Fmt<BITS>::CH;
    const uint32_t row_bytes = K * BITS / 8;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t row = row0 + 8 * r;
        const uint8_t* crow = codes + size_t(row) * row_bytes;
        const uint16_t* srow = scales + size_t(row) * G;
        const uint16_t* brow = biases + size_t(row) * G;
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            if (uint32_t(j) < valid) {
                const uint32_t grp = grp0 + j;
                if constexpr (BITS == 4) {
                    const uint2 v = ldg_nc_u2(crow + grp * 32 + cq * 8);
                    ch.w[r][j][0] = v.x; ch.w[r][j][1] = v.y;
                } else {
                    const uint4 v = ldg_nc_u4(crow + grp * 64 + cq * 16);
                    ch.w[r][j][0] = v.x; ch.w[r][j][1] = v.y; ch.w[r][j][2] = v.z; ch.w[r][j][3] = v.w;
                }
                ch.s[r][j] = __ldg(srow + grp);
                ch.b[r][j] = __ldg(brow + grp);
            }
        }
    }
}

// d(16 rows x 8 tokens) = sum over one 64-wide group of code * x, for the lane's two rows.
template <int BITS, bool SPLIT>
__device__ __forceinline__ void group_mma(float (&d)[4], const uint32_t (&w0)[Fmt<BITS>::WORDS], const uint32_t (&w1)[Fmt<BITS>::WORDS],
                                          const uint4 (&bh)[2], const uint4 (&bl)[2], bool q8_signed) {
    if constexpr (BITS == 4) {
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            uint32_t p0[4], p1[4];
            dequant_q4_word(w0[m], p0);
            dequant_q4_word(w1[m], p1);
            mma_bf16_16816(d, p0[0], p1[0], p0[1], p1[1], bh[m].x, bh[m].y);
            mma_bf16_16816(d, p0[2], p1[2], p0[3], p1[3], bh[m].z, bh[m].w);
            if constexpr (SPLIT) {
                mma_bf16_16816(d, p0[0], p1[0], p0[1], p1[1], bl[m].x, bl[m].y);
                mma_bf16_16816(d, p0[2], p1[2], p0[3], p1[3], bl[m].z, bl[m].w);
            }
        }
    } else {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            uint32_t p0[2], p1[2];
            dequant_q8_word(w0[m], q8_signed, p0);
            dequant_q8_word(w1[m], q8_signed, p1);
            const uint32_t b0 = (m & 1) ? bh[m / 2].z : bh[m / 2].x, b1 = (m & 1) ? bh[m / 2].w : bh[m / 2].y;
            mma_bf16_16816(d, p0[0], p1[0], p0[1], p1[1], b0, b1);
            if constexpr (SPLIT) {
                const uint32_t c0 = (m & 1) ? bl[m / 2].z : bl[m / 2].x, c1 = (m & 1) ? bl[m / 2].w : bl[m / 2].y;
                mma_bf16_16816(d, p0[0], p1[0], p0[1], p1[1], c0, c1);
            }
        }
    }
}

// acc += scale * d + bias * Sx for one group of one chunk.
template <int BITS, bool SPLIT>
__device__ __forceinline__ void consume_group(float (&acc)[4], const Chunk<BITS>& ch, int j, const uint4 (&bh)[2], const uint4 (&bl)[2],
                                              float2 sx, bool meta_f16, bool q8_signed) {
    float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    group_mma<BITS, SPLIT>(d, ch.w[0][j], ch.w[1][j], bh, bl, q8_signed);
    const float s0 = meta_to_float(ch.s[0][j], meta_f16), s1 = meta_to_float(ch.s[1][j], meta_f16);
    const float b0 = meta_to_float(ch.b[0][j], meta_f16), b1 = meta_to_float(ch.b[1][j], meta_f16);
    acc[0] += __fmaf_rn(s0, d[0], b0 * sx.x);
    acc[1] += __fmaf_rn(s0, d[1], b0 * sx.y);
    acc[2] += __fmaf_rn(s1, d[2], b1 * sx.x);
    acc[3] += __fmaf_rn(s1, d[3], b1 * sx.y);
}

__device__ __forceinline__ void load_b(const uint16_t* rowbase, uint32_t grp, uint32_t cq, uint4 (&b)[2]) {
    const uint16_t* p = rowbase + grp * 64 + cq * 16;
    b[0] = *reinterpret_cast<const uint4*>(p);
    b[1] = *reinterpret_cast<const uint4*>(p + 8);
}

// ---------------------------------------------------------------------------------------------
// gate/up + SwiGLU. Grid: (F/16, items). A CTA computes 16 rows of gate and the same 16 rows of up
// for all rows of its item; its four warps split K in chunks and add their partials in warp order.
// ---------------------------------------------------------------------------------------------
template <int BITS, bool SPLIT>
__global__ void __launch_bounds__(EXPERT_THREADS) gate_up_kernel(Call c) {
    constexpr int CH = Fmt<BITS>::CH;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    ItemInfo it;
    if (!decode_item(c, blockIdx.y, it)) return;
    const uint32_t K = c.H, G = K / 64, RS = K + ROW_PAD;
    uint16_t* xhi = reinterpret_cast<uint16_t*>(smem_raw);
    uint16_t* xlo = xhi + (SPLIT ? NTOK * RS : 0);
    float* Sx = reinterpret_cast<float*>(xhi + (SPLIT ? 2 : 1) * NTOK * RS);
    float* red = Sx + G * NTOK;                       // [4][2][16][NTOK]
    __shared__ int rows[NTOK];

    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane / 4, cq = lane % 4;
    const uint32_t r0 = blockIdx.x * 16;
    const uint8_t* gc = it.record + c.gate.codes; const uint8_t* uc = it.record + c.up.codes;
    const uint16_t* gs = reinterpret_cast<const uint16_t*>(it.record + c.gate.scales);
    const uint16_t* gb = reinterpret_cast<const uint16_t*>(it.record + c.gate.biases);
    const uint16_t* us = reinterpret_cast<const uint16_t*>(it.record + c.up.scales);
    const uint16_t* ub = reinterpret_cast<const uint16_t*>(it.record + c.up.biases);
    const uint32_t nchunks = (G + CH - 1) / CH;
    const bool meta_f16 = c.meta_f16, q8s = c.q8_signed;

    for (uint32_t pass = 0; pass * NTOK < it.count; ++pass) {
        __syncthreads();
        if (threadIdx.x < NTOK) {
            const uint32_t i = pass * NTOK + threadIdx.x;
            rows[threadIdx.x] = i < it.count ? (it.shared ? int(i) : c.perm[it.pos0 + i] / int(c.K)) : -1;
        }
        __syncthreads();
        stage_rows<BITS == 4, SPLIT>(c.x, c.act_dtype == ZC_F32, rows, K, c.ref && BITS == 4, xhi, xlo, Sx);
        __syncthreads();

        float accg[4] = {0, 0, 0, 0}, accu[4] = {0, 0, 0, 0};
        Chunk<BITS> cg[2], cu[2];
        uint32_t chunk = warp;
        if (chunk < nchunks) {
            const uint32_t grp0 = chunk * CH, valid = min(uint32_t(CH), G - grp0);
            load_chunk<BITS>(cg[0], gc, gs, gb, r0 + g, K, G, grp0, valid, cq);
            load_chunk<BITS>(cu[0], uc, us, ub, r0 + g, K, G, grp0, valid, cq);
        }
        int cur = 0;
        for (; chunk < nchunks; chunk += 4, cur ^= 1) {
            const uint32_t next = chunk + 4;
            if (next < nchunks) {
                const uint32_t grp0 = next * CH, valid = min(uint32_t(CH), G - grp0);
                if (cur == 0) { load_chunk<BITS>(cg[1], gc, gs, gb, r0 + g, K, G, grp0, valid, cq); load_chunk<BITS>(cu[1], uc, us, ub, r0 + g, K, G, grp0, valid, cq); }
                else          { load_chunk<BITS>(cg[0], gc, gs, gb, r0 + g, K, G, grp0, valid, cq); load_chunk<BITS>(cu[0], uc, us, ub, r0 + g, K, G, grp0, valid, cq); }
            }
            const uint32_t grp0 = chunk * CH, valid = min(uint32_t(CH), G - grp0);
#pragma unroll
            for (int j = 0; j < CH; ++j) {
                if (uint32_t(j) < valid) {
                    const uint32_t grp = grp0 + j;
                    uint4 bh[2], bl[2];
                    load_b(xhi + g * RS, grp, cq, bh);
                    if constexpr (SPLIT) load_b(xlo + g * RS, grp, cq, bl);
                    const float2 sx = *reinterpret_cast<const float2*>(Sx + grp * NTOK + 2 * cq);
                    if (cur == 0) { consume_group<BITS, SPLIT>(accg, cg[0], j, bh, bl, sx, meta_f16, q8s); consume_group<BITS, SPLIT>(accu, cu[0], j, bh, bl, sx, meta_f16, q8s); }
                    else          { consume_group<BITS, SPLIT>(accg, cg[1], j, bh, bl, sx, meta_f16, q8s); consume_group<BITS, SPLIT>(accu, cu[1], j, bh, bl, sx, meta_f16, q8s); }
                }
            }
        }
        // partials of this warp: [warp][matrix][row][token]
        float* mine = red + warp * 2 * 16 * NTOK;
        *reinterpret_cast<float2*>(mine + (0 * 16 + g) * NTOK + 2 * cq) = make_float2(accg[0], accg[1]);
        *reinterpret_cast<float2*>(mine + (0 * 16 + g + 8) * NTOK + 2 * cq) = make_float2(accg[2], accg[3]);
        *reinterpret_cast<float2*>(mine + (1 * 16 + g) * NTOK + 2 * cq) = make_float2(accu[0], accu[1]);
        *reinterpret_cast<float2*>(mine + (1 * 16 + g + 8) * NTOK + 2 * cq) = make_float2(accu[2], accu[3]);
        __syncthreads();
        {
            const uint32_t row = threadIdx.x / NTOK, n = threadIdx.x % NTOK;
            float gate = 0.0f, up = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                gate += red[((w * 2 + 0) * 16 + row) * NTOK + n];
                up += red[((w * 2 + 1) * 16 + row) * NTOK + n];
            }
            float h;
            if (c.ref) {   // qwen.metal:71-81
                gate = bf_round(gate); up = bf_round(up);
                h = bf_round(bf_round(gate * sigmoid_bf(gate)) * up);
            } else {
                h = (gate * sigmoid_f(gate)) * up;
            }
            const uint32_t i = pass * NTOK + n;
            if (i < it.count) c.hbuf[size_t(it.hrow0 + i) * c.F + r0 + row] = h;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// down projection. Grid: (H/64, items). Each warp owns 16 output rows over the whole K = F and
// writes its results straight to the slot's router position (the reference's linear_into /
// scatter_experts destination, pipeline.cpp:25-28).
// ---------------------------------------------------------------------------------------------
template <int BITS, bool SPLIT>
__global__ void __launch_bounds__(EXPERT_THREADS) down_kernel(Call c) {
    constexpr int CH = Fmt<BITS>::CH;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    ItemInfo it;
    if (!decode_item(c, blockIdx.y, it)) return;
    const uint32_t K = c.F, G = K / 64, RS = K + ROW_PAD;
    uint16_t* hhi = reinterpret_cast<uint16_t*>(smem_raw);
    uint16_t* hlo = hhi + (SPLIT ? NTOK * RS : 0);
    float* Sx = reinterpret_cast<float*>(hhi + (SPLIT ? 2 : 1) * NTOK * RS);
    __shared__ int rows[NTOK];
    __shared__ long long dest[NTOK];      // element offset of the destination row, or -1

    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane / 4, cq = lane % 4;
    const uint32_t r0 = blockIdx.x * 64 + warp * 16;
    const uint8_t* dc = it.record + c.down.codes;
    const uint16_t* ds = reinterpret_cast<const uint16_t*>(it.record + c.down.scales);
    const uint16_t* db = reinterpret_cast<const uint16_t*>(it.record + c.down.biases);
    const uint32_t nchunks = (G + CH - 1) / CH;
    const bool meta_f16 = c.meta_f16, q8s = c.q8_signed;
    float* out_base = it.shared ? c.shared_out : c.expert_out;

    for (uint32_t pass = 0; pass * NTOK < it.count; ++pass) {
        __syncthreads();
        if (threadIdx.x < NTOK) {
            const uint32_t i = pass * NTOK + threadIdx.x;
            if (i < it.count) {
                rows[threadIdx.x] = int(it.hrow0 + i);
                const uint32_t slot = it.shared ? i : uint32_t(c.perm[it.pos0 + i]);
                dest[threadIdx.x] = (long long)slot * c.H;
            } else { rows[threadIdx.x] = -1; dest[threadIdx.x] = -1; }
        }
        __syncthreads();
        stage_rows<BITS == 4, SPLIT>(c.hbuf, true, rows, K, c.ref && BITS == 4, hhi, hlo, Sx);
        __syncthreads();

        float acc[4] = {0, 0, 0, 0};
        Chunk<BITS> cd[2];
        {
            const uint32_t valid = min(uint32_t(CH), G);
            load_chunk<BITS>(cd[0], dc, ds, db, r0 + g, K, G, 0, valid, cq);
        }
        int cur = 0;
        for (uint32_t chunk = 0; chunk < nchunks; ++chunk, cur ^= 1) {
            const uint32_t next = chunk + 1;
            if (next < nchunks) {
                const uint32_t grp0 = next * CH, valid = min(uint32_t(CH), G - grp0);
                if (cur == 0) load_chunk<BITS>(cd[1], dc, ds, db, r0 + g, K, G, grp0, valid, cq);
                else          load_chunk<BITS>(cd[0], dc, ds, db, r0 + g, K, G, grp0, valid, cq);
            }
            const uint32_t grp0 = chunk * CH, valid = min(uint32_t(CH), G - grp0);
#pragma unroll
            for (int j = 0; j < CH; ++j) {
                if (uint32_t(j) < valid) {
                    const uint32_t grp = grp0 + j;
                    uint4 bh[2], bl[2];
                    load_b(hhi + g * RS, grp, cq, bh);
                    if constexpr (SPLIT) load_b(hlo + g * RS, grp, cq, bl);
                    const float2 sx = *reinterpret_cast<const float2*>(Sx + grp * NTOK + 2 * cq);
                    if (cur == 0) consume_group<BITS, SPLIT>(acc, cd[0], j, bh, bl, sx, meta_f16, q8s);
                    else          consume_group<BITS, SPLIT>(acc, cd[1], j, bh, bl, sx, meta_f16, q8s);
                }
            }
        }
        // lane holds rows g, g+8 for tokens 2cq, 2cq+1
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t n = 2 * cq + (i & 1), row = r0 + g + 8 * (i >> 1);
            const long long d = dest[n];
            if (d >= 0) out_base[d + row] = c.ref ? bf_round(acc[i]) : acc[i];
        }
    }
}

template <void (*kernel)(Call)>
int launch_one(zc_moe* m, dim3 grid, size_t smem, const Call& c, cudaStream_t s, const char* what, int kind) {
    if (smem > 200 * 1024) return fail(m, ZC_EINVAL, std::string(what) + ": shape needs too much shared memory");
    static bool configured = false;   // one flag per kernel instantiation
    if (!configured) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        configured = true;
    }
    Timed t(m, s, kind);
    kernel<<<grid, EXPERT_THREADS, smem, s>>>(c);
    return check_launch(m, what);
}

}  // namespace

int launch_experts_decode(zc_moe* m, const Call& c, cudaStream_t s) {
    const uint32_t routed = c.T * c.K < c.local_experts ? c.T * c.K : c.local_experts;
    const uint32_t items = routed + (c.has_shared ? 1 : 0);
    // A BF16 activation is exact as one BF16 term; an FP32 activation needs two, except under the
    // reference arithmetic, whose FP32 buffers hold BF16 values by contract.
    const bool split_x = c.act_dtype == ZC_F32 && !c.ref;
    const bool split_h = !c.ref;      // h is FP32 unless the reference rounds it to BF16
    {
        const uint32_t K = c.H, G = K / 64;
        const size_t smem = size_t(split_x ? 2 : 1) * NTOK * (K + ROW_PAD) * 2 + size_t(G) * NTOK * 4 + 4 * 2 * 16 * NTOK * 4;
        const dim3 grid(c.F / 16, items);
        int rc;
        if (c.gate.bits == 4) rc = split_x ? launch_one<gate_up_kernel<4, true>>(m, grid, smem, c, s, "gate_up", KERNEL_GATE_UP) : launch_one<gate_up_kernel<4, false>>(m, grid, smem, c, s, "gate_up", KERNEL_GATE_UP);
        else rc = split_x ? launch_one<gate_up_kernel<8, true>>(m, grid, smem, c, s, "gate_up", KERNEL_GATE_UP) : launch_one<gate_up_kernel<8, false>>(m, grid, smem, c, s, "gate_up", KERNEL_GATE_UP);
        if (rc < 0) return rc;
    }
    {
        const uint32_t K = c.F, G = K / 64;
        const size_t smem = size_t(split_h ? 2 : 1) * NTOK * (K + ROW_PAD) * 2 + size_t(G) * NTOK * 4;
        const dim3 grid(c.H / 64, items);
        int rc;
        if (c.down.bits == 4) rc = split_h ? launch_one<down_kernel<4, true>>(m, grid, smem, c, s, "down", KERNEL_DOWN) : launch_one<down_kernel<4, false>>(m, grid, smem, c, s, "down", KERNEL_DOWN);
        else rc = split_h ? launch_one<down_kernel<8, true>>(m, grid, smem, c, s, "down", KERNEL_DOWN) : launch_one<down_kernel<8, false>>(m, grid, smem, c, s, "down", KERNEL_DOWN);
        if (rc < 0) return rc;
    }
    return 2;
}

}  // namespace zc
