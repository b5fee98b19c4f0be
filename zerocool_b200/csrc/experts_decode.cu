// Decode family: the routed and shared experts for short token batches.
//
// Replaces, for every expert that received work, the reference's per-expert launches
//   gated_linear -> q4_gate_mv_r2 / q4_gate_up (kernels/metal/qwen.metal:333-376, 71-81)
//   linear_into  -> q4_mv_r* / q4_mm           (qwen.metal:289-330, 63-70), scatter_experts :800-803
// issued by encode_expert_rows (src/engine/pipeline.cpp:7-31), and the shared expert of
// Model::moe (src/engine/model.cpp:482-484), with two grouped launches per layer of one kernel
// template:
//   NMAT = 2 (gate/up): h[row, f]  = silu(gate_e . x_row) * (up_e . x_row)    for every (expert, row)
//   NMAT = 1 (down):    y[slot, c] = down_e . h_row, written at the slot's router position
//
// Each launch streams every selected record once per eight rows. At B200 rates the limiting resource
// is instruction issue, not arithmetic: 4-bit codes arrive at ~13 T weights/s, about three issue slots
// per weight per SM. So:
//  * The multiply-accumulates run on the tensor cores as m16n8k16 FP16 MMAs with up to eight token
//    rows in the N dimension. Integer codes are exact in FP16, a BF16 activation converts exactly, an
//    FP32 activation is split into two FP16 terms, and products are accumulated in FP32 per 64-wide
//    quantisation group. The group's scale and bias are applied to that FP32 accumulator:
//        acc += scale[row, g] * sum_k(q * x) + bias[row, g] * sum_k(x)
//    which is the reference's affine_dot form (qwen.metal:46-62) with an exact inner sum.
//  * Q4 codes become FP16 with one logic operation per two weights: (w & 0x000f000f) | 0x6400 is the
//    half2 (1024+q_lo, 1024+q_hi), and (w & 0x00f000f0) | 0x6400 is (1024+16 q, 1024+16 q). With FOLD
//    those values go into the MMA as they are: the activations that meet a "q" slot are staged multiplied by 16
//    (exact; the finished sum is divided by 16), and the 1024 offset is removed from the FP32 group sum as
//    1024 * sum(x as staged).
//    Without FOLD the offset and the factor 16 are removed in FP16 before the MMA (exact, 4 more ops per
//    word).
//  * Weights reach the warp through a private cp.async ring in shared memory (no registers held
//    across the latency, no block-wide barrier). A stage holds CH quantisation groups of a 16-row tile:
//    each row's CH * 32 (Q4) or CH * 64 (Q8) contiguous code bytes are fetched as 16-byte pieces by
//    adjacent lanes, so every sector of a record is requested once; the 32/64-byte blocks of a row are
//    XOR-swizzled by the row index so that the fragment reads stay bank-conflict free. The refill of a
//    slot is issued before the chunk that was waited for is multiplied, so STAGES-1 chunks are in
//    flight while the warp computes.
//  * Lanes whose token row is absent (fewer than eight rows in the pass) skip the activation reads.
//  * Because a dot product does not care about the order of k, the MMA's k slots are bound to whatever
//    k values fall out of the cheapest extraction; the activations are staged in the matching order.
// Activations must stay inside FP16 after the factor 16 (|x| < 4094 for Q4 projections, < 65504 for Q8); hidden
// states after a norm are O(1..100). A value beyond that raises ZC_STATUS_RANGE in the status word (the output of
// that row is then not meaningful); the same holds for the SwiGLU rows the down projection reads.
#include "common.cuh"

namespace zc {
namespace {

constexpr int NTOK = 8;               // token rows per MMA pass (the N of m16n8k16)
constexpr int WARPS = 8;
constexpr int EXPERT_THREADS = WARPS * 32;
constexpr int ROW_PAD = 8;            // halves added to each staged row (keeps 16-byte reads conflict free)
#ifndef ZC_MIN_BLOCKS
#define ZC_MIN_BLOCKS 2
#endif
#ifndef ZC_MIN_BLOCKS_DOWN
#define ZC_MIN_BLOCKS_DOWN 3
#endif

// One ring stage of one matrix holds CHT quantisation groups of 16 rows: for every row one LINE of CHT x ROWB
// contiguous code bytes (a full 128-byte line for Q4 with four groups and for Q8 with two).
template <int BITS, int CHT> struct Fmt {
    static constexpr int ROWB = BITS * 8;                 // code bytes of one row of one group (64 weights)
    static constexpr int LINE = CHT * ROWB;               // code bytes of one row in one stage
    static constexpr int PIECES = LINE / 16;              // 16-byte pieces (= lanes) per row
    static constexpr int ROWS_PER_PASS = 32 / PIECES;
    static constexpr int PASSES = 16 / ROWS_PER_PASS;
    static constexpr int CODES = 16 * LINE;
    static constexpr int MATRIX = CODES;                  // a ring stage holds the codes only
    // Metadata of a matrix, beside the ring: [buffer][row][scale, bias][MG halves]. MG = 8 groups per block (one 16-byte
    // copy per (row, kind), two buffers) where a warp walks K in order, else MG = CHT (one block per ring stage).
    __host__ __device__ static constexpr int meta_area(int mbg, int stages) { return mbg ? 2 * 32 * mbg * 2 : stages * 32 * CHT * 2; }     // bytes per matrix per warp (mbg: groups per block, 0 = per stage)
    // Rows whose lines fall into the same 128-byte bank window are ROWS_PER_WINDOW apart; the block index of a row is
    // xor-ed with swizzle(row) so that rows read together by one MMA fragment load use different banks.
    static constexpr int ROWS_PER_WINDOW = LINE >= 128 ? 1 : 128 / LINE;
    __host__ __device__ static constexpr uint32_t swizzle(uint32_t row) { return (row / ROWS_PER_WINDOW) & (CHT - 1); }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// D(16x8, fp32) += A(16x16, fp16, row) * B(16x8, fp16, col). Lane (g = lane/4, c = lane%4) holds
//   a0: A[g][2c,2c+1]   a1: A[g+8][2c,2c+1]   a2: A[g][2c+8,2c+9]   a3: A[g+8][2c+8,2c+9]
//   b0: B[2c,2c+1][g]   b1: B[2c+8,2c+9][g]
//   d0,d1: D[g][2c,2c+1]   d2,d3: D[g+8][2c,2c+1]
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Same product with the addend taken from c (the first MMA of a group starts from the folded offset).
__device__ __forceinline__ void mma_f16_16816_c(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1,
                                                float c0, float c1, float c2, float c3) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}

// Ring depth per warp: two stages of four groups or three of two keep the same bytes in flight.
__host__ __device__ constexpr int stages_for(int matrices_per_warp, int ch) { return (ch == 4 && matrices_per_warp == 2) ? 2 : 3; }

struct ItemInfo {
    const uint8_t* record;
    uint32_t count;     // rows of this item
    uint32_t pos0;      // routed: first position in perm; shared: first token of this block of rows
    uint32_t hrow0;     // first row in hbuf
    bool shared;
};

// Items of a launch: the shared expert contributes one item per NTOK tokens (so that its row blocks run
// in parallel instead of as passes of one CTA), then one item per routed expert that received work.
__device__ __forceinline__ bool decode_item(const Call& c, uint32_t item, ItemInfo& it) {
    if (c.has_shared) {
        const uint32_t blocks = (c.T + NTOK - 1) / NTOK;
        if (item < blocks) {
            it.record = c.shared_record; it.pos0 = item * NTOK; it.count = min(uint32_t(NTOK), c.T - it.pos0);
            it.hrow0 = c.T * c.K + it.pos0; it.shared = true;
            return true;
        }
        item -= blocks;
    }
    const int4 entry = __ldcg(c.items + item);            // one load: {expert, first position, rows}; x = -1 past the list's end
    if (entry.x < 0) return false;
    if (c.item_rows_max && uint32_t(entry.z) > c.item_rows_max) return false;      // this expert's rows go to the tensor-core family
    const uint32_t e = uint32_t(entry.x);
    it.record = c.records + size_t(e - c.first_expert) * c.record_stride;
    it.pos0 = uint32_t(entry.y);
    it.count = uint32_t(entry.z);
    it.hrow0 = it.pos0;
    it.shared = false;
    return true;
}

// Stage the valid source rows (n < nvalid) of K elements into shared memory as FP16 (hi, and lo when
// SPLIT), in the k order the MMA fragments expect, with the per-group sums
//   sums[grp][n] = (Sx, P):  Sx = sum of x over the group (REF: the reference's BF16 sum of four,
//   qwen.metal:55), P = -1024 * sum of the values as staged: the MMA accumulator starts from P, which
//   removes the folded 1024 offset of the codes (0 without FOLD).
//   Q4 order inside each block of 8: (0,4,1,5,2,6,3,7), even k staged x 16 when FOLD; Q8: natural order.
// Rows n >= nvalid are left as they are: an MMA column only depends on its own B column.
template <bool Q4ORDER, bool SPLIT, bool FOLD>
__device__ __forceinline__ void stage_rows(const void* src, bool src_f32, const int* rows, uint32_t nvalid,
                                           uint32_t K, bool ref, __half* hi, __half* lo, float* sums, uint32_t* status) {
    const uint32_t RS = K + ROW_PAD, blocks = K / 8, total = nvalid * blocks;
    bool out_of_range = false;
    // The trip count is uniform per warp (the shuffles below need all 32 lanes); lanes past the end carry zeros.
    for (uint32_t idx = threadIdx.x; (idx & ~31u) < total; idx += EXPERT_THREADS) {
        const bool live = idx < total;
        const uint32_t n = live ? idx / blocks : 0, q = live ? idx % blocks : 0;
        const int row = rows[n];
        float v[8];
        if (!live) {
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
        float sx;
        if (ref) sx = bf_round(bf_round(bf_round(v[0] + v[1]) + v[2]) + v[3]) + bf_round(bf_round(bf_round(v[4] + v[5]) + v[6]) + v[7]);
        else sx = (((v[0] + v[1]) + v[2]) + v[3]) + (((v[4] + v[5]) + v[6]) + v[7]);
        __half h[8], l[8];
        float sf = 0.0f, sn = 0.0f;        // sums of the values as fed to the MMA: as staged, and in natural scale
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            // folded Q4 codes: the value that meets a "1024 + 16 q" slot must be 1/16 of its neighbours'. Even slots are
            // staged x 16 rather than odd slots / 16, which keeps small activations out of FP16's subnormal range; the
            // accumulated result is multiplied by 1/16 (exact) when it is finished.
            const float pre = (FOLD && Q4ORDER && !(i & 1)) ? v[i] * 16.0f : v[i];
            out_of_range |= fabsf(pre) > 65504.0f;          // would become an FP16 infinity: reported, not hidden
            h[i] = __float2half_rn(pre);
            float fed = __half2float(h[i]);
            if (SPLIT) { l[i] = __float2half_rn(pre - fed); fed += __half2float(l[i]); }
            sf += fed;
            sn += (FOLD && Q4ORDER && !(i & 1)) ? fed * 0.0625f : fed;
        }
        // The bias term multiplies the sum of the activations. Outside the reference arithmetic it uses the sum of
        // the values the MMA really sees, so that a rounding of an activation to FP16 enters the result through the
        // weight s q + b and not through s q alone.
        if (!ref) sx = sn;
#pragma unroll
        for (int off = 1; off <= 4; off <<= 1) {
            sx += __shfl_xor_sync(0xffffffffu, sx, off);
            sf += __shfl_xor_sync(0xffffffffu, sf, off);
        }
        if (!live) continue;
        if ((q & 7) == 0) *reinterpret_cast<float2*>(sums + ((q / 8) * NTOK + n) * 2) = make_float2((FOLD && Q4ORDER) ? 16.0f * sx : sx, FOLD ? -1024.0f * sf : 0.0f);
        constexpr int order_q4[8] = {0, 4, 1, 5, 2, 6, 3, 7};
        uint32_t ph[4], pl[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int a = Q4ORDER ? order_q4[2 * i] : 2 * i, b = Q4ORDER ? order_q4[2 * i + 1] : 2 * i + 1;
            ph[i] = uint32_t(__half_as_ushort(h[a])) | (uint32_t(__half_as_ushort(h[b])) << 16);
            if (SPLIT) pl[i] = uint32_t(__half_as_ushort(l[a])) | (uint32_t(__half_as_ushort(l[b])) << 16);
        }
        *reinterpret_cast<uint4*>(hi + n * RS + q * 8) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
        if (SPLIT) *reinterpret_cast<uint4*>(lo + n * RS + q * 8) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
    }
    if (out_of_range) atomicOr(status, ZC_STATUS_RANGE);
}

// Source of one matrix for this lane's cp.async copies. A pass of the warp copies ROWS_PER_PASS rows: the
// PIECES lanes of a row fetch its LINE as one contiguous run (one 128-byte request per row where the line is
// 128 bytes, instead of one request per 32-byte sector). In shared memory a row's groups are stored with
// the group index xor-ed by Fmt::swizzle(row), which keeps the MMA's row-strided reads free of bank conflicts.
template <int BITS, int CHT>
struct LaneSource {
    using F = Fmt<BITS, CHT>;
    const uint8_t* codes;      // record + codes offset + (row in pass) * row_bytes + piece * 16
    const uint8_t* meta;       // record + scales or biases offset (by kind) + row * G * 2
    uint32_t row_bytes, dst0, meta_pair;      // meta_pair: this lane's (row, kind) index in a metadata block
    const uint8_t* tile_codes; // set per tile
    const uint8_t* tile_meta;
    __device__ __forceinline__ void init(const uint8_t* record, const Projection& pr, uint32_t lane, uint32_t G) {
        row_bytes = pr.K * BITS / 8;
        const uint32_t piece = lane % F::PIECES, rip = lane / F::PIECES;
        const uint32_t block = piece * 16 / F::ROWB, within = piece * 16 % F::ROWB;
        dst0 = rip * F::LINE + ((block ^ F::swizzle(rip)) * F::ROWB) + within;      // swizzle(rip) == swizzle(row): passes add multiples of 4 rows
        codes = record + pr.codes + size_t(rip) * row_bytes + piece * 16;
        meta = record + (lane / 16 ? pr.biases : pr.scales) + size_t(lane % 16) * G * 2;
        meta_pair = (lane % 16) * 2 + lane / 16;
    }
    __device__ __forceinline__ void set_tile(uint32_t row0, uint32_t G) {
        tile_codes = codes + size_t(row0) * row_bytes;
        tile_meta = meta + size_t(row0) * G * 2;
    }
};

// Issue the cp.async copies of one chunk (CHT groups starting at grp0) of one matrix into a ring stage, and the
// metadata that goes with it. MB8: one 16-byte copy per (row, kind) every eight groups, into buffer meta_buf of two (a
// 4-byte copy per chunk moves a whole 32-byte sector for it and costs as many shared-memory wavefronts as a code copy);
// otherwise the chunk's own scale and bias halves, into the buffer of its ring slot.
template <int BITS, int CHT, int MBG>
__device__ __forceinline__ void issue_matrix(uint32_t stage, uint32_t meta_area, const LaneSource<BITS, CHT>& src, uint32_t grp0, uint32_t meta_buf, bool meta_now) {
    using F = Fmt<BITS, CHT>;
    const uint8_t* g0 = src.tile_codes + grp0 * F::ROWB;
#pragma unroll
    for (int p = 0; p < F::PASSES; ++p)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(stage + src.dst0 + p * F::ROWS_PER_PASS * F::LINE),
                     "l"(g0 + size_t(p * F::ROWS_PER_PASS) * src.row_bytes) : "memory");
    if constexpr (MBG == 8) {
        if (meta_now) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(meta_area + meta_buf * 512 + src.meta_pair * 16), "l"(src.tile_meta + grp0 * 2) : "memory");
    } else if constexpr (MBG == 4) {
        if (meta_now) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(meta_area + meta_buf * 256 + src.meta_pair * 8), "l"(src.tile_meta + grp0 * 2) : "memory");
    } else if constexpr (CHT == 4) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(meta_area + meta_buf * (32 * CHT * 2) + src.meta_pair * CHT * 2), "l"(src.tile_meta + grp0 * 2) : "memory");
    } else {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(meta_area + meta_buf * (32 * CHT * 2) + src.meta_pair * CHT * 2), "l"(src.tile_meta + grp0 * 2) : "memory");
    }
}

// (a & b) | c in one logic instruction.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Q4: one word -> four half2 (k0,k4) (k1,k5) (k2,k6) (k3,k7) of its 8 codes.
template <bool FOLD>
__device__ __forceinline__ void dequant_q4(uint32_t w, uint32_t (&p)[4]) {
    const uint32_t lo = 0x000f000fu, hi = 0x00f000f0u, magic = 0x64006400u;
    const uint32_t w8 = w >> 8;
    p[0] = and_or(w, lo, magic);
    p[1] = and_or(w, hi, magic);
    p[2] = and_or(w8, lo, magic);
    p[3] = and_or(w8, hi, magic);
    if (!FOLD) {
        const __half2 k1024 = __floats2half2_rn(1024.0f, 1024.0f), k16 = __floats2half2_rn(0.0625f, 0.0625f), k64 = __floats2half2_rn(-64.0f, -64.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 v = *reinterpret_cast<__half2*>(&p[i]);
            v = (i & 1) ? __hfma2(v, k16, k64) : __hsub2(v, k1024);
            p[i] = *reinterpret_cast<uint32_t*>(&v);
        }
    }
}
// Q8: one word -> two half2 (k0,k1) (k2,k3); every integer in [-128, 255] is exact in FP16.
__device__ __forceinline__ void dequant_q8(uint32_t w, bool is_signed, uint32_t (&p)[2]) {
    if (is_signed) w ^= 0x80808080u;
    const float off = is_signed ? 8388608.0f + 128.0f : 8388608.0f;
    float f[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __uint_as_float(0x4b000000u | ((w >> (8 * i)) & 0xffu)) - off;
    const __half2 a = __floats2half2_rn(f[0], f[1]), b = __floats2half2_rn(f[2], f[3]);
    p[0] = *reinterpret_cast<const uint32_t*>(&a);
    p[1] = *reinterpret_cast<const uint32_t*>(&b);
}

// d(16 rows x 8 tokens) = sum over one 64-wide group of code * x for the lane's rows g (w0) and g+8 (w1).
template <int BITS, bool SPLIT, bool FOLD>
__device__ __forceinline__ void group_mma(float (&d)[4], float c0, float c1, const uint32_t* w0, const uint32_t* w1, const uint4 (&bh)[2], const uint4 (&bl)[2], bool q8_signed) {
    if constexpr (BITS == 4) {
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            uint32_t p0[4], p1[4];
            dequant_q4<FOLD>(w0[m], p0);
            dequant_q4<FOLD>(w1[m], p1);
            if (m == 0) mma_f16_16816_c(d, p0[0], p1[0], p0[1], p1[1], bh[m].x, bh[m].y, c0, c1, c0, c1);
            else mma_f16_16816(d, p0[0], p1[0], p0[1], p1[1], bh[m].x, bh[m].y);
            mma_f16_16816(d, p0[2], p1[2], p0[3], p1[3], bh[m].z, bh[m].w);
            if constexpr (SPLIT) {
                mma_f16_16816(d, p0[0], p1[0], p0[1], p1[1], bl[m].x, bl[m].y);
                mma_f16_16816(d, p0[2], p1[2], p0[3], p1[3], bl[m].z, bl[m].w);
            }
        }
    } else {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            uint32_t p0[2], p1[2];
            dequant_q8(w0[m], q8_signed, p0);
            dequant_q8(w1[m], q8_signed, p1);
            const uint32_t b0 = (m & 1) ? bh[m / 2].z : bh[m / 2].x, b1 = (m & 1) ? bh[m / 2].w : bh[m / 2].y;
            if (m == 0) mma_f16_16816_c(d, p0[0], p1[0], p0[1], p1[1], b0, b1, c0, c1, c0, c1);
            else mma_f16_16816(d, p0[0], p1[0], p0[1], p1[1], b0, b1);
            if constexpr (SPLIT) {
                const uint32_t c0 = (m & 1) ? bl[m / 2].z : bl[m / 2].x, c1 = (m & 1) ? bl[m / 2].w : bl[m / 2].y;
                mma_f16_16816(d, p0[0], p1[0], p0[1], p1[1], c0, c1);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The expert kernel. Grid: (N / (16 * RT * tiles_per_warp), items) with RT = WARPS / KS row tiles side
// by side in a CTA; a warp walks `tiles_per_warp` consecutive 16-row tiles, and its cp.async ring keeps
// streaming across the tile boundaries.
//   NMAT = 2: gate/up + SwiGLU into hbuf.   NMAT = 1: down projection into the router positions.
//   KS: warps that split K for one row tile (partials added in warp order through shared memory).
// ---------------------------------------------------------------------------------------------
//   MW: 1 = a warp streams all NMAT matrices of its rows; 2 (gate/up only) = gate and up of the same rows
//       go to two different warps, which halves the registers and ring of a warp (three CTAs per SM instead
//       of two) at the price of meeting in shared memory for the SwiGLU.
//   CH: quantisation groups per ring stage (4 when K is a multiple of 256, else 2; Q8 always 2).
//   MBG: scales and biases arrive MBG = 8 or 4 groups at a time (needs KS = 1 and a group count that is a multiple of MBG); 0: with every ring stage.
template <int BITS, bool SPLIT, int NMAT, int KS, bool FOLD, bool META_F16, int MW, int CH, int MBG>
__global__ void __launch_bounds__(EXPERT_THREADS, NMAT == 1 ? ZC_MIN_BLOCKS_DOWN : (MW == 2 ? 3 : ZC_MIN_BLOCKS)) expert_kernel(Call c, uint32_t tiles_per_warp) {
    using F = Fmt<BITS, CH>;
    constexpr int STAGES = stages_for(NMAT / MW, CH);
    constexpr int WM = NMAT / MW;                    // matrices per warp
    constexpr int RT = WARPS / (KS * MW);
    constexpr int STAGE = WM * F::MATRIX;
    constexpr int META_AREA = F::meta_area(MBG, STAGES);
    constexpr bool MB8 = MBG != 0;                   // metadata in blocks of MBG groups
    constexpr int MBLOCK = MBG ? MBG : 8;
    constexpr bool VIA_SMEM = KS > 1 || MW > 1;
    constexpr int WORDS = F::ROWB / 16;              // 32-bit words per lane per row per group: 2 (Q4) / 4 (Q8)
    constexpr bool FOLDQ = FOLD && BITS == 4;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // gate/up follows the routing kernel and needs its lists at once. down follows gate/up, whose own wait has
    // already seen the routing kernel complete: the item, the row lists and the first weight stages of down are
    // set up while gate/up is still draining, and only the read of the SwiGLU rows waits for it.
    if constexpr (NMAT == 2) { pdl_wait(); pdl_launch_dependents(); }
    ItemInfo it;
    if (!decode_item(c, blockIdx.y, it)) return;
    const uint32_t K = NMAT == 2 ? c.H : c.F, G = K / 64, RS = K + ROW_PAD;
    __half* xhi = reinterpret_cast<__half*>(smem_raw);
    __half* xlo = xhi + (SPLIT ? NTOK * RS : 0);
    float* sums = reinterpret_cast<float*>(xhi + (SPLIT ? 2 : 1) * NTOK * RS);       // [G][NTOK][2]
    uint8_t* ring = reinterpret_cast<uint8_t*>(sums + G * NTOK * 2);                  // [WARPS][STAGES][STAGE]
    uint8_t* meta_all = ring + WARPS * STAGES * STAGE;                                // [WARPS][WM][META_AREA]
    float* red = reinterpret_cast<float*>(meta_all + WARPS * WM * META_AREA);      // [KS][NMAT][RT*16][NTOK] when VIA_SMEM
    __shared__ int rows[NTOK];
    __shared__ long long dest[NTOK];

    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane / 4, cq = lane % 4;
    const uint32_t mw = warp % MW, ks = (warp / MW) % KS, rt = warp / (MW * KS);
    const uint32_t first_tile = (blockIdx.x * RT + rt) * tiles_per_warp;
    uint8_t* my_ring = ring + warp * STAGES * STAGE;
    uint8_t* my_meta = meta_all + warp * WM * META_AREA;
    const uint32_t nchunks = G / CH;                 // G is a multiple of CH
    const uint32_t my_n = ks < nchunks ? (nchunks - ks + KS - 1) / KS : 0;
    const uint32_t my_tiles = my_n ? tiles_per_warp : 0;
    const bool q8s = c.q8_signed;
    float* out_base = it.shared ? c.shared_out : c.expert_out;
    LaneSource<BITS, CH> src[WM];
#pragma unroll
    for (int j = 0; j < WM; ++j) {
        const uint32_t mi = mw * WM + j;             // 0 = gate (or down), 1 = up
        src[j].init(it.record, NMAT == 1 ? c.down : (mi == 0 ? c.gate : c.up), lane, G);
    }

    // An item with more than eight rows takes several passes; with gridDim.z > 1 they are spread over that many CTAs
    // (a pass is independent of the others), so that one long item does not set the duration of a launch.
    for (uint32_t pass = blockIdx.z; pass * NTOK < it.count; pass += gridDim.z) {
        const uint32_t nvalid = min(uint32_t(NTOK), it.count - pass * NTOK);
        uint32_t is_tile = 0, is_chunk = 0, is_slot = 0;        // producer position in the flattened (tile, chunk) sequence
        uint32_t is_mblk = 0;                  // MB8: metadata blocks issued so far; the next one goes to buffer is_mblk & 1
        const uint32_t ring_base = smem_u32(my_ring), meta_base = smem_u32(my_meta);
#pragma unroll
        for (int m = 0; m < WM; ++m) src[m].set_tile(first_tile * 16, G);
        auto issue = [&]() {
            if (is_tile < my_tiles) {
                const uint32_t stage = ring_base + is_slot * STAGE, grp0 = (ks + is_chunk * KS) * CH;
                const bool meta_now = MB8 && (is_chunk * CH) % MBLOCK == 0;
                const uint32_t meta_buf = MB8 ? (is_mblk & 1) : is_slot;
#pragma unroll
                for (int m = 0; m < WM; ++m) issue_matrix<BITS, CH, MBG>(stage + m * F::MATRIX, meta_base + m * META_AREA, src[m], grp0, meta_buf, meta_now);
                if (meta_now) ++is_mblk;
                if (++is_chunk == my_n) {
                    is_chunk = 0; ++is_tile;
#pragma unroll
                    for (int m = 0; m < WM; ++m) src[m].set_tile((first_tile + is_tile) * 16, G);
                }
            }
            cp_async_commit();
            is_slot = is_slot + 1 == STAGES ? 0 : is_slot + 1;
        };
        __syncthreads();                       // everything of the previous pass has been consumed
#pragma unroll
        for (int i = 0; i < STAGES - 1; ++i) issue();    // weights do not depend on the rows: start them first
        if (threadIdx.x < NTOK) {
            const uint32_t i = pass * NTOK + threadIdx.x;
            if (i < it.count) {
                if (NMAT == 2) rows[threadIdx.x] = it.shared ? int(it.pos0 + i) : c.perm[it.pos0 + i] / int(c.K);
                else rows[threadIdx.x] = int(it.hrow0 + i);
                const uint32_t slot = it.shared ? it.pos0 + i : uint32_t(c.perm[it.pos0 + i]);
                dest[threadIdx.x] = NMAT == 2 ? (long long)(it.hrow0 + i) * c.F : (long long)slot * c.H;
            } else { rows[threadIdx.x] = -1; dest[threadIdx.x] = -1; }
        }
        __syncthreads();
        if constexpr (NMAT == 1) { pdl_wait(); pdl_launch_dependents(); }
        stage_rows<BITS == 4, SPLIT, FOLDQ>(NMAT == 2 ? c.x : static_cast<const void*>(c.hbuf), NMAT == 2 ? c.act_dtype == ZC_F32 : true,
                                            rows, nvalid, K, c.ref && BITS == 4, xhi, xlo, sums, c.status);
        __syncthreads();

        // The lane holds rows g, g+8 of its tile for tokens 2cq, 2cq+1.
        auto finish = [&](uint32_t row, uint32_t n, float a0, float a1) {
            const long long d = dest[n];
            if (d < 0) return;
            if constexpr (FOLDQ) { a0 *= 0.0625f; a1 *= 0.0625f; }          // the rows were staged x 16
            if constexpr (NMAT == 2) {
                float h;
                if (c.ref) {   // qwen.metal:71-81
                    const float gate = bf_round(a0), up = bf_round(a1);
                    h = bf_round(bf_round(gate * sigmoid_bf(gate)) * up);
                } else {
                    h = (a0 * sigmoid_f(a0)) * a1;
                }
                c.hbuf[d + row] = h;
            } else {
                out_base[d + row] = c.ref ? bf_round(a0) : a0;
            }
        };

        uint32_t slot = 0, mblk = 0;           // mblk: metadata blocks the consumer has begun (MB8)
        for (uint32_t tile = 0; tile < tiles_per_warp; ++tile) {
            float acc[WM][4];
#pragma unroll
            for (int m = 0; m < WM; ++m) { acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.0f; }
            for (uint32_t i = 0; i < my_n; ++i) {
                cp_async_wait<STAGES - 2>();
                __syncwarp();
                const uint8_t* stage = my_ring + slot * STAGE;
                // this chunk's scale and bias halves: at its place in the current 8-group block (MB8), or in the buffer of its slot
                if (MB8 && (i * CH) % MBLOCK == 0) ++mblk;
                constexpr uint32_t PAIR = MB8 ? uint32_t(MBLOCK * 2) : uint32_t(CH * 2);          // bytes of one (row, kind) entry
                const uint8_t* mbase = MB8 ? my_meta + ((mblk - 1) & 1) * (32 * PAIR) + ((i * CH) % MBLOCK) * 2 : my_meta + slot * (32 * CH * 2);
                slot = slot + 1 == STAGES ? 0 : slot + 1;
                issue();          // refills the slot consumed by the previous iteration while this chunk is multiplied
                const uint32_t grp0 = (ks + i * KS) * CH;
                uint32_t mraw[WM][2][CH];                        // per row: CH scale halves then CH bias halves, two per word
#pragma unroll
                for (int m = 0; m < WM; ++m) {
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        const uint8_t* mp = mbase + m * META_AREA + (g + 8 * r) * 2 * PAIR;
                        if constexpr (CH == 4) {
                            const uint2 sc = *reinterpret_cast<const uint2*>(mp), bi = *reinterpret_cast<const uint2*>(mp + PAIR);
                            mraw[m][r][0] = sc.x; mraw[m][r][1] = sc.y; mraw[m][r][2] = bi.x; mraw[m][r][3] = bi.y;
                        } else if constexpr (MB8) {
                            mraw[m][r][0] = *reinterpret_cast<const uint32_t*>(mp); mraw[m][r][1] = *reinterpret_cast<const uint32_t*>(mp + PAIR);
                        } else {
                            const uint2 v = *reinterpret_cast<const uint2*>(mp);
                            mraw[m][r][0] = v.x; mraw[m][r][1] = v.y;
                        }
                    }
                }
                // scale / bias of row r (0: g, 1: g+8) for group j of the chunk, converted where it is used
                auto meta_of = [&](int m, int r, int j, bool bias) {
                    const uint32_t word = mraw[m][r][(bias ? CH / 2 : 0) + j / 2];
                    const uint16_t bits = (j & 1) ? uint16_t(word >> 16) : uint16_t(word & 0xffffu);
                    return META_F16 ? __half2float(__ushort_as_half(bits)) : bf_to_float(bits);
                };
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    const uint32_t grp = grp0 + j;
                    uint4 bh[2], bl[2];
                    bh[0] = bh[1] = bl[0] = bl[1] = make_uint4(0, 0, 0, 0);
                    if (g < nvalid) {             // lanes of absent token rows skip the reads (their MMA columns are never stored)
                        const __half* bp = xhi + g * RS + grp * 64 + cq * 16;
                        bh[0] = *reinterpret_cast<const uint4*>(bp);
                        bh[1] = *reinterpret_cast<const uint4*>(bp + 8);
                        if constexpr (SPLIT) {
                            const __half* lp = xlo + g * RS + grp * 64 + cq * 16;
                            bl[0] = *reinterpret_cast<const uint4*>(lp);
                            bl[1] = *reinterpret_cast<const uint4*>(lp + 8);
                        }
                    }
                    const float4 sm = *reinterpret_cast<const float4*>(sums + (grp * NTOK + 2 * cq) * 2);   // (Sx, P) of tokens 2cq, 2cq+1
#pragma unroll
                    for (int m = 0; m < WM; ++m) {
                        const uint8_t* ms = stage + m * F::MATRIX;
                        uint32_t w0[WORDS], w1[WORDS];
                        const uint32_t blk = ((uint32_t(j) ^ F::swizzle(g)) * F::ROWB);           // swizzle(g + 8) == swizzle(g)
                        if constexpr (BITS == 4) {
                            const uint2 a = *reinterpret_cast<const uint2*>(ms + g * F::LINE + blk + cq * 8);
                            const uint2 b = *reinterpret_cast<const uint2*>(ms + (g + 8) * F::LINE + blk + cq * 8);
                            w0[0] = a.x; w0[1] = a.y; w1[0] = b.x; w1[1] = b.y;
                        } else {
                            const uint4 a = *reinterpret_cast<const uint4*>(ms + g * F::LINE + blk + cq * 16);
                            const uint4 b = *reinterpret_cast<const uint4*>(ms + (g + 8) * F::LINE + blk + cq * 16);
                            w0[0] = a.x; w0[1] = a.y; w0[2] = a.z; w0[3] = a.w; w1[0] = b.x; w1[1] = b.y; w1[2] = b.z; w1[3] = b.w;
                        }
                        float d[4];
                        group_mma<BITS, SPLIT, FOLDQ>(d, sm.y, sm.w, w0, w1, bh, bl, q8s);    // starts from P: removes the folded offset
                        const float s0 = meta_of(m, 0, j, false), s1 = meta_of(m, 1, j, false), b0 = meta_of(m, 0, j, true), b1 = meta_of(m, 1, j, true);
                        acc[m][0] = __fmaf_rn(s0, d[0], acc[m][0]); acc[m][0] = __fmaf_rn(b0, sm.x, acc[m][0]);
                        acc[m][1] = __fmaf_rn(s0, d[1], acc[m][1]); acc[m][1] = __fmaf_rn(b0, sm.z, acc[m][1]);
                        acc[m][2] = __fmaf_rn(s1, d[2], acc[m][2]); acc[m][2] = __fmaf_rn(b1, sm.x, acc[m][2]);
                        acc[m][3] = __fmaf_rn(s1, d[3], acc[m][3]); acc[m][3] = __fmaf_rn(b1, sm.z, acc[m][3]);
                    }
                }
                __syncwarp();
            }
            const uint32_t cta_row0 = blockIdx.x * RT * tiles_per_warp * 16;
            if constexpr (!VIA_SMEM) {
                const uint32_t row0 = (first_tile + tile) * 16;
#pragma unroll
                for (int i = 0; i < 4; ++i) finish(row0 + g + 8 * (i >> 1), 2 * cq + (i & 1), acc[0][i], acc[WM - 1][i]);
            } else {
                // partials: [ks][matrix][row tile in CTA][row][token]
#pragma unroll
                for (int m = 0; m < WM; ++m) {
                    float* mine = red + ((ks * NMAT + mw * WM + m) * RT * 16 + rt * 16) * NTOK;
                    *reinterpret_cast<float2*>(mine + g * NTOK + 2 * cq) = make_float2(acc[m][0], acc[m][1]);
                    *reinterpret_cast<float2*>(mine + (g + 8) * NTOK + 2 * cq) = make_float2(acc[m][2], acc[m][3]);
                }
                __syncthreads();
                for (uint32_t o = threadIdx.x; o < RT * 16 * NTOK; o += EXPERT_THREADS) {
                    const uint32_t r = o / NTOK, n = o % NTOK;
                    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
                    for (int k = 0; k < KS; ++k) {
                        a0 += red[((k * NMAT + 0) * RT * 16 + r) * NTOK + n];
                        if constexpr (NMAT == 2) a1 += red[((k * NMAT + 1) * RT * 16 + r) * NTOK + n];
                    }
                    // row tile r/16 of this CTA walks tiles (blockIdx.x*RT + r/16) * tiles_per_warp + tile
                    finish(cta_row0 + ((r / 16) * tiles_per_warp + tile) * 16 + r % 16, n, a0, a1);
                }
                __syncthreads();
            }
        }
        cp_async_wait<0>();
    }
}

template <int BITS, bool SPLIT, int NMAT, int KS, bool FOLD, bool META_F16, int MW, int CH, int MBG>
int launch_expert_mb(zc_moe* m, const Call& c, uint32_t items, uint32_t tiles_per_warp, cudaStream_t s) {
    constexpr int RT = WARPS / (KS * MW);
    constexpr int STAGES = stages_for(NMAT / MW, CH);
    const uint32_t K = NMAT == 2 ? c.H : c.F, N = NMAT == 2 ? c.F : c.H, G = K / 64;
    const size_t smem = size_t(SPLIT ? 2 : 1) * NTOK * (K + ROW_PAD) * 2 + size_t(G) * NTOK * 2 * 4 +
                        size_t(WARPS) * (NMAT / MW) * (STAGES * Fmt<BITS, CH>::MATRIX + Fmt<BITS, CH>::meta_area(MBG, STAGES)) + ((KS > 1 || MW > 1) ? size_t(KS) * NMAT * RT * 16 * NTOK * 4 : 0);
    if (smem > 220 * 1024) return fail(m, ZC_EINVAL, "expert kernel: shape needs too much shared memory");
    while (tiles_per_warp > 1 && N % (16 * RT * tiles_per_warp)) --tiles_per_warp;
    if (N % (16 * RT * tiles_per_warp)) return fail(m, ZC_EINVAL, "expert kernel: rows not a multiple of the CTA tile");
    // Items that can have more than eight rows (two or more rows per expert on average, or the few-row side of a long
    // batch with its limit above eight): their passes run as separate CTAs.
    const uint32_t pass_ctas = (KS == 1 && (c.item_rows_max > NTOK || uint64_t(c.T) * c.K >= 2ull * c.local_experts)) ? 2u : 1u;
    auto kernel = expert_kernel<BITS, SPLIT, NMAT, KS, FOLD, META_F16, MW, CH, MBG>;
    static SmemOptIn configured;        // one per instantiation of this function template
    if (opt_in_smem(kernel, configured, m->device, smem) != cudaSuccess) return check_launch(m, "expert kernel attribute");
    Timed t(m, s, NMAT == 2 ? KERNEL_GATE_UP : KERNEL_DOWN);
    const cudaError_t e = launch_chained(m, NMAT == 2 ? KERNEL_GATE_UP : KERNEL_DOWN, kernel, dim3(N / (16 * RT * tiles_per_warp), items, pass_ctas), dim3(EXPERT_THREADS), smem, s, nullptr, 0, c, tiles_per_warp);
    if (e != cudaSuccess) return fail(m, ZC_EEXEC, std::string("expert kernel launch: ") + cudaGetErrorString(e));
    return check_launch(m, NMAT == 2 ? "gate_up" : "down");
}

// Metadata in 8-group blocks: possible where a warp walks K in order (KS = 1) and every block of a row's metadata is
// 16-byte aligned; used for gate/up with long rows (hidden 4096: 423 -> 368 us at 512 experts x 5 rows). With short rows
// the extra kilobyte per warp pushes two CTAs per SM over a shared-memory carve-out step, which costs the L1 that serves
// the small copies (97 -> 104 us at hidden 2048), and down's short K does not gain (56 -> 58 us): those keep one block per
// ring stage. Option meta_blocks: 0 never, 1 by this rule, 2 wherever possible, 3 four-group blocks for gate/up.
template <int BITS, bool SPLIT, int NMAT, int KS, bool FOLD, bool META_F16, int MW, int CH>
int launch_expert_ch(zc_moe* m, const Call& c, uint32_t items, uint32_t tiles_per_warp, cudaStream_t s) {
    if constexpr (KS == 1) {
        const uint32_t K = NMAT == 2 ? c.H : c.F, G = K / 64;
        const bool long_rows = NMAT == 2 && K >= 4096;
        if (G % 8 == 0 && (m->meta_blocks == 2 || (m->meta_blocks == 1 && long_rows)))
            return launch_expert_mb<BITS, SPLIT, NMAT, KS, FOLD, META_F16, MW, CH, 8>(m, c, items, tiles_per_warp, s);
        if constexpr (CH == 2 && NMAT == 2) {       // 4-group blocks (8-byte copies every second stage; stays inside the carve-out): 99.7 against 98.1 us at hidden 2048, so only on request
            if (G % 4 == 0 && m->meta_blocks == 3)
                return launch_expert_mb<BITS, SPLIT, NMAT, KS, FOLD, META_F16, MW, CH, 4>(m, c, items, tiles_per_warp, s);
        }
    }
    return launch_expert_mb<BITS, SPLIT, NMAT, KS, FOLD, META_F16, MW, CH, 0>(m, c, items, tiles_per_warp, s);
}

// Two groups per ring stage for gate/up: four groups per stage (a full 128-byte line per Q4 row) leave room for
// only two stages next to the staged rows and measured 13 % slower at hidden 2048.
template <int BITS, bool SPLIT, int NMAT, int KS, bool FOLD, bool META_F16, int MW>
int launch_expert(zc_moe* m, const Call& c, uint32_t items, uint32_t tiles_per_warp, cudaStream_t s) {
    // down, whose K is short (eight groups at ffn 512), is bound by instruction issue: four groups per stage halve
    // its per-stage bookkeeping (three stages still fit beside its small row tile).
    if constexpr (BITS == 4 && NMAT == 1 && KS == 1) {
        if ((c.F / 64) % 4 == 0) return launch_expert_ch<BITS, SPLIT, NMAT, KS, FOLD, META_F16, MW, 4>(m, c, items, tiles_per_warp, s);
    }
    return launch_expert_ch<BITS, SPLIT, NMAT, KS, FOLD, META_F16, MW, 2>(m, c, items, tiles_per_warp, s);
}

template <int NMAT, int KS, bool META_F16, int MW>
int dispatch_bits(zc_moe* m, const Call& c, uint32_t items, uint32_t tpw, bool split, uint32_t bits, bool fold, cudaStream_t s) {
    if (bits == 4) {
        if (fold) return split ? launch_expert<4, true, NMAT, KS, true, META_F16, MW>(m, c, items, tpw, s) : launch_expert<4, false, NMAT, KS, true, META_F16, MW>(m, c, items, tpw, s);
        return split ? launch_expert<4, true, NMAT, KS, false, META_F16, MW>(m, c, items, tpw, s) : launch_expert<4, false, NMAT, KS, false, META_F16, MW>(m, c, items, tpw, s);
    }
    return split ? launch_expert<8, true, NMAT, KS, false, META_F16, MW>(m, c, items, tpw, s) : launch_expert<8, false, NMAT, KS, false, META_F16, MW>(m, c, items, tpw, s);
}
template <int NMAT, int KS, int MW = 1>
int dispatch_expert(zc_moe* m, const Call& c, uint32_t items, uint32_t tpw, bool split, uint32_t bits, bool fold, cudaStream_t s) {
    return c.meta_f16 ? dispatch_bits<NMAT, KS, true, MW>(m, c, items, tpw, split, bits, fold, s)
                      : dispatch_bits<NMAT, KS, false, MW>(m, c, items, tpw, split, bits, fold, s);
}

}  // namespace

static int launch_experts_decode_one(zc_moe* m, const Call& c, cudaStream_t s);

// A shared expert whose record has other bit widths than the routed experts' (the reference's mixed artifact: routed Q4,
// shared Q8) cannot share a launch with them - the code width is a template parameter - so it runs as launches of its
// own over the same buffers (its rows of hbuf and shared_out are disjoint from the routed ones).
int launch_experts_decode(zc_moe* m, const Call& c, cudaStream_t s) {
    if (!(c.has_shared && c.shared_split)) return launch_experts_decode_one(m, c, s);
    int total = 0, n;
    if (c.items != m->empty_items) {
        Call routed = c;
        routed.has_shared = 0;
        if ((n = launch_experts_decode_one(m, routed, s)) < 0) return n;
        total += n;
    }
    Call shared = c;
    shared.gate = c.sgate; shared.up = c.sup; shared.down = c.sdown; shared.shared_split = 0;
    shared.items = m->empty_items; shared.counters = m->zero_counters;
    if ((n = launch_experts_decode_one(m, shared, s)) < 0) return n;
    return total + n;
}

static int launch_experts_decode_one(zc_moe* m, const Call& c, cudaStream_t s) {
    const uint32_t routed = c.T * c.K < c.local_experts ? c.T * c.K : c.local_experts;
    const uint32_t items = routed + (c.has_shared ? (c.T + NTOK - 1) / NTOK : 0);
    // A BF16 activation is exact as one FP16 term; an FP32 activation needs two, except under the
    // reference arithmetic, whose FP32 buffers hold BF16 values by contract.
    const bool split_x = c.act_dtype == ZC_F32 && !c.ref;
    // The SwiGLU rows h are FP32 in memory. By default the down product reads them as one FP16 term (11 significant
    // bits, against the 8 of the BF16 the reference rounds h to; measured 1.2e-3 x RMS max-abs at 64 tokens, inside the
    // 2e-3 bound); with the "exact_h" option as two FP16 terms, which costs a second MMA per fragment (73 us against
    // 56 us for the down launch of the benchmark layer). The reference arithmetic's h is BF16: exact in one term.
    const bool split_h = !c.ref && m->exact_h;
    const bool fold = m->fold_q4;
    // Few rows in flight: split K over all eight warps so that even one token fills the machine.
    const bool small = c.T * (c.K + (c.has_shared ? 1 : 0)) <= 64;
    int rc;
    if (small) rc = dispatch_expert<2, 8>(m, c, items, 1, split_x, c.gate.bits, fold, s);
#ifndef ZC_TPW_GU
#define ZC_TPW_GU 2
#endif
#ifndef ZC_TPW_DN
#define ZC_TPW_DN 4
#endif
    // As the few-row side of a long batch only a fraction of the items has work (the others leave at once): fewer
    // tiles per warp, i.e. more and shorter CTAs per item, keep the SMs filled.
    else rc = dispatch_expert<2, 1>(m, c, items, c.item_rows_max ? m->few_tiles_gate_up : ZC_TPW_GU, split_x, c.gate.bits, fold, s);
    if (rc < 0) return rc;
    if (small) rc = dispatch_expert<1, 2>(m, c, items, 1, split_h, c.down.bits, fold, s);
    else rc = dispatch_expert<1, 1>(m, c, items, c.item_rows_max ? m->few_tiles_down : ZC_TPW_DN, split_h, c.down.bits, fold, s);
    if (rc < 0) return rc;
    return 2;
}

}  // namespace zc
