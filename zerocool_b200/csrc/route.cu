// Top-k selection with renormalised softmax, and the token -> expert permutation.
//
// route_kernel replaces route_simd (kernels/metal/qwen.metal:768-795; serial twin :742-765): one warp
// per token, K rounds of "largest remaining score, ties to the lower expert index"; only scores
// greater than -inf can win, so NaN and -inf are never selected and unfilled ranks get id -1. The
// winning score is re-read from the logits (keeps signed zero). Weights: four values per lane,
// lane-sequential sum, xor-butterfly lane sum, one reciprocal, one multiply.
//
// permute_kernel replaces the CPU dispatch of Model::moe (src/engine/model.cpp:449-461, 473-474) and
// the row lists of encode_expert_rows (src/engine/pipeline.cpp:18-23): a stable counting sort of the
// flat slots p = t*K + j by expert id, done by one CTA. Each warp owns a contiguous range of slots;
// per-warp histograms, an exclusive scan over (expert, warp), and a second pass that places slots with
// warp match operations keep slots of one expert in ascending order without atomics on the order.
#include "common.cuh"

namespace zc {
namespace {

constexpr int ROUTE_THREADS = 256;
constexpr int ROUTE_WARPS = ROUTE_THREADS / 32;

struct RouteArgs {
    const float* logits;        // [T, E]
    int32_t* ids; float* weights;
    uint32_t T, E, K;
    uint32_t* status;
    // permutation tail (run by the last CTA to finish when do_permute is set)
    int32_t* offsets; int32_t* perm; int32_t* active; int4* items; int32_t* counters; uint32_t* done;
    uint32_t first_expert, local_experts, layer, do_permute;
};

// Order-preserving integer image of a score: a larger float gives a larger key, +0 and -0 share one key (they
// compare equal, so the lower expert index must win), and 0 means "cannot be selected" (NaN or -inf).
__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t u = __float_as_uint(__fadd_rn(v, 0.0f));          // -0 + 0 = +0
    const uint32_t k = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return v > __int_as_float(0xff800000) ? k : 0u;
}

// One warp per token. Lane l holds the keys of experts l, l+32, ... in registers; a round is a register tree for
// the lane's best (ties to the lower slot), one warp max-reduce of the key and one warp min-reduce of the index
// among the lanes that hold that key. `row` is the warp's shared-memory copy of the scores (the winner's own
// value is read back from it, which keeps a signed zero like the reference's re-read of the logit).
template <int MAXC>
__device__ __forceinline__ void route_token(const RouteArgs& a, uint32_t t, uint32_t lane, float* row, float* scores, int32_t* selected) {
    const uint32_t E = a.E, K = a.K, nc = E / 32;
    const float ninf = __int_as_float(0xff800000);
    uint32_t key[MAXC];
    const float* src = a.logits + size_t(t) * E;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
        key[i] = 0u;
        if (uint32_t(i) < nc) {
            const float v = __ldcg(src + lane + 32 * i);
            row[lane + 32 * i] = v;
            key[i] = order_key(v);
        }
    }
    for (uint32_t j = 0; j < K; ++j) {
        // lane's best key and its slot: pairwise tree, the right element wins only when strictly larger
        uint32_t bk[MAXC / 2], bs[MAXC / 2];
#pragma unroll
        for (int i = 0; i < MAXC / 2; ++i) {
            const bool right = key[2 * i + 1] > key[2 * i];
            bk[i] = right ? key[2 * i + 1] : key[2 * i];
            bs[i] = right ? 2 * i + 1 : 2 * i;
        }
#pragma unroll
        for (int width = MAXC / 4; width >= 1; width /= 2) {
#pragma unroll
            for (int i = 0; i < width; ++i) {
                const bool right = bk[2 * i + 1] > bk[2 * i];
                bk[i] = right ? bk[2 * i + 1] : bk[2 * i];
                bs[i] = right ? bs[2 * i + 1] : bs[2 * i];
            }
        }
        const uint32_t top = __reduce_max_sync(0xffffffffu, bk[0]);
        const uint32_t mine = (bk[0] == top && top != 0u) ? lane + 32 * bs[0] : 0xffffffffu;
        const uint32_t winner = __reduce_min_sync(0xffffffffu, mine);       // 0xffffffff: nothing left to select
#pragma unroll
        for (int i = 0; i < MAXC; ++i) key[i] = (lane + 32 * i == winner) ? 0u : key[i];
        if (lane == 0) selected[j] = winner < E ? int32_t(winner) : -1;
    }
    __syncwarp();
    if (lane < K) {
        const int32_t id = selected[lane];
        scores[lane] = id >= 0 ? row[id] : ninf;
    }
    __syncwarp();
    float values[4], sum = 0.0f;
    const float top = scores[0];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t j = lane * 4 + i;
        values[i] = j < K ? expf(scores[j < 32 ? j : 0] - top) : 0.0f;
        sum = __fadd_rn(sum, values[i]);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, off));
    const float inverse = __fdiv_rn(1.0f, sum);
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t j = lane * 4 + i;
        if (j < K) {
            const int32_t id = selected[j];
            a.ids[size_t(t) * K + j] = id;
            a.weights[size_t(t) * K + j] = __fmul_rn(values[i], inverse);
            bad |= id < 0;
        }
    }
    if (bad) atomicOr(a.status, ZC_STATUS_INVALID_ROUTE);
}

// Weights for a selection that is given, not searched (replay of a recorded route): the same renormalised softmax
// over the K selected scores, with the same lane layout and summation order as route_token. The first id of a token
// plays the role of rank 0 (its score is subtracted before the exponential). ids outside [0, E) get weight 0 and
// raise the status bit.
__global__ void __launch_bounds__(ROUTE_THREADS) forced_weights_kernel(const float* __restrict__ logits, const int32_t* __restrict__ forced,
                                                                        int32_t* __restrict__ ids, float* __restrict__ weights,
                                                                        uint32_t T, uint32_t E, uint32_t K, uint32_t* status) {
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= T) return;
    const float ninf = __int_as_float(0xff800000);
    const int32_t top_id = forced[size_t(t) * K];
    const float top = top_id >= 0 && uint32_t(top_id) < E ? __ldcg(logits + size_t(t) * E + top_id) : ninf;
    float values[4], sum = 0.0f;
    int32_t id[4];
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t j = lane * 4 + i;
        values[i] = 0.0f; id[i] = -1;
        if (j < K) {
            id[i] = forced[size_t(t) * K + j];
            const bool valid = id[i] >= 0 && uint32_t(id[i]) < E;
            bad |= !valid;
            if (!valid) id[i] = -1;
            values[i] = valid ? expf(__ldcg(logits + size_t(t) * E + id[i]) - top) : 0.0f;
        }
        sum = __fadd_rn(sum, values[i]);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, off));
    const float inverse = __fdiv_rn(1.0f, sum);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t j = lane * 4 + i;
        if (j < K) { ids[size_t(t) * K + j] = id[i]; weights[size_t(t) * K + j] = __fmul_rn(values[i], inverse); }
    }
    if (bad) atomicOr(status, ZC_STATUS_INVALID_ROUTE);
}

constexpr int PERMUTE_THREADS = 1024;
constexpr int PERMUTE_CACHE = 4;          // 32-slot chunks of a warp's range kept in registers between the two passes
constexpr int PERMUTE_OWN = 4;            // consecutive experts owned by one thread in the scan (E <= 4 x threads)

// Exclusive scan of one 64-bit value per thread over a CTA of NT threads; returns the exclusive prefix and the total.
template <int NT>
__device__ __forceinline__ unsigned long long block_exclusive_scan(unsigned long long value, unsigned long long* warp_totals, unsigned long long& total) {
    constexpr int NW = NT / 32;
    const uint32_t lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    unsigned long long inclusive = value;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const unsigned long long n = __shfl_up_sync(0xffffffffu, inclusive, off);
        if (lane >= uint32_t(off)) inclusive += n;
    }
    if (lane == 31) warp_totals[warp] = inclusive;
    __syncthreads();
    if (warp == 0) {
        const unsigned long long w = lane < NW ? warp_totals[lane] : 0ull;
        unsigned long long inc = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const unsigned long long n = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= uint32_t(off)) inc += n;
        }
        if (lane < NW) warp_totals[lane] = inc - w;   // exclusive prefix of the warp totals
        if (lane == 31) warp_totals[32] = inc;        // grand total
    }
    __syncthreads();
    total = warp_totals[32];
    return warp_totals[warp] + inclusive - value;
}

// Stable counting sort of the slots by expert id by one CTA of NT threads (hist: [NT/32][E] ints, zero on entry).
// Each warp owns a contiguous range of slots. Pass 1 counts per (warp, expert); one scan over the experts (each
// thread owns up to PERMUTE_OWN consecutive ones; slot counts in the low word and "has work" flags in the high
// word of one 64-bit scan) turns the counts into starting positions; pass 2 places the slots. CACHED keeps the
// ids of the warp's range in registers between the passes (ranges up to 32 x PERMUTE_CACHE slots).
template <int NT, bool CACHED>
__device__ __forceinline__ void permute_body(const int32_t* ids, uint32_t slots, uint32_t E,
                                             uint32_t first_expert, uint32_t local_experts,
                                             int32_t* __restrict__ offsets, int32_t* __restrict__ perm,
                                             int32_t* __restrict__ active, int4* __restrict__ items, int32_t* __restrict__ counters,
                                             uint32_t layer, uint32_t* status, int32_t* hist, uint32_t range) {
    constexpr int NW = NT / 32;
    __shared__ unsigned long long warp_totals[33];
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t begin = min(slots, warp * range), end = min(slots, begin + range);
    const int used = int(min(uint32_t(NW), (slots + range - 1) / max(range, 1u)));       // warps whose range is not empty: only their histograms count
    int32_t* mine = hist + warp * E;
    for (uint32_t i = threadIdx.x; i < E; i += NT) items[i].x = -1;        // entries past the end of the new list (ordered before the fill by the barriers below)
    int32_t cached[PERMUTE_CACHE];
    if constexpr (CACHED) {
#pragma unroll
        for (int q = 0; q < PERMUTE_CACHE; ++q) {
            const uint32_t p = begin + 32 * q + lane;
            cached[q] = p < end ? __ldcg(ids + p) : -1;
        }
    }
    bool bad = false;
    auto count_chunk = [&](uint32_t p, int32_t id) {
        const bool valid = id >= 0 && uint32_t(id) < E;
        bad |= p < end && !valid;
        const uint32_t key = valid ? uint32_t(id) : E + lane;     // invalid lanes match nobody
        const uint32_t peers = __match_any_sync(0xffffffffu, key);
        if (valid && (peers & ((1u << lane) - 1)) == 0) mine[id] += __popc(peers);
        __syncwarp();
    };
    if constexpr (CACHED) {
#pragma unroll
        for (int q = 0; q < PERMUTE_CACHE; ++q) if (begin + 32 * q < end) count_chunk(begin + 32 * q + lane, cached[q]);
    } else {
        for (uint32_t blk = begin; blk < end; blk += 32 * PERMUTE_CACHE) {      // four loads in flight per lane
            int32_t v[PERMUTE_CACHE];
#pragma unroll
            for (int q = 0; q < PERMUTE_CACHE; ++q) { const uint32_t p = blk + 32 * q + lane; v[q] = p < end ? __ldcg(ids + p) : -1; }
#pragma unroll
            for (int q = 0; q < PERMUTE_CACHE; ++q) if (blk + 32 * q < end) count_chunk(blk + 32 * q + lane, v[q]);
        }
    }
    if (bad && status) atomicOr(status, ZC_STATUS_INVALID_ROUTE);
    __syncthreads();
    // Per-warp counts become per-warp starting ranks inside the expert; the scan gives the expert's first position.
    const uint32_t own = (E + NT - 1) / NT;                        // <= PERMUTE_OWN, checked at launch
    const uint32_t e_first = threadIdx.x * own;
    int count[PERMUTE_OWN];
    unsigned long long packed = 0;
#pragma unroll
    for (int q = 0; q < PERMUTE_OWN; ++q) {
        const uint32_t e = e_first + q;
        count[q] = 0;
        if (uint32_t(q) < own && e < E) {
            int running = 0;
            for (int w = 0; w < used; ++w) { const int n = hist[w * E + e]; hist[w * E + e] = running; running += n; }
            count[q] = running;
            const bool has_work = running > 0 && e >= first_expert && e < first_expert + local_experts;
            packed += (unsigned long long)(running) | ((unsigned long long)(has_work ? 1 : 0) << 32);
        }
    }
    unsigned long long total;
    const unsigned long long before = block_exclusive_scan<NT>(packed, warp_totals, total);
    int offset = int(uint32_t(before)), slot = int(before >> 32);
#pragma unroll
    for (int q = 0; q < PERMUTE_OWN; ++q) {
        const uint32_t e = e_first + q;
        if (uint32_t(q) < own && e < E) {
            offsets[e] = offset;
            for (int w = 0; w < used; ++w) hist[w * E + e] += offset;
            if (count[q] > 0 && e >= first_expert && e < first_expert + local_experts) {
                active[slot] = int32_t(e);
                items[slot] = make_int4(int(e), offset, count[q], 0);
                ++slot;
            }
            offset += count[q];
        }
    }
    if (threadIdx.x == 0) { offsets[E] = int(uint32_t(total)); counters[0] = int(total >> 32); counters[16 + layer] = int(total >> 32); }
    __syncthreads();
    auto place_chunk = [&](uint32_t p, int32_t id) {
        const bool valid = id >= 0 && uint32_t(id) < E;
        const uint32_t key = valid ? uint32_t(id) : E + lane;
        const uint32_t peers = __match_any_sync(0xffffffffu, key);
        const uint32_t before_me = peers & ((1u << lane) - 1);
        int cursor = 0;
        if (valid) cursor = mine[id];
        __syncwarp();
        if (valid) {
            perm[cursor + __popc(before_me)] = int32_t(p);
            if (before_me == 0) mine[id] = cursor + __popc(peers);
        }
        __syncwarp();
    };
    if constexpr (CACHED) {
#pragma unroll
        for (int q = 0; q < PERMUTE_CACHE; ++q) if (begin + 32 * q < end) place_chunk(begin + 32 * q + lane, cached[q]);
    } else {
        for (uint32_t blk = begin; blk < end; blk += 32 * PERMUTE_CACHE) {
            int32_t v[PERMUTE_CACHE];
#pragma unroll
            for (int q = 0; q < PERMUTE_CACHE; ++q) { const uint32_t p = blk + 32 * q + lane; v[q] = p < end ? __ldcg(ids + p) : -1; }
#pragma unroll
            for (int q = 0; q < PERMUTE_CACHE; ++q) if (blk + 32 * q < end) place_chunk(blk + 32 * q + lane, v[q]);
        }
    }
}

// Contiguous slot range of one warp: a multiple of 32 long so that chunks stay aligned.
__host__ __device__ inline uint32_t permute_range(uint32_t slots, uint32_t warps) { return ((slots + warps - 1) / warps + 31) / 32 * 32; }

template <int NT>
__device__ __forceinline__ void permute_any(const int32_t* ids, uint32_t slots, uint32_t E, uint32_t first_expert, uint32_t local_experts,
                                            int32_t* offsets, int32_t* perm, int32_t* active, int4* items, int32_t* counters, uint32_t layer,
                                            uint32_t* status, int32_t* hist) {
    const uint32_t range = permute_range(slots, NT / 32);
    if (range <= 32 * PERMUTE_CACHE) permute_body<NT, true>(ids, slots, E, first_expert, local_experts, offsets, perm, active, items, counters, layer, status, hist, range);
    else permute_body<NT, false>(ids, slots, E, first_expert, local_experts, offsets, perm, active, items, counters, layer, status, hist, range);
}

__global__ void __launch_bounds__(PERMUTE_THREADS) permute_kernel(const int32_t* __restrict__ ids, uint32_t slots, uint32_t E,
                                                                   uint32_t first_expert, uint32_t local_experts,
                                                                   int32_t* __restrict__ offsets, int32_t* __restrict__ perm,
                                                                   int32_t* __restrict__ active, int4* __restrict__ items, int32_t* __restrict__ counters,
                                                                   uint32_t layer, uint32_t* status) {
    extern __shared__ int32_t hist[];
    const uint32_t used = min(uint32_t(PERMUTE_THREADS / 32), (slots + permute_range(slots, PERMUTE_THREADS / 32) - 1) / max(permute_range(slots, PERMUTE_THREADS / 32), 1u));
    for (uint32_t i = threadIdx.x; i < used * E; i += PERMUTE_THREADS) hist[i] = 0;
    __syncthreads();
    permute_any<PERMUTE_THREADS>(ids, slots, E, first_expert, local_experts, offsets, perm, active, items, counters, layer, status, hist);
}

// Expert-parallel owner: wait for the sources' rows, write the expert id of every row slot, and sort the slots, in one
// launch of one CTA (the two steps were separate launches of the same shape; one of them is a wait).
__global__ void __launch_bounds__(PERMUTE_THREADS) ep_receive_permute_kernel(EpArgs a, int32_t* __restrict__ row_ids, uint32_t* __restrict__ counts,
                                                                              uint32_t slots, uint32_t E, uint32_t first_expert, uint32_t local_experts,
                                                                              int32_t* __restrict__ offsets, int32_t* __restrict__ perm,
                                                                              int32_t* __restrict__ active, int4* __restrict__ items, int32_t* __restrict__ counters, uint32_t layer) {
    extern __shared__ int32_t hist[];
    __shared__ uint32_t count_s[EP_MAX_RANKS];
    const uint32_t used = min(uint32_t(PERMUTE_THREADS / 32), (slots + permute_range(slots, PERMUTE_THREADS / 32) - 1) / max(permute_range(slots, PERMUTE_THREADS / 32), 1u));
    for (uint32_t i = threadIdx.x; i < used * E; i += PERMUTE_THREADS) hist[i] = 0;
    pdl_wait();                             // the send kernel of this rank (its local rows and flag) has completed
    pdl_launch_dependents();
    ep_receive_body(a, row_ids, counts, count_s);
    __syncthreads();                        // the ids written above are read back by other threads of this CTA
    permute_any<PERMUTE_THREADS>(row_ids, slots, E, first_expert, local_experts, offsets, perm, active, items, counters, layer, nullptr, hist);
}

// Long batches (tens of thousands of slots): the same stable counting sort by many CTAs, in three launches.
//   permute_count_kernel: CTA b counts the experts of its PERMUTE_BLOCK consecutive slots      -> blocks[b][e]
//   permute_scan_kernel:  one CTA turns each expert's column into an exclusive running count over the CTAs
//                         (blocks[b][e] = slots of e before CTA b), scans the expert totals (offsets), and writes
//                         the list of experts with work, as the one-CTA form does
//   permute_place_kernel: CTA b ranks its own slots (per-warp counts, ids kept in registers between the passes) on
//                         top of offsets[e] + blocks[b][e] and writes perm
constexpr uint32_t PERMUTE_BLOCK = 2048;          // slots per CTA: 64 per warp of 1024 threads

__global__ void __launch_bounds__(PERMUTE_THREADS) permute_count_kernel(const int32_t* __restrict__ ids, uint32_t slots, uint32_t E,
                                                                         int32_t* __restrict__ blocks, uint32_t* status) {
    extern __shared__ int32_t hist[];
    for (uint32_t e = threadIdx.x; e < E; e += PERMUTE_THREADS) hist[e] = 0;
    __syncthreads();
    bool bad = false;
    for (uint32_t i = threadIdx.x; i < PERMUTE_BLOCK; i += PERMUTE_THREADS) {
        const uint32_t p = blockIdx.x * PERMUTE_BLOCK + i;
        if (p >= slots) break;
        const int32_t id = __ldcg(ids + p);
        if (id >= 0 && uint32_t(id) < E) atomicAdd(&hist[id], 1);
        else bad = true;
    }
    if (bad && status) atomicOr(status, ZC_STATUS_INVALID_ROUTE);
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < E; e += PERMUTE_THREADS) blocks[size_t(blockIdx.x) * E + e] = hist[e];
}

__global__ void __launch_bounds__(PERMUTE_THREADS) permute_scan_kernel(int32_t* __restrict__ blocks, uint32_t nblocks, uint32_t E,
                                                                        uint32_t first_expert, uint32_t local_experts,
                                                                        int32_t* __restrict__ offsets, int32_t* __restrict__ active, int4* __restrict__ items,
                                                                        int32_t* __restrict__ counters, uint32_t layer) {
    __shared__ unsigned long long warp_totals[33];
    for (uint32_t i = threadIdx.x; i < E; i += PERMUTE_THREADS) items[i].x = -1;        // entries past the end of the new list
    __syncthreads();
    const uint32_t own = (E + PERMUTE_THREADS - 1) / PERMUTE_THREADS;      // <= PERMUTE_OWN, checked at launch
    // Thread i owns experts i, i + NT, ... for the column sums (coalesced) ...
    for (uint32_t q = 0; q < own; ++q) {
        const uint32_t e = q * PERMUTE_THREADS + threadIdx.x;
        if (e >= E) break;
        int running = 0;
        for (uint32_t b = 0; b < nblocks; ++b) { const int n = blocks[size_t(b) * E + e]; blocks[size_t(b) * E + e] = running; running += n; }
        offsets[e] = running;                   // the expert's total for now; becomes its first position below
    }
    __syncthreads();
    // ... and `own` consecutive experts for the scan, as the one-CTA form.
    const uint32_t e_first = threadIdx.x * own;
    int count[PERMUTE_OWN];
    unsigned long long packed = 0;
#pragma unroll
    for (int q = 0; q < PERMUTE_OWN; ++q) {
        const uint32_t e = e_first + q;
        count[q] = 0;
        if (uint32_t(q) < own && e < E) {
            count[q] = offsets[e];
            const bool has_work = count[q] > 0 && e >= first_expert && e < first_expert + local_experts;
            packed += (unsigned long long)(count[q]) | ((unsigned long long)(has_work ? 1 : 0) << 32);
        }
    }
    __syncthreads();
    unsigned long long total;
    const unsigned long long before = block_exclusive_scan<PERMUTE_THREADS>(packed, warp_totals, total);
    int offset = int(uint32_t(before)), slot = int(before >> 32);
#pragma unroll
    for (int q = 0; q < PERMUTE_OWN; ++q) {
        const uint32_t e = e_first + q;
        if (uint32_t(q) < own && e < E) {
            offsets[e] = offset;
            if (count[q] > 0 && e >= first_expert && e < first_expert + local_experts) {
                active[slot] = int32_t(e);
                items[slot] = make_int4(int(e), offset, count[q], 0);
                ++slot;
            }
            offset += count[q];
        }
    }
    if (threadIdx.x == 0) { offsets[E] = int(uint32_t(total)); counters[0] = int(total >> 32); counters[16 + layer] = int(total >> 32); }
}

__global__ void __launch_bounds__(PERMUTE_THREADS) permute_place_kernel(const int32_t* __restrict__ ids, uint32_t slots, uint32_t E,
                                                                         const int32_t* __restrict__ blocks, const int32_t* __restrict__ offsets,
                                                                         int32_t* __restrict__ perm) {
    extern __shared__ int32_t hist[];            // [32 warps][E]
    constexpr uint32_t NW = PERMUTE_THREADS / 32, CHUNKS = PERMUTE_BLOCK / PERMUTE_THREADS;
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t begin = blockIdx.x * PERMUTE_BLOCK + warp * (32 * CHUNKS);
    int32_t* mine = hist + warp * E;
    for (uint32_t i = threadIdx.x; i < NW * E; i += PERMUTE_THREADS) hist[i] = 0;
    int32_t cached[CHUNKS];
#pragma unroll
    for (uint32_t q = 0; q < CHUNKS; ++q) { const uint32_t p = begin + 32 * q + lane; cached[q] = p < slots ? __ldcg(ids + p) : -1; }
    __syncthreads();
#pragma unroll
    for (uint32_t q = 0; q < CHUNKS; ++q) {
        const int32_t id = cached[q];
        const bool valid = id >= 0 && uint32_t(id) < E;
        const uint32_t peers = __match_any_sync(0xffffffffu, valid ? uint32_t(id) : E + lane);
        if (valid && (peers & ((1u << lane) - 1)) == 0) mine[id] += __popc(peers);
        __syncwarp();
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < E; e += PERMUTE_THREADS) {
        int running = offsets[e] + blocks[size_t(blockIdx.x) * E + e];
        for (uint32_t w = 0; w < NW; ++w) { const int n = hist[w * E + e]; hist[w * E + e] = running; running += n; }
    }
    __syncthreads();
#pragma unroll
    for (uint32_t q = 0; q < CHUNKS; ++q) {
        const int32_t id = cached[q];
        const bool valid = id >= 0 && uint32_t(id) < E;
        const uint32_t peers = __match_any_sync(0xffffffffu, valid ? uint32_t(id) : E + lane);
        const uint32_t before_me = peers & ((1u << lane) - 1);
        int cursor = 0;
        if (valid) cursor = mine[id];
        __syncwarp();
        if (valid) {
            perm[cursor + __popc(before_me)] = int32_t(begin + 32 * q + lane);
            if (before_me == 0) mine[id] = cursor + __popc(peers);
        }
        __syncwarp();
    }
}

// Route (one warp per token, eight tokens per CTA) and, when asked, the permutation as the tail of the
// last CTA to finish, so that a layer needs one launch for both. Dynamic shared memory: the eight score rows
// [8][E] floats, reused as the [8][E] histogram of the permutation.
// The permutation of a batch that one routing CTA covers (at most eight tokens, so at most 256 slots): the selections
// are still in shared memory, so each slot finds its place by counting - its expert's first position is the number of
// slots with a smaller expert id, its rank the number of earlier slots with the same id - and each expert's first slot
// writes the expert's entry of the work list. No histogram, no scan, no re-read of the ids from global memory, and no
// arrival counter; the result is the same stable counting sort.
__device__ __forceinline__ void permute_small(const RouteArgs& a, const int32_t (*selected)[32], int32_t* flat, int32_t* opens /* [256] shared each */) {
    const uint32_t slots = a.T * a.K, E = a.E, tid = threadIdx.x;
    for (uint32_t i = tid; i < E; i += ROUTE_THREADS) a.items[i].x = -1;         // entries past the end of the new list
    if (tid < slots) {                      // slot p = t K + j in one flat array; anything that is not an expert id becomes -1
        const int32_t id = selected[tid / a.K][tid % a.K];
        flat[tid] = (id >= 0 && uint32_t(id) < E) ? id : -1;
    }
    __syncthreads();
    int32_t mine = -1, before = 0, rank = 0, count = 0;
    bool opener = false;
    if (tid < slots) {
        mine = flat[tid];
        if (mine >= 0) {
            for (uint32_t q = 0; q < slots; ++q) {
                const int32_t other = flat[q];
                before += other >= 0 && other < mine;
                count += other == mine;
                rank += (other == mine) && q < tid;
            }
            a.perm[before + rank] = int32_t(tid);
            opener = rank == 0 && uint32_t(mine) >= a.first_expert && uint32_t(mine) < a.first_expert + a.local_experts;
        }
    }
    if (tid < 256) opens[tid] = opener ? mine : -1;                             // the expert ids that open a work-list entry
    for (uint32_t e = tid; e <= E; e += ROUTE_THREADS) {                        // offsets[e] = slots routed to experts below e
        int32_t below = 0;
        for (uint32_t q = 0; q < slots; ++q) below += flat[q] >= 0 && uint32_t(flat[q]) < e;
        a.offsets[e] = below;
    }
    __syncthreads();
    if (opener) {
        int32_t entry = 0;
        for (uint32_t q = 0; q < slots; ++q) entry += opens[q] >= 0 && opens[q] < mine;
        a.active[entry] = mine;
        a.items[entry] = make_int4(mine, before, count, 0);
    }
    if (tid == 0) {
        int32_t entries = 0;
        for (uint32_t q = 0; q < slots; ++q) entries += opens[q] >= 0;
        a.counters[0] = entries; a.counters[16 + a.layer] = entries;
    }
}

// Route (one warp per token, eight tokens per CTA) and, when asked, the permutation as the tail of the
// last CTA to finish, so that a layer needs one launch for both. Dynamic shared memory: the eight score rows
// [8][E] floats, reused as the [8][E] histogram of the permutation.
// The permutation of a batch that one routing CTA covers (at most eight tokens, so at most 256 slots): the selections
// are still in shared memory, so each slot finds its place by counting - its expert's first position is the number of
// slots with a smaller expert id, its rank the number of earlier slots with the same id - and each expert's first slot
// writes the expert's entry of the work list. No histogram, no scan, no re-read of the ids from global memory, and no
// arrival counter; the result is the same stable counting sort.
__device__ __forceinline__ void permute_small(const RouteArgs& a, const int32_t (*selected)[32], int32_t* flags /* [256] shared */) {
    const uint32_t slots = a.T * a.K, E = a.E, tid = threadIdx.x;
    auto id_of = [&](uint32_t p) { return selected[p / a.K][p % a.K]; };
    for (uint32_t i = tid; i < E; i += ROUTE_THREADS) a.items[i].x = -1;         // entries past the end of the new list
    int32_t mine = -1, before = 0, rank = 0, count = 0;
    bool first = false, local = false;
    if (tid < slots) {
        mine = id_of(tid);
        if (mine >= 0 && uint32_t(mine) < E) {
            for (uint32_t q = 0; q < slots; ++q) {
                const int32_t other = id_of(q);
                if (other < 0 || uint32_t(other) >= E) continue;
                before += other < mine;
                count += other == mine;
                rank += (other == mine) && q < tid;
            }
            first = rank == 0;
            local = uint32_t(mine) >= a.first_expert && uint32_t(mine) < a.first_expert + a.local_experts;
            a.perm[before + rank] = int32_t(tid);
        }
    }
    if (tid < 256) flags[tid] = (first && local) ? mine : -1;                   // the expert ids that open a work-list entry
    // offsets[e] = slots routed to experts below e
    uint32_t valid = 0;
    for (uint32_t e = tid; e <= E; e += ROUTE_THREADS) {
        int32_t below = 0;
        for (uint32_t q = 0; q < slots; ++q) { const int32_t other = id_of(q); below += other >= 0 && uint32_t(other) < E && uint32_t(other) < e; }
        a.offsets[e] = below;
        if (e == E) valid = uint32_t(below);
    }
    (void)valid;
    __syncthreads();
    if (first && local) {
        int32_t entry = 0;
        for (uint32_t q = 0; q < slots; ++q) entry += flags[q] >= 0 && flags[q] < mine;
        a.active[entry] = mine;
        a.items[entry] = make_int4(mine, before, count, 0);
    }
    if (tid == 0) {
        int32_t entries = 0;
        for (uint32_t q = 0; q < slots; ++q) entries += flags[q] >= 0;
        a.counters[0] = entries; a.counters[16 + a.layer] = entries;
    }
}

// Route (one warp per token, eight tokens per CTA) and, when asked, the permutation as the tail of the
// last CTA to finish, so that a layer needs one launch for both. Dynamic shared memory: the eight score rows
// [8][E] floats, reused as the [8][E] histogram of the permutation.
template <int MAXC>
__global__ void __launch_bounds__(ROUTE_THREADS) route_kernel(RouteArgs a) {
    extern __shared__ int32_t hist[];
    __shared__ float scores[ROUTE_WARPS][32];
    __shared__ int32_t selected[ROUTE_WARPS][32];
    __shared__ int32_t flat[256], opens[256];
    __shared__ bool last;
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t t = blockIdx.x * ROUTE_WARPS + warp;
    pdl_wait();
    pdl_launch_dependents();
    if (t < a.T) route_token<MAXC>(a, t, lane, reinterpret_cast<float*>(hist) + warp * a.E, scores[warp], selected[warp]);
    if (!a.do_permute) return;
    if (gridDim.x == 1) {                   // this CTA routed every token: ROUTE_WARPS x K <= 256 slots
        __syncthreads();
        permute_small(a, selected, flat, opens);
        return;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(a.done, 1u) == gridDim.x - 1;
    {
        const uint32_t slots = a.T * a.K, range = permute_range(slots, ROUTE_WARPS), used = min(uint32_t(ROUTE_WARPS), (slots + range - 1) / max(range, 1u));
        for (uint32_t i = threadIdx.x; i < used * a.E; i += ROUTE_THREADS) hist[i] = 0;      // overlaps the atomic's round trip
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (threadIdx.x == 0) *a.done = 0;
    permute_any<ROUTE_THREADS>(a.ids, a.T * a.K, a.E, a.first_expert, a.local_experts, a.offsets, a.perm, a.active, a.items, a.counters, a.layer, a.status, hist);
}

}  // namespace

size_t permute_block_count(size_t slots) { return (slots + PERMUTE_BLOCK - 1) / PERMUTE_BLOCK; }

int launch_ep_receive_permute(zc_moe* m, const Call& q, cudaStream_t s) {
    const size_t slots = size_t(q.T) * q.K;
    if (slots > 4096 || q.E % 32 || q.E > 1024 || slots != size_t(m->ep_world) * m->ep_layout.cap) return 0;       // the caller issues the two launches
    static SmemOptIn configured;
    if (opt_in_smem(ep_receive_permute_kernel, configured, m->device, 160 * 1024) != cudaSuccess) return check_launch(m, "permute attribute");
    const size_t hist_bytes = size_t(PERMUTE_THREADS / 32) * q.E * sizeof(int32_t);
    Timed t(m, s, KERNEL_EP);
    const cudaError_t e = launch_chained(m, KERNEL_EP, ep_receive_permute_kernel, dim3(1), dim3(PERMUTE_THREADS), hist_bytes, s, nullptr, 0,
                                         ep_args(m), m->ep_row_ids, static_cast<uint32_t*>(m->ep_counts), uint32_t(slots), q.E, q.first_expert, q.local_experts,
                                         q.offsets, q.perm, q.active, q.items, q.counters, q.layer);
    if (e != cudaSuccess) return fail(m, ZC_EEXEC, std::string("ep receive launch: ") + cudaGetErrorString(e));
    const int rc = check_launch(m, "ep receive + permute");
    return rc < 0 ? rc : 1;
}

int launch_forced_weights(zc_moe* m, const Call& c, const int32_t* forced, cudaStream_t s) {
    if (c.K > 32) return fail(m, ZC_EINVAL, "route: top_k above 32");
    Timed t(m, s, KERNEL_ROUTE);
    forced_weights_kernel<<<(c.T + ROUTE_WARPS - 1) / ROUTE_WARPS, ROUTE_THREADS, 0, s>>>(c.logits, forced, c.ids, c.weights, c.T, c.E, c.K, c.status);
    const int rc = check_launch(m, "forced route weights");
    return rc < 0 ? rc : 1;
}

int launch_route_permute(zc_moe* m, const Call& c, cudaStream_t s, bool do_route, bool do_permute) {
    int launched = 0;
    if (c.E % 32 || c.E > 1024) return fail(m, ZC_EINVAL, "route: experts must be a multiple of 32, at most 1024");
    if (c.K > 32) return fail(m, ZC_EINVAL, "route: top_k above 32");
    const size_t hist_bytes = size_t(PERMUTE_THREADS / 32) * c.E * sizeof(int32_t);
    // Long batches: the permutation runs as its own launch of 1024 threads instead of as the tail of one 256-thread
    // routing CTA (20480 slots at 2048 tokens).
    const bool separate = do_route && do_permute && size_t(c.T) * c.K > 4096;
    if (separate) do_permute = false;
    if (do_route) {
        RouteArgs a{};
        a.logits = c.logits;
        a.ids = c.ids; a.weights = c.weights; a.T = c.T; a.E = c.E; a.K = c.K; a.status = c.status;
        a.offsets = c.offsets; a.perm = c.perm; a.active = c.active; a.items = c.items; a.counters = c.counters; a.done = reinterpret_cast<uint32_t*>(c.counters + 1);
        a.first_expert = c.first_expert; a.local_experts = c.local_experts; a.layer = c.layer; a.do_permute = do_permute;
        const size_t smem = size_t(ROUTE_THREADS / 32) * c.E * sizeof(int32_t);
        const bool small = c.E <= 512;
        static SmemOptIn configured[2];
        {
            const cudaError_t e = small ? opt_in_smem(route_kernel<16>, configured[1], m->device, smem)
                                        : opt_in_smem(route_kernel<32>, configured[0], m->device, smem);
            if (e != cudaSuccess) return check_launch(m, "route attribute");
        }
        const uint32_t grid = (c.T + ROUTE_WARPS - 1) / ROUTE_WARPS;
        int rc;
        {
            Timed t(m, s, KERNEL_ROUTE);
            const cudaError_t e = small ? launch_chained(m, KERNEL_ROUTE, route_kernel<16>, dim3(grid), dim3(ROUTE_THREADS), smem, s, nullptr, 0, a)
                                        : launch_chained(m, KERNEL_ROUTE, route_kernel<32>, dim3(grid), dim3(ROUTE_THREADS), smem, s, nullptr, 0, a);
            if (e != cudaSuccess) return fail(m, ZC_EEXEC, std::string("route launch: ") + cudaGetErrorString(e));
            rc = check_launch(m, "route");
        }
        if (rc < 0) return rc;
        ++launched;
    }
    if ((separate || (!do_route && do_permute)) && size_t(c.T) * c.K > 4096 && m->permute_blocks) {
        const uint32_t slots = c.T * c.K, nblocks = uint32_t(permute_block_count(slots));
        static SmemOptIn configured;
        if (opt_in_smem(permute_place_kernel, configured, m->device, 160 * 1024) != cudaSuccess) return check_launch(m, "permute attribute");
        int rc;
        {
            Timed t(m, s, KERNEL_PERMUTE);
            permute_count_kernel<<<nblocks, PERMUTE_THREADS, c.E * sizeof(int32_t), s>>>(c.ids, slots, c.E, m->permute_blocks, c.quiet_drop ? nullptr : c.status);
            permute_scan_kernel<<<1, PERMUTE_THREADS, 0, s>>>(m->permute_blocks, nblocks, c.E, c.first_expert, c.local_experts, c.offsets, c.active, c.items, c.counters, c.layer);
            permute_place_kernel<<<nblocks, PERMUTE_THREADS, hist_bytes, s>>>(c.ids, slots, c.E, m->permute_blocks, c.offsets, c.perm);
            rc = check_launch(m, "permute");
        }
        if (rc < 0) return rc;
        launched += 3;
    } else if (separate || (!do_route && do_permute)) {
        static SmemOptIn configured;
        if (opt_in_smem(permute_kernel, configured, m->device, 160 * 1024) != cudaSuccess) return check_launch(m, "permute attribute");
        int rc;
        {
            Timed t(m, s, KERNEL_PERMUTE);
            permute_kernel<<<1, PERMUTE_THREADS, hist_bytes, s>>>(c.ids, c.T * c.K, c.E, c.first_expert, c.local_experts, c.offsets, c.perm,
                                                                 c.active, c.items, c.counters, c.layer, c.quiet_drop ? nullptr : c.status);
            rc = check_launch(m, "permute");
        }
        if (rc < 0) return rc;
        ++launched;
    }
    return launched;
}

}  // namespace zc
