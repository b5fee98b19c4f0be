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

constexpr int ROUTE_WARPS = 8;
constexpr int MAX_CAND = 32;   // experts / 32 per lane, experts <= 1024

__global__ void __launch_bounds__(ROUTE_WARPS * 32) route_kernel(const float* __restrict__ logits, uint32_t T, uint32_t E,
                                                                  uint32_t K, int32_t* __restrict__ ids,
                                                                  float* __restrict__ weights, uint32_t* status) {
    __shared__ float scores[ROUTE_WARPS][32];
    __shared__ int32_t selected[ROUTE_WARPS][32];
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= T) return;
    const float* row = logits + size_t(t) * E;
    const uint32_t nc = E / 32;
    const float ninf = __int_as_float(0xff800000);
    float cand[MAX_CAND];
#pragma unroll
    for (int i = 0; i < MAX_CAND; ++i) cand[i] = uint32_t(i) < nc ? row[lane + 32 * i] : ninf;
    for (uint32_t j = 0; j < K; ++j) {
        float best = ninf;
        uint32_t index = E;
#pragma unroll
        for (int i = 0; i < MAX_CAND; ++i) if (cand[i] > best) { best = cand[i]; index = lane + 32 * i; }
        float maximum = best;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, off));
        uint32_t winner = best == maximum ? index : E;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) winner = min(winner, __shfl_xor_sync(0xffffffffu, winner, off));
        if (lane == 0) {
            selected[warp][j] = winner < E ? int32_t(winner) : -1;
            scores[warp][j] = winner < E ? row[winner] : ninf;
        }
#pragma unroll
        for (int i = 0; i < MAX_CAND; ++i) if (lane + 32 * i == winner) cand[i] = ninf;
    }
    __syncwarp();
    float values[4], sum = 0.0f;
    const float top = scores[warp][0];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t j = lane * 4 + i;
        values[i] = j < K ? expf(scores[warp][j < 32 ? j : 0] - top) : 0.0f;
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
            const int32_t id = selected[warp][j];
            ids[size_t(t) * K + j] = id;
            weights[size_t(t) * K + j] = __fmul_rn(values[i], inverse);
            bad |= id < 0;
        }
    }
    if (bad) atomicOr(status, ZC_STATUS_INVALID_ROUTE);
}

constexpr int PERMUTE_THREADS = 1024;
constexpr int PERMUTE_WARPS = PERMUTE_THREADS / 32;

// Exclusive scan of one value per thread over the whole CTA; returns the exclusive prefix and the total.
__device__ __forceinline__ int block_exclusive_scan(int value, int* warp_totals, int& total) {
    const uint32_t lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    int inclusive = value;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inclusive, off);
        if (lane >= uint32_t(off)) inclusive += n;
    }
    if (lane == 31) warp_totals[warp] = inclusive;
    __syncthreads();
    if (warp == 0) {
        int w = warp_totals[lane];
        int inc = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= uint32_t(off)) inc += n;
        }
        warp_totals[lane] = inc - w;              // exclusive prefix of the warp totals
        if (lane == 31) warp_totals[32] = inc;    // grand total
    }
    __syncthreads();
    total = warp_totals[32];
    const int result = warp_totals[warp] + inclusive - value;
    __syncthreads();
    return result;
}

__global__ void __launch_bounds__(PERMUTE_THREADS) permute_kernel(const int32_t* __restrict__ ids, uint32_t slots, uint32_t E,
                                                                   uint32_t first_expert, uint32_t local_experts,
                                                                   int32_t* __restrict__ offsets, int32_t* __restrict__ perm,
                                                                   int32_t* __restrict__ active, int32_t* __restrict__ counters,
                                                                   uint32_t layer, uint32_t* status) {
    extern __shared__ int32_t hist[];                 // [PERMUTE_WARPS][E] per-warp counts, then cursors
    __shared__ int warp_totals[33];
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    for (uint32_t i = threadIdx.x; i < PERMUTE_WARPS * E; i += PERMUTE_THREADS) hist[i] = 0;
    __syncthreads();
    // Contiguous slot range of this warp, a multiple of 32 long so that chunks stay aligned.
    const uint32_t range = ((slots + PERMUTE_WARPS - 1) / PERMUTE_WARPS + 31) / 32 * 32;
    const uint32_t begin = warp * range, end = min(slots, begin + range);
    int32_t* mine = hist + warp * E;
    bool bad = false;
    for (uint32_t base = begin; base < end; base += 32) {
        const uint32_t p = base + lane;
        int32_t id = p < end ? ids[p] : -1;
        const bool valid = id >= 0 && uint32_t(id) < E;
        bad |= p < end && !valid;
        const uint32_t key = valid ? uint32_t(id) : E + lane;     // invalid lanes match nobody
        const uint32_t peers = __match_any_sync(0xffffffffu, key);
        if (valid && (peers & ((1u << lane) - 1)) == 0) mine[id] += __popc(peers);
        __syncwarp();
    }
    if (bad) atomicOr(status, ZC_STATUS_INVALID_ROUTE);
    __syncthreads();
    // Per expert: turn the per-warp counts into per-warp starting ranks; total = expert count.
    int count = 0;
    if (threadIdx.x < E) {
        for (int w = 0; w < PERMUTE_WARPS; ++w) {
            const int n = hist[w * E + threadIdx.x];
            hist[w * E + threadIdx.x] = count;
            count += n;
        }
    }
    int total;
    const int offset = block_exclusive_scan(count, warp_totals, total);
    if (threadIdx.x < E) {
        offsets[threadIdx.x] = offset;
        for (int w = 0; w < PERMUTE_WARPS; ++w) hist[w * E + threadIdx.x] += offset;
    }
    if (threadIdx.x == 0) offsets[E] = total;
    // Ascending list of locally held experts that received work.
    const bool local = threadIdx.x >= first_expert && threadIdx.x < first_expert + local_experts;
    const int has_work = threadIdx.x < E && local && count > 0;
    int n_active;
    const int slot = block_exclusive_scan(has_work, warp_totals, n_active);
    if (has_work) active[slot] = int32_t(threadIdx.x);
    if (threadIdx.x == 0) { counters[0] = n_active; counters[16 + layer] = n_active; }
    __syncthreads();
    for (uint32_t base = begin; base < end; base += 32) {
        const uint32_t p = base + lane;
        int32_t id = p < end ? ids[p] : -1;
        const bool valid = id >= 0 && uint32_t(id) < E;
        const uint32_t key = valid ? uint32_t(id) : E + lane;
        const uint32_t peers = __match_any_sync(0xffffffffu, key);
        const uint32_t before = peers & ((1u << lane) - 1);
        int cursor = 0;
        if (valid) cursor = mine[id];
        __syncwarp();
        if (valid) {
            perm[cursor + __popc(before)] = int32_t(p);
            if (before == 0) mine[id] = cursor + __popc(peers);
        }
        __syncwarp();
    }
}

}  // namespace

int launch_route_permute(zc_moe* m, const Call& c, cudaStream_t s, bool do_route, bool do_permute) {
    int launched = 0;
    if (do_route) {
        int rc;
        { Timed t(m, s, KERNEL_ROUTE); route_kernel<<<(c.T + ROUTE_WARPS - 1) / ROUTE_WARPS, ROUTE_WARPS * 32, 0, s>>>(c.logits, c.T, c.E, c.K, c.ids, c.weights, c.status); rc = check_launch(m, "route"); }
        if (rc < 0) return rc;
        ++launched;
    }
    if (do_permute) {
        const size_t smem = size_t(PERMUTE_WARPS) * c.E * sizeof(int32_t);
        static bool configured = false;
        if (!configured) {
            cudaFuncSetAttribute(permute_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            configured = true;
        }
        int rc;
        { Timed t(m, s, KERNEL_PERMUTE);
          permute_kernel<<<1, PERMUTE_THREADS, smem, s>>>(c.ids, c.T * c.K, c.E, c.first_expert, c.local_experts, c.offsets, c.perm,
                                                         c.active, c.counters, c.layer, c.status);
          rc = check_launch(m, "permute"); }
        if (rc < 0) return rc;
        ++launched;
    }
    return launched;
}

}  // namespace zc
