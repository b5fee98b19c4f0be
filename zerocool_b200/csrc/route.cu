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
    const float* logits_in;     // [T, E] when the logits already exist
    const float* partial;       // [16, T, rows_padded] router partials, or null
    float* logits_out;          // [T, E], written when reading partials
    float* gate_logit;          // [T], written when reading partials and the layer has a shared expert
    int32_t* ids; float* weights;
    uint32_t T, E, K, rows_padded, has_shared;
    uint32_t* status;
    // permutation tail (run by the last CTA to finish when do_permute is set)
    int32_t* offsets; int32_t* perm; int32_t* active; int32_t* counters; uint32_t* done;
    uint32_t first_expert, local_experts, layer, do_permute;
};

// One warp per token.
template <int MAXC>
__device__ __forceinline__ void route_token(const RouteArgs& a, uint32_t t, uint32_t lane, float* scores, int32_t* selected) {
    const uint32_t E = a.E, K = a.K, nc = E / 32;
    const float ninf = __int_as_float(0xff800000);
    float cand[MAXC];
    if (a.partial) {
        // ordered sum of the sixteen router partials, starting from zero (qwen.metal:529-534)
#pragma unroll
        for (int i = 0; i < MAXC; ++i) {
            float sum = ninf;
            if (uint32_t(i) < nc) {
                sum = 0.0f;
#pragma unroll
                for (uint32_t p = 0; p < 16; ++p) sum = __fadd_rn(sum, __ldcg(a.partial + (size_t(p) * a.T + t) * a.rows_padded + lane + 32 * i));
                a.logits_out[size_t(t) * E + lane + 32 * i] = sum;
            }
            cand[i] = sum;
        }
        if (a.has_shared && lane == 0) {
            float sum = 0.0f;
#pragma unroll
            for (uint32_t p = 0; p < 16; ++p) sum = __fadd_rn(sum, __ldcg(a.partial + (size_t(p) * a.T + t) * a.rows_padded + E));
            a.gate_logit[t] = sum;
        }
    } else {
        const float* row = a.logits_in + size_t(t) * E;
#pragma unroll
        for (int i = 0; i < MAXC; ++i) cand[i] = uint32_t(i) < nc ? row[lane + 32 * i] : ninf;
    }
    for (uint32_t j = 0; j < K; ++j) {
        float best = ninf;
        uint32_t index = E;
#pragma unroll
        for (int i = 0; i < MAXC; ++i) if (cand[i] > best) { best = cand[i]; index = lane + 32 * i; }
        float maximum = best;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, off));
        uint32_t winner = best == maximum ? index : E;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) winner = min(winner, __shfl_xor_sync(0xffffffffu, winner, off));
        // The winner's own value (keeps signed zero, like the reference's re-read of the logit).
        float mine = ninf;
#pragma unroll
        for (int i = 0; i < MAXC; ++i) if (lane + 32 * i == winner) { mine = cand[i]; cand[i] = ninf; }
        const float score = __shfl_sync(0xffffffffu, mine, winner & 31);
        if (lane == 0) {
            selected[j] = winner < E ? int32_t(winner) : -1;
            scores[j] = winner < E ? score : ninf;
        }
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

constexpr int PERMUTE_THREADS = 1024;

// Exclusive scan of one value per thread over a CTA of NT threads; returns the exclusive prefix and the total.
template <int NT>
__device__ __forceinline__ int block_exclusive_scan(int value, int* warp_totals, int& total) {
    constexpr int NW = NT / 32;
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
        int w = lane < NW ? warp_totals[lane] : 0;
        int inc = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= uint32_t(off)) inc += n;
        }
        if (lane < NW) warp_totals[lane] = inc - w;   // exclusive prefix of the warp totals
        if (lane == 31) warp_totals[32] = inc;        // grand total
    }
    __syncthreads();
    total = warp_totals[32];
    const int result = warp_totals[warp] + inclusive - value;
    __syncthreads();
    return result;
}

// Stable counting sort of the slots by expert id by one CTA of NT threads (hist: [NT/32][E] ints).
template <int NT>
__device__ __forceinline__ void permute_body(const int32_t* ids, uint32_t slots, uint32_t E,
                                             uint32_t first_expert, uint32_t local_experts,
                                             int32_t* __restrict__ offsets, int32_t* __restrict__ perm,
                                             int32_t* __restrict__ active, int32_t* __restrict__ counters,
                                             uint32_t layer, uint32_t* status, int32_t* hist) {
    constexpr int NW = NT / 32;
    __shared__ int warp_totals[33];
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    for (uint32_t i = threadIdx.x; i < NW * E; i += NT) hist[i] = 0;
    __syncthreads();
    // Contiguous slot range of this warp, a multiple of 32 long so that chunks stay aligned.
    const uint32_t range = ((slots + NW - 1) / NW + 31) / 32 * 32;
    const uint32_t begin = min(slots, warp * range), end = min(slots, begin + range);
    int32_t* mine = hist + warp * E;
    bool bad = false;
    for (uint32_t base = begin; base < end; base += 32) {
        const uint32_t p = base + lane;
        int32_t id = p < end ? __ldcg(ids + p) : -1;
        const bool valid = id >= 0 && uint32_t(id) < E;
        bad |= p < end && !valid;
        const uint32_t key = valid ? uint32_t(id) : E + lane;     // invalid lanes match nobody
        const uint32_t peers = __match_any_sync(0xffffffffu, key);
        if (valid && (peers & ((1u << lane) - 1)) == 0) mine[id] += __popc(peers);
        __syncwarp();
    }
    if (bad) atomicOr(status, ZC_STATUS_INVALID_ROUTE);
    __syncthreads();
    // Experts in passes of NT: per-warp counts become per-warp starting ranks; running offset carried across passes.
    int carry = 0, carry_active = 0;
    for (uint32_t e0 = 0; e0 < E; e0 += NT) {
        const uint32_t e = e0 + threadIdx.x;
        int count = 0;
        if (e < E) {
            for (int w = 0; w < NW; ++w) {
                const int n = hist[w * E + e];
                hist[w * E + e] = count;
                count += n;
            }
        }
        int total;
        const int offset = carry + block_exclusive_scan<NT>(count, warp_totals, total);
        if (e < E) {
            offsets[e] = offset;
            for (int w = 0; w < NW; ++w) hist[w * E + e] += offset;
        }
        carry += total;
        // Ascending list of locally held experts that received work.
        const int has_work = e < E && e >= first_expert && e < first_expert + local_experts && count > 0;
        int n_active;
        const int slot = carry_active + block_exclusive_scan<NT>(has_work, warp_totals, n_active);
        if (has_work) active[slot] = int32_t(e);
        carry_active += n_active;
    }
    if (threadIdx.x == 0) { offsets[E] = carry; counters[0] = carry_active; counters[16 + layer] = carry_active; }
    __syncthreads();
    for (uint32_t base = begin; base < end; base += 32) {
        const uint32_t p = base + lane;
        int32_t id = p < end ? __ldcg(ids + p) : -1;
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

__global__ void __launch_bounds__(PERMUTE_THREADS) permute_kernel(const int32_t* __restrict__ ids, uint32_t slots, uint32_t E,
                                                                   uint32_t first_expert, uint32_t local_experts,
                                                                   int32_t* __restrict__ offsets, int32_t* __restrict__ perm,
                                                                   int32_t* __restrict__ active, int32_t* __restrict__ counters,
                                                                   uint32_t layer, uint32_t* status) {
    extern __shared__ int32_t hist[];
    permute_body<PERMUTE_THREADS>(ids, slots, E, first_expert, local_experts, offsets, perm, active, counters, layer, status, hist);
}

// Route (one warp per token, eight tokens per CTA) and, when asked, the permutation as the tail of the
// last CTA to finish, so that a layer needs one launch for both.
template <int MAXC>
__global__ void __launch_bounds__(ROUTE_THREADS) route_kernel(RouteArgs a) {
    extern __shared__ int32_t hist[];
    __shared__ float scores[ROUTE_WARPS][32];
    __shared__ int32_t selected[ROUTE_WARPS][32];
    __shared__ bool last;
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t t = blockIdx.x * ROUTE_WARPS + warp;
    if (t < a.T) route_token<MAXC>(a, t, lane, scores[warp], selected[warp]);
    if (!a.do_permute) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(a.done, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (threadIdx.x == 0) *a.done = 0;
    permute_body<ROUTE_THREADS>(a.ids, a.T * a.K, a.E, a.first_expert, a.local_experts, a.offsets, a.perm, a.active, a.counters, a.layer, a.status, hist);
}

}  // namespace

// do_route with partials: the router's [16, T, rows] partial sums are reduced in order on the fly.
int launch_route_permute(zc_moe* m, const Call& c, cudaStream_t s, bool do_route, bool do_permute, bool from_partials) {
    int launched = 0;
    const size_t hist_bytes = size_t(PERMUTE_THREADS / 32) * c.E * sizeof(int32_t);
    if (do_route) {
        RouteArgs a{};
        a.logits_in = c.logits; a.partial = from_partials ? m->router_partial : nullptr; a.logits_out = c.logits; a.gate_logit = c.gate_logit;
        a.ids = c.ids; a.weights = c.weights; a.T = c.T; a.E = c.E; a.K = c.K; a.rows_padded = router_rows_padded(m->d);
        a.has_shared = c.has_shared; a.status = c.status;
        a.offsets = c.offsets; a.perm = c.perm; a.active = c.active; a.counters = c.counters; a.done = reinterpret_cast<uint32_t*>(c.counters + 1);
        a.first_expert = c.first_expert; a.local_experts = c.local_experts; a.layer = c.layer; a.do_permute = do_permute;
        const size_t smem = do_permute ? size_t(ROUTE_THREADS / 32) * c.E * sizeof(int32_t) : 0;
        const bool small = c.E <= 512;
        static size_t configured[2] = {0, 0};
        if (smem > configured[small]) {
            cudaError_t e = small ? cudaFuncSetAttribute(route_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem))
                                  : cudaFuncSetAttribute(route_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
            if (e != cudaSuccess) return check_launch(m, "route attribute");
            configured[small] = smem;
        }
        const uint32_t grid = (c.T + ROUTE_WARPS - 1) / ROUTE_WARPS;
        int rc;
        {
            Timed t(m, s, KERNEL_ROUTE);
            if (small) route_kernel<16><<<grid, ROUTE_THREADS, smem, s>>>(a);
            else route_kernel<32><<<grid, ROUTE_THREADS, smem, s>>>(a);
            rc = check_launch(m, "route");
        }
        if (rc < 0) return rc;
        ++launched;
    } else if (do_permute) {
        static bool configured = false;
        if (!configured) {
            cudaFuncSetAttribute(permute_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            configured = true;
        }
        int rc;
        {
            Timed t(m, s, KERNEL_PERMUTE);
            permute_kernel<<<1, PERMUTE_THREADS, hist_bytes, s>>>(c.ids, c.T * c.K, c.E, c.first_expert, c.local_experts, c.offsets, c.perm,
                                                                 c.active, c.counters, c.layer, c.status);
            rc = check_launch(m, "permute");
        }
        if (rc < 0) return rc;
        ++launched;
    }
    return launched;
}

}  // namespace zc
