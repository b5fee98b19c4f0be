// Expert parallelism: the device-side pieces around the all-to-all exchange.
//
// The reference is a single-GPU engine and has no counterpart. Experts are sharded over ranks in
// contiguous ranges (rank r holds experts [r*E/N, (r+1)*E/N) of every layer); tokens start data
// parallel. Per layer, on each rank:
//   dispatch : router + route + permutation of the local tokens over ALL experts, then the token rows
//              are gathered in expert order — rows for one owner rank are contiguous, so the exchange
//              is one all-to-all with split sizes read from the permutation's offsets;
//   experts  : the rows received from all ranks, each tagged with its expert id, run through the
//              grouped expert kernels (a permutation with one slot per row regroups them by expert);
//   combine  : the results, returned by the reverse all-to-all in the order they were sent, are
//              scattered to their router slots and reduced in fixed slot order with the locally
//              computed shared expert — so the result does not depend on arrival order.
#include "common.cuh"

namespace zc {
namespace {

// rows[i, :] = x[perm[i] / K, :] (16-byte pieces), row_experts[i] = ids[perm[i]], for i < offsets[E].
__global__ void ep_gather_kernel(const void* __restrict__ x, uint32_t row_bytes, const int32_t* __restrict__ perm, const int32_t* __restrict__ ids,
                                 const int32_t* __restrict__ offsets, uint32_t E, uint32_t K, void* __restrict__ rows, int32_t* __restrict__ row_experts) {
    const uint32_t i = blockIdx.x;
    if (i >= uint32_t(offsets[E])) return;
    const uint32_t slot = uint32_t(perm[i]);
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(x) + size_t(slot / K) * row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(rows) + size_t(i) * row_bytes);
    for (uint32_t j = threadIdx.x; j < row_bytes / 16; j += blockDim.x) dst[j] = src[j];
    if (threadIdx.x == 0) row_experts[i] = ids[slot];
}

// expert_out[perm[i], :] = y[i, :] for i < offsets[E].
__global__ void ep_scatter_kernel(const float* __restrict__ y, const int32_t* __restrict__ perm, const int32_t* __restrict__ offsets, uint32_t E,
                                  uint32_t H, float* __restrict__ expert_out) {
    const uint32_t i = blockIdx.x;
    if (i >= uint32_t(offsets[E])) return;
    const float4* src = reinterpret_cast<const float4*>(y + size_t(i) * H);
    float4* dst = reinterpret_cast<float4*>(expert_out + size_t(uint32_t(perm[i])) * H);
    for (uint32_t j = threadIdx.x; j < H / 4; j += blockDim.x) dst[j] = src[j];
}

}  // namespace

int launch_ep_gather(zc_moe* m, const Call& c, void* rows, int32_t* row_experts, cudaStream_t s) {
    const uint32_t row_bytes = c.H * (c.act_dtype == ZC_F32 ? 4 : 2);
    ep_gather_kernel<<<c.T * c.K, 128, 0, s>>>(c.x, row_bytes, c.perm, c.ids, c.offsets, c.E, c.K, rows, row_experts);
    int rc = check_launch(m, "ep gather");
    return rc < 0 ? rc : 1;
}

int launch_ep_scatter(zc_moe* m, const Call& c, const float* y, cudaStream_t s) {
    ep_scatter_kernel<<<c.T * c.K, 128, 0, s>>>(y, c.perm, c.offsets, c.E, c.H, c.expert_out);
    int rc = check_launch(m, "ep scatter");
    return rc < 0 ? rc : 1;
}

}  // namespace zc
