// Expert parallelism: the device-side pieces around the exchange of token rows between ranks.
//
// The reference is a single-GPU engine and has no counterpart. Experts are sharded over ranks in
// contiguous ranges (rank r holds experts [r*E/N, (r+1)*E/N) of every layer); tokens start data
// parallel. Per layer, on each rank:
//   dispatch : router + route + permutation of the local tokens over ALL experts, then the token rows
//              leave in expert order, so rows for one owner rank are contiguous;
//   experts  : the rows received from all ranks, each tagged with its expert id, run through the
//              grouped expert kernels (a permutation with one slot per row regroups them by expert);
//   combine  : the results come back to the router slots of the rank that sent the rows and are reduced
//              there in fixed slot order with the locally computed shared expert — so the result does
//              not depend on arrival order.
//
// Two transports share these steps.
//  * Library all-to-all (zc_moe_ep_dispatch / _experts / _combine): gather into a send buffer, the caller
//    exchanges rows and ids with a collective whose split sizes it reads from the permutation offsets.
//  * Peer stores (zc_moe_ep_layer, zc_moe_ep_stack): every rank owns a "window" of device memory that all
//    ranks of the node map (NVLink peer access). The send kernel stores each row straight into the owner's
//    window with plain 16-byte st.global, then publishes {epoch, row count} to the owner with one
//    release store per owner. The owner waits for all sources' flags (bounded, see ep_wait below), runs
//    its experts on the rows in place, stores every result row into the sender's window at its router slot
//    and publishes a return flag. No host value is needed anywhere, so the whole layer - and a whole stack
//    of layers - is one stream of launches that can be captured in a CUDA graph. Only plain loads and
//    stores and scalar release/acquire operations touch peer memory: no TMA, no multicast.
//
// Protocol invariants (why no buffer is overwritten while it is still read):
//   - a rank sends layer l+1 only after its combine of layer l, which waited for the return flag of every
//     owner, and an owner publishes its return flag only after its expert kernels have consumed all
//     received rows: so the receive area of an owner is free when the next rows arrive;
//   - an owner stores results of layer l+1 into a sender's window only after it has seen that sender's
//     send flag of layer l+1, which the sender publishes after its combine of layer l has read the
//     previous results.
//   Every rank must issue the same sequence of expert-parallel layer calls (the epoch counts them).
#include "common.cuh"

namespace zc {

EpWindow ep_window_layout(const zc_moe_desc& d) {
    EpWindow w{};
    const uint32_t local = d.local_experts ? d.local_experts : d.experts;
    w.world = (d.experts + local - 1) / local;
    w.cap = d.max_tokens * d.top_k;
    const uint64_t row_bytes = uint64_t(d.hidden) * (d.act_dtype == ZC_F32 ? 4 : 2);
    auto take = [&](uint64_t bytes) { const uint64_t at = w.bytes; w.bytes += (bytes + 255) / 256 * 256; return at; };
    w.rows = take(uint64_t(w.world) * w.cap * row_bytes);
    w.tags = take(uint64_t(w.world) * w.cap * sizeof(int2));
    w.in_flags = take(uint64_t(EP_MAX_RANKS) * 8);
    w.ret_flags = take(uint64_t(EP_MAX_RANKS) * 8);
    w.out = take(uint64_t(w.cap) * d.hidden * 4);
    return w;
}

namespace {

constexpr int EP_THREADS = 128;

// Last-block election: every thread's stores are fenced at system scope, then one arrival per block.
__device__ __forceinline__ bool ep_last_block(uint32_t* counter) {
    __shared__ bool last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(counter, 1u) == gridDim.x - 1;
    __syncthreads();
    return last;
}

// Position i of the expert-sorted slot list -> the owner's window: row, {expert, router slot} tag. The last
// block to finish publishes {epoch, rows for that owner} to every owner.
__global__ void __launch_bounds__(EP_THREADS) ep_send_kernel(EpArgs a, const void* __restrict__ x, uint32_t row_bytes, const int32_t* __restrict__ perm,
                                                             const int32_t* __restrict__ ids, const int32_t* __restrict__ offsets, uint32_t E, uint32_t K) {
    pdl_wait();                             // the routing kernel's lists
    pdl_launch_dependents();
    const uint32_t i = blockIdx.x, total = uint32_t(offsets[E]);
    if (i < total) {
        const uint32_t slot = uint32_t(perm[i]);
        const int32_t e = ids[slot];
        const uint32_t owner = uint32_t(e) / a.per;
        if (e >= 0 && owner < a.world) {
            const uint32_t j = i - uint32_t(offsets[owner * a.per]);
            if (j < a.win.cap) {
                uint8_t* base = a.peers.base[owner];
                const size_t at = size_t(a.me) * a.win.cap + j;
                const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(x) + size_t(slot / K) * row_bytes);
                uint4* dst = reinterpret_cast<uint4*>(base + a.win.rows + at * row_bytes);
                for (uint32_t q = threadIdx.x; q < row_bytes / 16; q += EP_THREADS) dst[q] = src[q];
                if (threadIdx.x == 0) reinterpret_cast<int2*>(base + a.win.tags)[at] = make_int2(e, int(slot));
            }
        }
    }
    if (!ep_last_block(a.ctl + 1)) return;
    __shared__ uint32_t epoch_s;
    if (threadIdx.x == 0) { epoch_s = a.ctl[0] + 1; a.ctl[0] = epoch_s; a.ctl[1] = 0; }
    __syncthreads();
    if (threadIdx.x < a.world) {
        const uint32_t r = threadIdx.x;
        const uint32_t count = min(uint32_t(offsets[(r + 1) * a.per] - offsets[r * a.per]), a.win.cap);
        __threadfence_system();
        st_release_sys(reinterpret_cast<unsigned long long*>(a.peers.base[r] + a.win.in_flags) + a.me, (unsigned long long)(epoch_s) << 32 | count);
    }
}

// Owner side: waits for every source's flag of the current epoch, then writes the expert id of every row slot
// of the receive area (-1 for slots beyond a source's count, and for ids outside this rank's range).
__global__ void __launch_bounds__(1024) ep_receive_kernel(EpArgs a, int32_t* __restrict__ row_ids, uint32_t* __restrict__ counts) {
    __shared__ uint32_t count_s[EP_MAX_RANKS];
    ep_receive_body(a, row_ids, counts, count_s);
}

// Owner side: result row i of the receive area -> the sender's window at the row's router slot. The last block
// publishes the return flag to every sender.
__global__ void __launch_bounds__(EP_THREADS) ep_return_kernel(EpArgs a, const float* __restrict__ y, const uint32_t* __restrict__ counts, uint32_t H) {
    pdl_wait();                             // the down kernel's result rows
    pdl_launch_dependents();
    const uint32_t i = blockIdx.x, src = i / a.win.cap, j = i % a.win.cap;
    const uint8_t* mine = a.peers.base[a.me];
    if (src < a.world && j < counts[src]) {
        const int2 tag = __ldcg(reinterpret_cast<const int2*>(mine + a.win.tags) + i);
        if (uint32_t(tag.y) < a.win.cap) {
            const float4* from = reinterpret_cast<const float4*>(y + size_t(i) * H);
            float4* to = reinterpret_cast<float4*>(a.peers.base[src] + a.win.out + size_t(uint32_t(tag.y)) * H * 4);
            for (uint32_t q = threadIdx.x; q < H / 4; q += EP_THREADS) to[q] = __ldcg(from + q);
        }
    }
    if (!ep_last_block(a.ctl + 2)) return;
    if (threadIdx.x == 0) a.ctl[2] = 0;
    if (threadIdx.x < a.world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<unsigned long long*>(a.peers.base[threadIdx.x] + a.win.ret_flags) + a.me, (unsigned long long)(a.ctl[0]) << 32);
    }
}

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

EpArgs ep_args(const zc_moe* m) {
    EpArgs a{};
    a.peers = m->ep_peers; a.win = m->ep_layout; a.me = m->ep_rank; a.world = m->ep_world; a.per = m->d.local_experts;
    a.ctl = m->ep_ctl; a.status = m->scratch.status; a.wait_ns = (unsigned long long)(m->ep_wait_ms) * 1000000ull;
    return a;
}

int launch_ep_gather(zc_moe* m, const Call& c, void* rows, int32_t* row_experts, cudaStream_t s) {
    const uint32_t row_bytes = c.H * (c.act_dtype == ZC_F32 ? 4 : 2);
    Timed t(m, s, KERNEL_EP);
    ep_gather_kernel<<<c.T * c.K, 128, 0, s>>>(c.x, row_bytes, c.perm, c.ids, c.offsets, c.E, c.K, rows, row_experts);
    int rc = check_launch(m, "ep gather");
    return rc < 0 ? rc : 1;
}

int launch_ep_scatter(zc_moe* m, const Call& c, const float* y, cudaStream_t s) {
    Timed t(m, s, KERNEL_EP);
    ep_scatter_kernel<<<c.T * c.K, 128, 0, s>>>(y, c.perm, c.offsets, c.E, c.H, c.expert_out);
    int rc = check_launch(m, "ep scatter");
    return rc < 0 ? rc : 1;
}

int launch_ep_send(zc_moe* m, const Call& c, cudaStream_t s) {
    const uint32_t row_bytes = c.H * (c.act_dtype == ZC_F32 ? 4 : 2);
    Timed t(m, s, KERNEL_EP);
    // The exchange kernels are links of the layer's launch chain like the others (see launch_chained): set-up overlaps the
    // tail of the kernel before, and a kernel that waits for a peer does so after its own grid-dependency wait.
    const cudaError_t e = launch_chained(m, KERNEL_EP, ep_send_kernel, dim3(c.T * c.K), dim3(EP_THREADS), 0, s, nullptr, 0,
                                         ep_args(m), c.x, row_bytes, c.perm, c.ids, c.offsets, c.E, c.K);
    if (e != cudaSuccess) return fail(m, ZC_EEXEC, std::string("ep send launch: ") + cudaGetErrorString(e));
    int rc = check_launch(m, "ep send");
    return rc < 0 ? rc : 1;
}

int launch_ep_receive(zc_moe* m, cudaStream_t s) {
    Timed t(m, s, KERNEL_EP);
    ep_receive_kernel<<<1, 1024, 0, s>>>(ep_args(m), m->ep_row_ids, m->ep_counts);
    int rc = check_launch(m, "ep receive");
    return rc < 0 ? rc : 1;
}

int launch_ep_return(zc_moe* m, cudaStream_t s) {
    Timed t(m, s, KERNEL_EP);
    const cudaError_t e = launch_chained(m, KERNEL_EP, ep_return_kernel, dim3(m->ep_world * m->ep_layout.cap), dim3(EP_THREADS), 0, s, nullptr, 0,
                                         ep_args(m), static_cast<const float*>(m->ep.expert_out), static_cast<const uint32_t*>(m->ep_counts), m->d.hidden);
    if (e != cudaSuccess) return fail(m, ZC_EEXEC, std::string("ep return launch: ") + cudaGetErrorString(e));
    int rc = check_launch(m, "ep return");
    return rc < 0 ? rc : 1;
}

}  // namespace zc
