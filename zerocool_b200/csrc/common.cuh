// Shared device helpers and the handle layout of the B200 MoE library.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <string>
#include <vector>
#include <map>
#include <tuple>

#include "../../include/zc_moe.h"

namespace zc {

// ---------------------------------------------------------------------------------------------
// Scalar helpers
// ---------------------------------------------------------------------------------------------

// Round fp32 to the nearest-even bf16 value, NaN stays NaN (kernels/metal/qwen.metal:17-21).
__device__ __forceinline__ float bf_round(float x) {
    uint32_t u = __float_as_uint(x);
    if ((u & 0x7fffffffu) > 0x7f800000u) return __uint_as_float(0x7fc00000u);
    return __uint_as_float((u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u);
}
__device__ __forceinline__ uint16_t bf_bits(float x) { return uint16_t(__float_as_uint(bf_round(x)) >> 16); }
__device__ __forceinline__ float bf_to_float(uint16_t v) { return __uint_as_float(uint32_t(v) << 16); }
__device__ __forceinline__ float meta_to_float(uint16_t v, bool is_f16) {
    return is_f16 ? __half2float(__ushort_as_half(v)) : bf_to_float(v);
}

// Sigmoid in the reference's form (qwen.metal:30-32): 1/(1+exp|x|), mirrored for x >= 0.
__device__ __forceinline__ float sigmoid_f(float x) {
    float y = __fdiv_rn(1.0f, 1.0f + expf(fabsf(x)));
    return x < 0 ? y : 1.0f - y;
}
// BF16-staged sigmoid (qwen.metal:33-35). The exponential is evaluated in double and rounded once,
// which is the correctly rounded single-precision value the reference's activation tables pin.
__device__ __forceinline__ float sigmoid_bf(float x) {
    float e = float(exp(double(fabsf(x))));
    float y = bf_round(__fdiv_rn(1.0f, bf_round(1.0f + bf_round(e))));
    return x < 0 ? y : bf_round(1.0f - y);
}

// ---------------------------------------------------------------------------------------------
// Record geometry (expert_linear, src/engine/metal.mm:1124-1129, parametric)
// ---------------------------------------------------------------------------------------------
struct Projection {
    uint64_t codes, scales, biases;  // byte offsets inside a record
    uint32_t N, K, bits;
};
inline uint64_t projection_bytes(uint32_t N, uint32_t K, uint32_t bits, uint32_t group) {
    return uint64_t(N) * K * bits / 8 + 2 * uint64_t(N) * (K / group) * 2;
}
inline Projection projection_of(const zc_moe_desc& d, int p) {
    const uint32_t bits[3] = {d.gate_bits, d.up_bits, d.down_bits};
    uint64_t offset = 0;
    for (int i = 0; i < p; ++i) offset += projection_bytes(i == 2 ? d.hidden : d.ffn, i == 2 ? d.ffn : d.hidden, bits[i], d.group);
    Projection r;
    r.N = p == 2 ? d.hidden : d.ffn;
    r.K = p == 2 ? d.ffn : d.hidden;
    r.bits = bits[p];
    r.codes = offset;
    r.scales = offset + uint64_t(r.N) * r.K * r.bits / 8;
    r.biases = r.scales + uint64_t(r.N) * (r.K / d.group) * 2;
    return r;
}

// The descriptor of the shared expert's record: the routed geometry with the shared expert's own bit widths.
inline zc_moe_desc shared_desc_of(const zc_moe_desc& d) {
    zc_moe_desc s = d;
    if (d.shared_gate_bits) s.gate_bits = d.shared_gate_bits;
    if (d.shared_up_bits) s.up_bits = d.shared_up_bits;
    if (d.shared_down_bits) s.down_bits = d.shared_down_bits;
    return s;
}
inline uint64_t record_bytes_of(const zc_moe_desc& d) {
    const Projection pr = projection_of(d, 2);
    return pr.biases + uint64_t(pr.N) * (pr.K / d.group) * 2;
}

// ---------------------------------------------------------------------------------------------
// Handle
// ---------------------------------------------------------------------------------------------
struct LayerMem {
    uint8_t* records = nullptr;       // [local_experts, record_stride]
    void* router_w = nullptr;         // [E, H]
    uint8_t* shared_record = nullptr; // one record, or null
    void* shared_gate_w = nullptr;    // [1, H], or null
    float* router_bias = nullptr;     // [E] added to the logits after the partition sum; storage always present
    bool bias_set = false;
};

// Everything a kernel needs to know about one call, passed by value.
struct Call {
    const void* x;            // [T, H] act dtype
    void* out;                // [T, H] out dtype
    const uint8_t* records;
    const void* router_w;
    const uint8_t* shared_record;
    const void* shared_gate_w;
    const float* router_bias;   // [E] or null
    float* logits;            // [T, E]
    float* gate_logit;        // [T]
    int32_t* ids;             // [T, K]
    float* weights;           // [T, K]
    int32_t* offsets;         // [E+1]
    int32_t* perm;            // [T*K]
    int32_t* active;          // [E] ascending ids of experts with work
    int4* items;              // [E] the same list as {expert, first position in perm, rows, 0}; x = -1 past its end
    int32_t* counters;        // [0] number of active experts; [16 + layer] the same, kept per layer
    float* hbuf;              // [T*K + T, F]: rows in permuted slot order, then shared rows
    float* expert_out;        // [T*K, H] by original slot
    float* shared_out;        // [T, H]
    uint32_t* status;
    uint32_t T, H, F, E, K, layer;
    uint32_t first_expert, local_experts;
    uint64_t record_stride;
    Projection gate, up, down;
    Projection sgate, sup, sdown;   // the shared expert's record (equal to gate, up, down unless shared_split)
    uint8_t shared_split;           // the shared record has other bit widths: it runs as launches of its own
    uint8_t act_dtype, out_dtype, meta_f16, router_dtype, has_shared, ref, q8_signed;
    uint32_t item_rows_max;   // decode family: items with more rows than this are left to the tensor-core family (0 = no limit)
    uint8_t quiet_drop;       // the permutation drops ids outside [0, E) without raising the status bit (unused row slots of a receive area)
    // expert parallelism, sender side: the combine waits (bounded) for every owner's return flag of the current epoch
    const unsigned long long* ep_ret_flags;   // [ep_world] in this rank's window; null outside expert parallelism
    const uint32_t* ep_ctl;                   // [0] = epoch
    uint32_t ep_world;
    unsigned long long ep_wait_ns;
};

// Expert parallelism over peer memory (csrc/ep.cu). Every rank owns one window with this layout (byte offsets).
constexpr int EP_MAX_RANKS = 16;
struct EpWindow {
    uint64_t rows;        // [world][cap][row bytes]  token rows received from each source rank
    uint64_t tags;        // [world][cap] int2 {expert id, router slot on the source}
    uint64_t in_flags;    // [EP_MAX_RANKS] u64 {epoch << 32 | rows sent}, written by each source
    uint64_t ret_flags;   // [EP_MAX_RANKS] u64 {epoch << 32}, written by each owner when its results are stored
    uint64_t out;         // [cap][H] fp32: results by router slot, written by the owners (the combine's expert_out)
    uint64_t bytes;
    uint32_t cap;         // rows one source can send to one owner: max_tokens x top_k
    uint32_t world;
};
struct EpPeers { uint8_t* base[EP_MAX_RANKS]; };
EpWindow ep_window_layout(const zc_moe_desc& d);

struct EpArgs {
    EpPeers peers;
    EpWindow win;
    uint32_t me, world, per;          // this rank, ranks, experts per rank
    uint32_t* ctl;                    // [0] epoch, [1] send arrivals, [2] return arrivals
    uint32_t* status;
    unsigned long long wait_ns;
};

#ifdef __CUDACC__
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait of one thread for flag word `p` to carry an epoch >= `epoch`. Returns the word, or 0 after
// the limit (the caller then treats the source as having sent nothing). Once the status word carries the
// time-out bit, later waits give up at once, so a stack of layers does not wait the limit again per layer.
__device__ __forceinline__ unsigned long long ep_wait(const unsigned long long* p, uint32_t epoch, uint32_t* status, unsigned long long limit_ns) {
    unsigned long long v = ld_acquire_sys(p);
    if (uint32_t(v >> 32) >= epoch) return v;
    if (*reinterpret_cast<volatile uint32_t*>(status) & ZC_STATUS_TIMEOUT) return 0;
    const unsigned long long t0 = global_ns();
    for (;;) {
        __nanosleep(200);
        v = ld_acquire_sys(p);
        if (uint32_t(v >> 32) >= epoch) return v;
        if (global_ns() - t0 > limit_ns) break;
    }
    atomicOr(status, ZC_STATUS_TIMEOUT);
    return 0;
}
// Owner side of the peer transport: wait for every source's flag of the current epoch, then write the expert id of every
// row slot of the receive area (-1 for slots beyond a source's count, and for ids outside this rank's range). One CTA.
__device__ __forceinline__ void ep_receive_body(const EpArgs& a, int32_t* __restrict__ row_ids, uint32_t* __restrict__ counts, uint32_t* count_s /* shared [EP_MAX_RANKS] */) {
    const uint8_t* mine = a.peers.base[a.me];
    const uint32_t epoch = a.ctl[0];
    if (threadIdx.x < a.world) {
        const unsigned long long v = ep_wait(reinterpret_cast<const unsigned long long*>(mine + a.win.in_flags) + threadIdx.x, epoch, a.status, a.wait_ns);
        const uint32_t n = uint32_t(v >> 32) >= epoch && epoch ? min(uint32_t(v), a.win.cap) : 0u;
        count_s[threadIdx.x] = n;
        counts[threadIdx.x] = n;
    }
    __syncthreads();
    const int2* tags = reinterpret_cast<const int2*>(mine + a.win.tags);
    const uint32_t first = a.me * a.per;
    for (uint32_t i = threadIdx.x; i < a.world * a.win.cap; i += blockDim.x) {
        const uint32_t src = i / a.win.cap, j = i % a.win.cap;
        int32_t id = -1;
        if (j < count_s[src]) {
            id = __ldcg(&tags[i].x);
            if (id < int32_t(first) || id >= int32_t(first + a.per)) id = -1;
        }
        row_ids[i] = id;
    }
}
// Sender side, inside the combine kernels: every CTA waits for the owners' return flags before it reads the results.
__device__ __forceinline__ void ep_wait_results(const Call& c) {
    if (!c.ep_ret_flags) return;
    if (threadIdx.x < c.ep_world) ep_wait(c.ep_ret_flags + threadIdx.x, c.ep_ctl[0], c.status, c.ep_wait_ns);
    __syncthreads();
}
#endif

}  // namespace zc

struct zc_moe {
    zc_moe_desc d{};
    int device = 0;
    uint32_t sms = 148;                  // SMs of the device (grids of the persistent-style kernels are sized in resident waves)
    std::vector<zc::LayerMem> layers;
    std::vector<void*> allocations;
    zc::Call scratch{};           // scratch pointers (x/out/layer fields filled per call)
    __half* xp = nullptr;                // [max_tokens, H] FP16 activations in the prefill kernels' k order
    __half* xsum = nullptr;              // [max_tokens, 4 H/64] group sums of xp (prefill correction stages)
    __half* hsum = nullptr;              // [max_tokens*K + max_tokens, 4 F/64] group sums of hbuf16
    __half* hbuf16 = nullptr;            // [max_tokens*K + max_tokens, F] FP16 SwiGLU outputs (prefill)
    void* pf_tiles = nullptr;            // tile list of the prefill launches
    int32_t* pf_ntiles = nullptr;
    int32_t* permute_blocks = nullptr;   // [ceil(max slots / 2048)][E]: per-CTA expert counts of the multi-CTA permutation
    uint32_t pf_max_tiles = 0;
    uint32_t* router_done = nullptr;     // arrival counters of the router's (row tile, token tile) pairs
    zc::Call ep{};                       // second scratch set: the experts step of expert parallelism (rows from all ranks)
    uint32_t ep_rows_cap = 0;
    // peer transport of expert parallelism (allocated when local_experts < experts; usable after zc_moe_ep_attach)
    uint8_t* ep_window = nullptr;
    zc::EpWindow ep_layout{};
    zc::EpPeers ep_peers{};
    void* ep_opened[zc::EP_MAX_RANKS] = {};   // mappings opened from IPC handles (closed at destroy)
    uint32_t ep_rank = 0, ep_world = 0;   // world = 0: not attached
    uint32_t* ep_ctl = nullptr;           // [0] epoch, [1] send arrivals, [2] return arrivals
    int32_t* ep_row_ids = nullptr;        // [world x cap] expert id of every row slot of the receive area (-1: unused)
    uint32_t* ep_counts = nullptr;        // [EP_MAX_RANKS] rows received from each source in the current epoch
    uint32_t ep_wait_ms = 2000;           // limit of one device-side wait for a peer's flag
    const int32_t* cancel = nullptr;      // host flag read before a layer is issued (zc_moe_set_cancel)
    int4* empty_items = nullptr;         // an item list with no entries (launches that run the shared expert only)
    int32_t* zero_counters = nullptr;    // an always-zero counter block (launches that run the shared expert only)
    float* router_partial = nullptr;     // [16, max_tokens, rows_padded] partition sums of the router
    void* act[2] = {nullptr, nullptr};   // stack ping-pong activations [max_tokens, H]
    void* host_x = nullptr;       // pinned staging for the host entry points
    void* host_out = nullptr;
    void* dev_x = nullptr;
    void* dev_out = nullptr;
    void* dev_final = nullptr;
    cudaStream_t own_stream = nullptr;
    std::string error;
    uint64_t launches = 0;
    // Captured stacks, keyed by everything a capture bakes in (kind of stack, token count, input and output address);
    // at most GRAPH_CACHE entries, the least recently used one is dropped.
    struct Graph { cudaGraphExec_t exec; uint64_t nodes; uint64_t last_use; };
    static constexpr size_t GRAPH_CACHE = 8;
    std::map<std::tuple<int, uint32_t, const void*, const void*>, Graph> graphs;
    uint64_t graph_clock = 0;
    // Optional per-kernel timing (zc_moe_profile_begin/end): one event pair per launch.
    uint32_t pdl = 0xffffffffu;   // bit per KernelKind: that kernel launches with programmatic stream serialization (see launch_chained)
    bool exact_h = false;         // down reads the FP32 SwiGLU rows as two FP16 terms instead of one
    uint32_t few_tiles_gate_up = 1, few_tiles_down = 2;      // 16-row tiles per warp of the streaming launches for those experts (few items: more, shorter CTAs)
    uint32_t router_db = 1;              // long batches: double-buffered whole-K router tiles (FP32 router rows, BF16 activations)
    uint32_t meta_blocks = 1;            // streaming kernels fetch scales and biases eight groups at a time: 0 never, 1 for gate/up with long rows, 2 wherever possible
    uint32_t prefill_small_rows = 16;   // long batches: experts with at most this many rows run on the streaming kernels (0 = none)
    bool prefill_wide = true;     // long batches: wide-tile kernel with accumulators resident in TMEM (false: per-group drain kernel)
    bool fold_q4 = true;          // Q4 codes enter the MMA with their 1024 offset (removed from the FP32 group sum)
    bool profiling = false;
    struct Span { int kind; cudaEvent_t start, stop; };
    std::vector<Span> spans;
};

namespace zc {
// Launchers (each returns the number of kernels launched, or a negative ZC_* code with moe->error set).
int launch_router(zc_moe* m, const Call& c, cudaStream_t s);
int launch_router_partial(zc_moe* m, const Call& c, cudaStream_t s);
uint32_t router_rows_padded(const zc_moe_desc& d);
int launch_route_permute(zc_moe* m, const Call& c, cudaStream_t s, bool do_route, bool do_permute);
int launch_forced_weights(zc_moe* m, const Call& c, const int32_t* forced, cudaStream_t s);
int launch_experts_decode(zc_moe* m, const Call& c, cudaStream_t s);
int launch_experts_prefill(zc_moe* m, const Call& c, cudaStream_t s, uint32_t skip_rows_upto = 0);
bool prefill_supported(const zc_moe_desc& d);
size_t prefill_tile_capacity(const zc_moe_desc& d);
size_t prefill_tile_bytes();
size_t permute_block_count(size_t slots);   // CTAs of the multi-CTA permutation for this many slots
int launch_wait_selftest(zc_moe* m, uint32_t polls, uint32_t* report, cudaStream_t s);
size_t prefill_sum_halves(uint32_t K);      // group-sum halves per row the tensor-core family keeps for a projection with this K
int launch_combine(zc_moe* m, const Call& c, cudaStream_t s);
int launch_ep_gather(zc_moe* m, const Call& c, void* rows, int32_t* row_experts, cudaStream_t s);
int launch_ep_scatter(zc_moe* m, const Call& c, const float* y, cudaStream_t s);
int launch_ep_send(zc_moe* m, const Call& c, cudaStream_t s);
int launch_ep_receive(zc_moe* m, cudaStream_t s);
int launch_ep_receive_permute(zc_moe* m, const Call& q, cudaStream_t s);   // both in one launch (route.cu); 0 = not applicable
EpArgs ep_args(const zc_moe* m);
int launch_ep_return(zc_moe* m, cudaStream_t s);
int launch_hc_mix(zc_moe* m, const float* n, const float* mix, uint32_t T, uint32_t H, void* x, int x_dtype, cudaStream_t s);
int launch_combine_hc(zc_moe* m, const Call& c, const float* hyper, const float* inject, float* out, cudaStream_t s);
int launch_activation_table(const float* x, uint32_t n, float* sigmoid_out, float* silu_out, cudaStream_t s);
int launch_combine_norm(zc_moe* m, const Call& c, void* next, int next_dtype, cudaStream_t s);
int launch_synth_layer(zc_moe* m, uint32_t layer, uint64_t seed, cudaStream_t s);
enum KernelKind { KERNEL_ROUTER = 0, KERNEL_ROUTE, KERNEL_PERMUTE, KERNEL_GATE_UP, KERNEL_DOWN, KERNEL_COMBINE, KERNEL_EP,
                  KERNEL_PREFILL_PREP, KERNEL_PREFILL_GATE_UP, KERNEL_PREFILL_DOWN, KERNEL_KINDS };
// Brackets one kernel launch with events when profiling is enabled.
struct Timed {
    zc_moe* m; cudaStream_t s; int kind; cudaEvent_t stop = nullptr;
    Timed(zc_moe* m_, cudaStream_t s_, int kind_) : m(m_), s(s_), kind(kind_) {
        if (!m->profiling) return;
        cudaEvent_t start;
        cudaEventCreate(&start); cudaEventCreate(&stop);
        cudaEventRecord(start, s);
        m->spans.push_back({kind, start, stop});
    }
    ~Timed() { if (stop) cudaEventRecord(stop, s); }
};
int fail(zc_moe* m, int code, const std::string& text);
int check_launch(zc_moe* m, const char* what);

// cudaFuncSetAttribute is a per-device setting: the largest dynamic shared-memory size a kernel has been opted
// into is remembered per device, so that a process that owns handles on several GPUs configures each of them.
constexpr int MAX_DEVICES = 64;
struct SmemOptIn { size_t bytes[MAX_DEVICES] = {}; };
template <typename Kernel>
inline cudaError_t opt_in_smem(Kernel kernel, SmemOptIn& state, int device, size_t smem) {
    if (device < 0 || device >= MAX_DEVICES) return cudaErrorInvalidDevice;
    if (smem <= state.bytes[device]) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e == cudaSuccess) state.bytes[device] = smem;
    return e;
}

// Makes the handle's device current for the duration of an entry point and restores the caller's device.
inline uint32_t sm_count(const zc_moe* m) { return m ? m->sms : 148u; }

struct DeviceGuard {
    int previous = -1;
    bool changed = false;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&previous) == cudaSuccess && previous != device) changed = cudaSetDevice(device) == cudaSuccess;
    }
    ~DeviceGuard() { if (changed) cudaSetDevice(previous); }
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;
};

// Programmatic dependent launch. The kernels of a layer form a chain on one stream; each is launched with
// "programmatic stream serialization", which lets its CTAs be placed on SMs that the previous kernel no longer
// needs and run everything that does not depend on that kernel (index set-up, weight prefetch) before
// pdl_wait(). pdl_wait() returns once the previous kernel has completed and its writes are visible. Rules kept
// by every kernel launched through launch_chained: it calls pdl_wait() before its first read of anything an
// earlier kernel of the chain wrote and before its first global write, and calls pdl_launch_dependents() only
// after pdl_wait() - so the kernel after it cannot start before the kernel before it has finished, and at most
// two kernels of the chain ever overlap. Both calls do nothing in a launch without the attribute.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(const zc_moe* m, int kind, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                  const cudaLaunchAttribute* extra, int n_extra, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[4];
    int n = 0;
    for (int i = 0; i < n_extra && i < 3; ++i) attr[n++] = extra[i];
    if (m && kind >= 0 && ((m->pdl >> kind) & 1u) && !m->profiling) {      // event pairs around a launch would serialise it anyway
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr; cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif
}  // namespace zc
