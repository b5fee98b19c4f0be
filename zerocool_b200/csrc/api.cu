// C ABI of the B200 MoE library: handle lifetime, argument validation, layer orchestration.
//
// The orchestration is the device-side replacement of Model::moe (src/engine/model.cpp:431-557):
// router -> route -> permute -> experts (gate/up, down; shared expert as one more item) -> combine,
// all stream-ordered with no host synchronisation in between (the reference drains the GPU once per
// layer to build the dispatch lists on the CPU, model.cpp:446).
#include "common.cuh"
#include <cstdlib>

#include <cstdio>
#include <cstring>
#include <initializer_list>

namespace zc {

static thread_local std::string g_error;

int fail(zc_moe* m, int code, const std::string& text) {
    if (m) m->error = text;
    g_error = text;
    return code;
}
int check_launch(zc_moe* m, const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(m, ZC_EEXEC, std::string("CUDA launch of ") + what + ": " + cudaGetErrorString(e));
    return ZC_OK;
}

namespace {

size_t elem_bytes(int dtype) { return dtype == ZC_F32 ? 4 : 2; }

int cuda_fail(zc_moe* m, cudaError_t e, const char* what) {
    return fail(m, e == cudaErrorMemoryAllocation ? ZC_ENOMEM : ZC_EEXEC, std::string(what) + ": " + cudaGetErrorString(e));
}

template <typename T>
int dev_alloc(zc_moe* m, T** p, size_t bytes) {
    void* q = nullptr;
    const cudaError_t e = cudaMalloc(&q, bytes ? bytes : 16);
    if (e != cudaSuccess) return cuda_fail(m, e, "cudaMalloc");
    m->allocations.push_back(q);
    *p = static_cast<T*>(q);
    return ZC_OK;
}

int validate_desc(const zc_moe_desc& d, std::string& why) {
    auto bad = [&](const char* t) { why = t; return ZC_EINVAL; };
    if (!d.hidden || !d.ffn || !d.experts || !d.top_k || !d.layers || !d.max_tokens) return bad("zero dimension in descriptor");
    if (d.group != 64) return bad("unsupported affine matrix geometry: group must be 64");
    if (d.hidden % 128 || d.ffn % 128) return bad("unsupported affine matrix geometry: hidden and ffn must be multiples of 128");
    if (d.hidden > 4096) return bad("hidden above 4096 is not supported");
    if (d.experts % 32 || d.experts > 1024) return bad("experts must be a multiple of 32 and at most 1024");
    if (d.top_k > 32 || d.top_k > d.experts) return bad("top_k must be at most 32 and at most experts");
    for (uint8_t b : {d.gate_bits, d.up_bits, d.down_bits}) if (b != 4 && b != 8) return bad("unsupported affine matrix geometry: bits must be 4 or 8");
    if (d.gate_bits != d.up_bits) return bad("fused gate/up requires matching affine matrices");
    for (uint8_t b : {d.shared_gate_bits, d.shared_up_bits, d.shared_down_bits}) if (b != 0 && b != 4 && b != 8) return bad("unsupported affine matrix geometry: shared bits must be 0, 4 or 8");
    { const zc_moe_desc sd = shared_desc_of(d); if (sd.gate_bits != sd.up_bits) return bad("fused gate/up requires matching affine matrices (shared expert)"); }
    if (d.meta_dtype != ZC_BF16 && d.meta_dtype != ZC_F16) return bad("metadata dtype must be BF16 or F16");
    if (d.act_dtype != ZC_BF16 && d.act_dtype != ZC_F32) return bad("activation dtype must be BF16 or F32");
    if (d.out_dtype != ZC_BF16 && d.out_dtype != ZC_F32) return bad("output dtype must be BF16 or F32");
    if (d.router_dtype != ZC_BF16 && d.router_dtype != ZC_F32) return bad("router dtype must be BF16 or F32");
    if (d.arith != ZC_ARITH_FP32 && d.arith != ZC_ARITH_REFERENCE) return bad("unknown arithmetic mode");
    if (d.first_expert + (d.local_experts ? d.local_experts : d.experts) > d.experts) return bad("local expert range outside the router's experts");
    uint64_t bytes = 0;
    for (int p = 0; p < 3; ++p) { const Projection pr = projection_of(d, p); bytes = pr.biases + uint64_t(pr.N) * (pr.K / d.group) * 2; }
    if (d.record_bytes != bytes) return bad("record_bytes does not match the projection geometry");
    if (d.record_stride < d.record_bytes || d.record_stride % 16) return bad("record_stride must cover the record and be a multiple of 16");
    return ZC_OK;
}

Call make_call(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, void* out) {
    Call c = m->scratch;
    const LayerMem& L = m->layers[layer];
    c.x = x; c.out = out;
    c.records = L.records; c.router_w = L.router_w; c.shared_record = L.shared_record; c.shared_gate_w = L.shared_gate_w;
    c.router_bias = L.bias_set ? L.router_bias : nullptr;
    c.T = tokens;
    c.layer = layer;
    return c;
}

// Every caller buffer is read or written with 16-byte accesses: a misaligned pointer is an argument error here,
// not a misaligned-address fault on the device.
bool aligned16(std::initializer_list<const void*> ptrs) {
    for (const void* p : ptrs) if (reinterpret_cast<uintptr_t>(p) & 15) return false;
    return true;
}
bool overlaps(const void* a, size_t a_bytes, const void* b, size_t b_bytes) {
    const char* p = static_cast<const char*>(a); const char* q = static_cast<const char*>(b);
    return p < q + b_bytes && q < p + a_bytes;
}
// The reference's cancel flag (const std::atomic<bool>* cancel, include/engine/model.hpp:156): read on the host.
bool cancelled(const zc_moe* m) { return m->cancel && *static_cast<const volatile int32_t*>(m->cancel) != 0; }
void drop_graphs(zc_moe* m) {
    for (auto& g : m->graphs) cudaGraphExecDestroy(g.second.exec);
    m->graphs.clear();
}

int check_call(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, const void* out) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (layer >= m->d.layers) return fail(m, ZC_ERANGE, "layer outside the model");
    if (!tokens || tokens > m->d.max_tokens) return fail(m, ZC_EINVAL, "token count outside 1..max_tokens");
    if (!x || !out) return fail(m, ZC_EINVAL, "missing input or output buffer");
    const size_t xb = size_t(tokens) * m->d.hidden * elem_bytes(m->d.act_dtype), ob = size_t(tokens) * m->d.hidden * elem_bytes(m->d.out_dtype);
    if (overlaps(x, xb, out, ob)) return fail(m, ZC_EINVAL, "invalid or overlapping output");
    if (!aligned16({x, out})) return fail(m, ZC_EINVAL, "buffers must be 16-byte aligned");
    if (cancelled(m)) return fail(m, ZC_ECANCELLED, "generation cancelled");
    return ZC_OK;
}

// The experts of a layer. Long batches run on the tensor-core family, whose tile costs about the same whether it holds
// 128 token rows or 8 (the dequantisation of its 128 x K weights sets the pace): experts with only a few rows therefore
// go to the streaming kernels (eight rows per pass at HBM speed) first, and the grouped GEMM takes the rest. Which
// family an expert takes depends on its row count only, so a token's result does not depend on its place in the batch.
int launch_experts(zc_moe* m, const Call& c, cudaStream_t s, int family) {
    if (family != 1) return launch_experts_decode(m, c, s);
    int n, total = 0;
    const uint32_t small = m->prefill_small_rows;
    if (small) {
        Call few = c;
        few.has_shared = 0;                 // the shared expert sees every token: its rows stay with the grouped GEMM
        few.item_rows_max = small;
        if ((n = launch_experts_decode(m, few, s)) < 0) return n; total += n;
    }
    if ((n = launch_experts_prefill(m, c, s, small)) < 0) return n; total += n;
    return total;
}

// One layer: router partials -> route + permutation (one launch) -> gate/up -> down -> combine.
// With `next` set the combine also writes the normalised input of the following layer (the chained stack).
// family: 0 = decode kernels, 1 = prefill kernels (tensor-core grouped GEMM), -1 = by token count.
struct HcEpilogue { const float* hyper; const float* inject; float* out; };
int run_layer(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, void* out, cudaStream_t s, void* next = nullptr, int family = -1,
              const HcEpilogue* hc = nullptr) {
    const Call c = make_call(m, layer, x, tokens, out);
    // The tensor-core family pays from about 24 rows per expert on (measured crossover with every expert active:
    // 30 rows per expert at hidden 2048, 20 at hidden 4096); below that the streaming kernels are faster.
    if (family < 0) family = (tokens >= 64 && uint64_t(tokens) * m->d.top_k >= 24ull * m->d.local_experts) ? 1 : 0;
    if (family == 1 && !m->pf_tiles) family = 0;      // formats the prefill kernels do not take, or a decode-sized handle
    int n, total = 0;
    if ((n = launch_router_partial(m, c, s)) < 0) return n; total += n;
    if ((n = launch_route_permute(m, c, s, true, true)) < 0) return n; total += n;
    if ((n = launch_experts(m, c, s, family)) < 0) return n; total += n;
    if (hc) n = launch_combine_hc(m, c, hc->hyper, hc->inject, hc->out, s);
    else if (next) n = launch_combine_norm(m, c, next, m->d.act_dtype, s);
    else n = launch_combine(m, c, s);
    if (n < 0) return n; total += n;
    return total;
}

}  // namespace
}  // namespace zc

using namespace zc;

extern "C" {

const char* zc_last_error(void) { return g_error.c_str(); }
const char* zc_moe_last_error(const zc_moe* m) { return m ? m->error.c_str() : g_error.c_str(); }
uint64_t zc_moe_launch_count(const zc_moe* m) { return m ? m->launches : 0; }

int zc_moe_desc_finalize(zc_moe_desc* d) {
    if (!d) return fail(nullptr, ZC_EINVAL, "null descriptor");
    if (!d->group) d->group = 64;
    if (!d->hidden || !d->ffn || d->hidden % d->group || d->ffn % d->group) return fail(nullptr, ZC_EINVAL, "unsupported affine matrix geometry");
    if (!d->local_experts) d->local_experts = d->experts - d->first_expert;
    uint64_t bytes = 0;
    for (int p = 0; p < 3; ++p) { const Projection pr = projection_of(*d, p); bytes = pr.biases + uint64_t(pr.N) * (pr.K / d->group) * 2; }
    d->record_bytes = bytes;
    d->record_stride = (bytes + 16383) / 16384 * 16384;
    return ZC_OK;
}

int zc_moe_create(const zc_moe_desc* desc, int device, zc_moe** out) {
    if (out) *out = nullptr;
    if (!desc || !out) return fail(nullptr, ZC_EINVAL, "null descriptor or output");
    zc_moe_desc d = *desc;
    if (!d.local_experts) d.local_experts = d.experts - d.first_expert;
    std::string why;
    if (validate_desc(d, why) != ZC_OK) return fail(nullptr, ZC_EINVAL, why);
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) return fail(nullptr, ZC_EEXEC, "no CUDA device: this library has no CPU path");
    if (device < 0 || device >= count || device >= MAX_DEVICES) return fail(nullptr, ZC_EINVAL, "device index outside the visible devices");
    DeviceGuard guard(device);          // the caller's current device is restored on return
    int current = -1;
    if (cudaGetDevice(&current) != cudaSuccess || current != device) return fail(nullptr, ZC_EEXEC, "cudaSetDevice failed");
    cudaDeviceProp prop{};
    cudaGetDeviceProperties(&prop, device);
    if (prop.major < 10) return fail(nullptr, ZC_EEXEC, "this library is built for sm_100a (B200) only");

    zc_moe* m = new zc_moe();
    m->d = d; m->device = device; m->sms = prop.multiProcessorCount > 0 ? uint32_t(prop.multiProcessorCount) : 148u;
    if (const char* v = std::getenv("ZC_MOE_PDL")) m->pdl = uint32_t(std::strtoul(v, nullptr, 0)) ? (std::strtoul(v, nullptr, 0) == 1 ? 0xffffffffu : uint32_t(std::strtoul(v, nullptr, 0))) : 0u;   // 0 off, 1 on, else a mask of kernel kinds
    m->layers.resize(d.layers);
    const size_t T = d.max_tokens, H = d.hidden, F = d.ffn, E = d.experts, K = d.top_k;
    int rc = ZC_OK;
    auto A = [&](auto** p, size_t bytes) { if (rc == ZC_OK) rc = dev_alloc(m, p, bytes); };
    for (uint32_t l = 0; l < d.layers; ++l) {
        LayerMem& L = m->layers[l];
        A(&L.records, size_t(d.local_experts) * d.record_stride);
        uint8_t* rw = nullptr; A(&rw, E * H * elem_bytes(d.router_dtype)); L.router_w = rw;
        A(&L.router_bias, E * 4);
        if (d.has_shared) {
            A(&L.shared_record, (record_bytes_of(shared_desc_of(d)) + 16383) / 16384 * 16384);
            uint8_t* gw = nullptr; A(&gw, H * elem_bytes(d.router_dtype)); L.shared_gate_w = gw;
        }
    }
    Call& c = m->scratch;
    A(&c.logits, T * E * 4); A(&c.gate_logit, T * 4); A(&c.ids, T * K * 4); A(&c.weights, T * K * 4);
    A(&c.offsets, (E + 1) * 4); A(&c.perm, T * K * 4); A(&c.active, E * 4); A(&c.items, E * 16); A(&c.counters, (16 + size_t(d.layers)) * 4);
    if (T * K > 4096) A(&m->permute_blocks, permute_block_count(T * K) * E * 4);
    A(&m->router_partial, 16 * T * size_t(router_rows_padded(d)) * 4);
    const size_t done_n = size_t(router_rows_padded(d) / 32) * ((T + 7) / 8);
    A(&m->router_done, done_n * 4);
    if (rc == ZC_OK && (e = cudaMemset(m->router_done, 0, done_n * 4)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMemset");
    A(&c.hbuf, (T * K + T) * F * 4);
    if (prefill_supported(d) && T > 64) {
        A(&m->xp, T * H * 2); A(&m->hbuf16, (T * K + T) * F * 2);
        A(&m->xsum, T * prefill_sum_halves(d.hidden) * 2); A(&m->hsum, (T * K + T) * prefill_sum_halves(d.ffn) * 2);
        m->pf_max_tiles = uint32_t(prefill_tile_capacity(d));
        uint8_t* tl = nullptr; A(&tl, m->pf_max_tiles * prefill_tile_bytes()); m->pf_tiles = tl;
        A(&m->pf_ntiles, 16);
        // rows of dropped slots are never written: start from zeros so that the range check of the group sums only ever sees values a kernel stored
        if (rc == ZC_OK && (e = cudaMemset(m->hbuf16, 0, (T * K + T) * F * 2)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMemset");
    } A(&c.expert_out, T * K * H * 4); A(&c.shared_out, T * H * 4); A(&c.status, 16);
    A(&m->empty_items, E * 16);
    if (rc == ZC_OK && (e = cudaMemset(m->empty_items, 0xff, E * 16)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMemset");
    if (rc == ZC_OK && (e = cudaMemset(c.items, 0xff, E * 16)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMemset");
    A(&m->zero_counters, (16 + size_t(d.layers)) * 4);
    if (rc == ZC_OK && (e = cudaMemset(m->zero_counters, 0, (16 + size_t(d.layers)) * 4)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMemset");
    if (d.local_experts < d.experts) {
        // expert parallelism: rows can arrive from every rank's tokens
        const size_t ranks = (d.experts + d.local_experts - 1) / d.local_experts;
        const size_t R = T * K * ranks;
        m->ep_rows_cap = uint32_t(R);
        Call& q = m->ep;
        A(&q.offsets, (E + 1) * 4); A(&q.perm, R * 4); A(&q.active, E * 4); A(&q.items, E * 16); A(&q.counters, (16 + size_t(d.layers)) * 4);
        A(&q.hbuf, R * F * 4);
        if (rc == ZC_OK && (e = cudaMemset(q.counters, 0, (16 + size_t(d.layers)) * 4)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMemset");
        // peer transport: the window other ranks store into, and what the owner side needs around it
        if (d.experts % d.local_experts == 0 && d.first_expert % d.local_experts == 0 && ranks <= size_t(EP_MAX_RANKS)) {
            m->ep_layout = ep_window_layout(d);
            A(&m->ep_window, m->ep_layout.bytes);
            if (rc == ZC_OK && (e = cudaMemset(m->ep_window, 0, m->ep_layout.bytes)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMemset");
            A(&m->ep_ctl, 64); A(&m->ep_counts, EP_MAX_RANKS * 4); A(&m->ep_row_ids, R * 4); A(&q.expert_out, R * H * 4);
            if (rc == ZC_OK && (e = cudaMemset(m->ep_ctl, 0, 64)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMemset");
            if (rc == ZC_OK && (e = cudaMemset(m->ep_counts, 0, EP_MAX_RANKS * 4)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMemset");
        }
    }
    uint8_t* p0 = nullptr; uint8_t* p1 = nullptr; uint8_t* dx = nullptr; uint8_t* dout = nullptr; uint8_t* dfin = nullptr;
    A(&p0, T * H * 4); A(&p1, T * H * 4); A(&dx, T * H * 4); A(&dout, T * H * 4); A(&dfin, T * H * 4);
    m->act[0] = p0; m->act[1] = p1; m->dev_x = dx; m->dev_out = dout; m->dev_final = dfin;
    if (rc == ZC_OK && (e = cudaMemset(c.status, 0, 16)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMemset");
    if (rc == ZC_OK && (e = cudaMemset(c.counters, 0, (16 + size_t(d.layers)) * 4)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMemset");
    if (rc == ZC_OK && (e = cudaMallocHost(&m->host_x, T * H * 4)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMallocHost");
    if (rc == ZC_OK && (e = cudaMallocHost(&m->host_out, T * H * 4)) != cudaSuccess) rc = cuda_fail(m, e, "cudaMallocHost");
    if (rc == ZC_OK && (e = cudaStreamCreateWithFlags(&m->own_stream, cudaStreamNonBlocking)) != cudaSuccess) rc = cuda_fail(m, e, "cudaStreamCreate");
    if (rc != ZC_OK) { g_error = m->error; zc_moe_destroy(m); return rc; }
    c.H = d.hidden; c.F = d.ffn; c.E = d.experts; c.K = d.top_k;
    c.first_expert = d.first_expert; c.local_experts = d.local_experts; c.record_stride = d.record_stride;
    c.gate = projection_of(d, 0); c.up = projection_of(d, 1); c.down = projection_of(d, 2);
    {
        const zc_moe_desc sd = shared_desc_of(d);
        c.sgate = projection_of(sd, 0); c.sup = projection_of(sd, 1); c.sdown = projection_of(sd, 2);
        c.shared_split = d.has_shared && (sd.gate_bits != d.gate_bits || sd.up_bits != d.up_bits || sd.down_bits != d.down_bits);
    }
    c.act_dtype = d.act_dtype; c.out_dtype = d.out_dtype; c.meta_f16 = d.meta_dtype == ZC_F16; c.router_dtype = d.router_dtype;
    c.has_shared = d.has_shared; c.ref = d.arith == ZC_ARITH_REFERENCE; c.q8_signed = d.q8_signed;
    if (m->ep_rows_cap) {
        Call& q = m->ep;
        const Call keep = q;
        q = c;                                   // geometry and formats
        q.offsets = keep.offsets; q.perm = keep.perm; q.active = keep.active; q.items = keep.items; q.counters = keep.counters; q.hbuf = keep.hbuf;
        q.expert_out = keep.expert_out;
        q.K = 1; q.has_shared = 0;
    }
    *out = m;
    return ZC_OK;
}

void zc_moe_destroy(zc_moe* m) {
    if (!m) return;
    DeviceGuard guard(m->device);
    cudaDeviceSynchronize();
    drop_graphs(m);
    for (void* p : m->ep_opened) if (p) cudaIpcCloseMemHandle(p);
    for (void* p : m->allocations) cudaFree(p);
    if (m->host_x) cudaFreeHost(m->host_x);
    if (m->host_out) cudaFreeHost(m->host_out);
    if (m->own_stream) cudaStreamDestroy(m->own_stream);
    delete m;
}

int zc_moe_load_layer(zc_moe* m, uint32_t layer, const void* records, uint32_t first_expert, uint32_t count,
                      const void* router_w, const void* shared_record, const void* shared_gate_w) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (layer >= m->d.layers) return fail(m, ZC_ERANGE, "layer outside the model");
    const zc_moe_desc& d = m->d;
    LayerMem& L = m->layers[layer];
    DeviceGuard guard(m->device);
    cudaError_t e;
    if (records) {
        if (first_expert < d.first_expert || uint64_t(first_expert) + count > uint64_t(d.first_expert) + d.local_experts)
            return fail(m, ZC_ERANGE, "expert range outside the records this handle holds");
        e = cudaMemcpy(L.records + size_t(first_expert - d.first_expert) * d.record_stride, records, size_t(count) * d.record_stride, cudaMemcpyDefault);
        if (e != cudaSuccess) return cuda_fail(m, e, "copy of expert records");
    }
    if (router_w && (e = cudaMemcpy(L.router_w, router_w, size_t(d.experts) * d.hidden * elem_bytes(d.router_dtype), cudaMemcpyDefault)) != cudaSuccess)
        return cuda_fail(m, e, "copy of router weight");
    if ((shared_record || shared_gate_w) && !d.has_shared) return fail(m, ZC_EINVAL, "layer has no shared expert");
    if (shared_record && (e = cudaMemcpy(L.shared_record, shared_record, record_bytes_of(shared_desc_of(d)), cudaMemcpyDefault)) != cudaSuccess)
        return cuda_fail(m, e, "copy of shared expert record");
    if (shared_gate_w && (e = cudaMemcpy(L.shared_gate_w, shared_gate_w, size_t(d.hidden) * elem_bytes(d.router_dtype), cudaMemcpyDefault)) != cudaSuccess)
        return cuda_fail(m, e, "copy of shared gate weight");
    return ZC_OK;
}

int zc_moe_set_router_bias(zc_moe* m, uint32_t layer, const float* bias) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (layer >= m->d.layers) return fail(m, ZC_ERANGE, "layer outside the model");
    LayerMem& L = m->layers[layer];
    DeviceGuard guard(m->device);
    drop_graphs(m);                      // captured launches hold the old argument (bias pointer or none)
    if (!bias) { L.bias_set = false; return ZC_OK; }
    const cudaError_t e = cudaMemcpy(L.router_bias, bias, size_t(m->d.experts) * 4, cudaMemcpyDefault);
    if (e != cudaSuccess) return cuda_fail(m, e, "copy of router bias");
    L.bias_set = true;
    return ZC_OK;
}

int zc_moe_layer_buffers(zc_moe* m, uint32_t layer, void** records, void** router_w, void** shared_record, void** shared_gate_w) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (layer >= m->d.layers) return fail(m, ZC_ERANGE, "layer outside the model");
    const LayerMem& L = m->layers[layer];
    if (records) *records = L.records;
    if (router_w) *router_w = L.router_w;
    if (shared_record) *shared_record = L.shared_record;
    if (shared_gate_w) *shared_gate_w = L.shared_gate_w;
    return ZC_OK;
}

int zc_moe_router(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, float* logits, void* stream) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (layer >= m->d.layers) return fail(m, ZC_ERANGE, "layer outside the model");
    if (!tokens || tokens > m->d.max_tokens || !x || !logits) return fail(m, ZC_EINVAL, "linear input shape");
    if (!aligned16({x, logits})) return fail(m, ZC_EINVAL, "buffers must be 16-byte aligned");
    DeviceGuard guard(m->device);
    Call c = make_call(m, layer, x, tokens, nullptr);
    c.logits = logits;
    const int n = launch_router(m, c, static_cast<cudaStream_t>(stream));
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

int zc_moe_route(zc_moe* m, const float* logits, uint32_t tokens, int32_t* ids, float* weights, void* stream) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    // Metal::route: "invalid route selection buffers" (src/engine/metal.mm:262-264)
    if (!tokens || tokens > m->d.max_tokens || !logits || !ids || !weights) return fail(m, ZC_EINVAL, "invalid route selection buffers");
    if (!aligned16({logits, ids, weights})) return fail(m, ZC_EINVAL, "buffers must be 16-byte aligned");
    DeviceGuard guard(m->device);
    Call c = m->scratch;
    c.T = tokens; c.logits = const_cast<float*>(logits); c.ids = ids; c.weights = weights;
    const int n = launch_route_permute(m, c, static_cast<cudaStream_t>(stream), true, false);
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

int zc_moe_permute(zc_moe* m, const int32_t* ids, uint32_t tokens, int32_t* offsets, int32_t* perm, void* stream) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (!tokens || tokens > m->d.max_tokens || !ids || !offsets || !perm) return fail(m, ZC_EINVAL, "invalid permutation buffers");
    if (!aligned16({ids, offsets, perm})) return fail(m, ZC_EINVAL, "buffers must be 16-byte aligned");
    DeviceGuard guard(m->device);
    Call c = m->scratch;
    c.T = tokens; c.ids = const_cast<int32_t*>(ids); c.offsets = offsets; c.perm = perm;
    const int n = launch_route_permute(m, c, static_cast<cudaStream_t>(stream), false, true);
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

int zc_moe_combine(zc_moe* m, const float* expert_out, const float* weights, const int32_t* ids, const float* shared, const float* gate_logit,
                   uint32_t tokens, void* out, void* stream) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (!tokens || tokens > m->d.max_tokens || !expert_out || !weights || !ids || !out) return fail(m, ZC_EINVAL, "token count outside 1..max_tokens or missing buffer");
    if ((shared == nullptr) != (gate_logit == nullptr)) return fail(m, ZC_EINVAL, "shared rows and gate values come together");
    if (!aligned16({expert_out, weights, ids, shared, gate_logit, out})) return fail(m, ZC_EINVAL, "buffers must be 16-byte aligned");
    DeviceGuard guard(m->device);
    Call c = m->scratch;
    c.T = tokens; c.out = out;
    c.expert_out = const_cast<float*>(expert_out); c.weights = const_cast<float*>(weights); c.ids = const_cast<int32_t*>(ids);
    c.shared_out = const_cast<float*>(shared); c.gate_logit = const_cast<float*>(gate_logit); c.has_shared = shared != nullptr;
    const int n = launch_combine(m, c, static_cast<cudaStream_t>(stream));
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

int zc_activation_bf16(const float* x, uint32_t n, float* sigmoid_out, float* silu_out, void* stream) {
    if (!x || !n || (!sigmoid_out && !silu_out)) return fail(nullptr, ZC_EINVAL, "missing buffer");
    return launch_activation_table(x, n, sigmoid_out, silu_out, static_cast<cudaStream_t>(stream));
}

static int forward_family(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, void* out, void* stream, int family) {
    int rc = check_call(m, layer, x, tokens, out);
    if (rc != ZC_OK) return rc;
    DeviceGuard guard(m->device);
    const int n = run_layer(m, layer, x, tokens, out, static_cast<cudaStream_t>(stream), nullptr, family);
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

int zc_moe_hc_mix(zc_moe* m, const float* normed, const float* mix, uint32_t tokens, void* x, void* stream) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (!tokens || tokens > m->d.max_tokens || !normed || !mix || !x) return fail(m, ZC_EINVAL, "token count outside 1..max_tokens or missing buffer");
    if (!aligned16({normed, mix, x})) return fail(m, ZC_EINVAL, "buffers must be 16-byte aligned");
    DeviceGuard guard(m->device);
    const int n = launch_hc_mix(m, normed, mix, tokens, m->d.hidden, x, m->d.act_dtype, static_cast<cudaStream_t>(stream));
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

int zc_moe_forward_hc(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, const float* hyper, const float* inject, float* hyper_out, void* stream) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (layer >= m->d.layers) return fail(m, ZC_ERANGE, "layer outside the model");
    if (!tokens || tokens > m->d.max_tokens || !x || !hyper || !inject || !hyper_out) return fail(m, ZC_EINVAL, "token count outside 1..max_tokens or missing buffer");
    if (!aligned16({x, hyper, inject, hyper_out})) return fail(m, ZC_EINVAL, "buffers must be 16-byte aligned");
    const size_t xb = size_t(tokens) * m->d.hidden * elem_bytes(m->d.act_dtype), hb = size_t(tokens) * 4 * m->d.hidden * 4;
    if (overlaps(x, xb, hyper_out, hb)) return fail(m, ZC_EINVAL, "invalid or overlapping output");
    if (cancelled(m)) return fail(m, ZC_ECANCELLED, "generation cancelled");
    DeviceGuard guard(m->device);
    const HcEpilogue hc{hyper, inject, hyper_out};
    const int n = run_layer(m, layer, x, tokens, nullptr, static_cast<cudaStream_t>(stream), nullptr, -1, &hc);
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

int zc_moe_forward_routed(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, const int32_t* ids, void* out, void* stream) {
    int rc = check_call(m, layer, x, tokens, out);
    if (rc != ZC_OK) return rc;
    if (!ids) return fail(m, ZC_EINVAL, "invalid route selection buffers");
    if (!aligned16({ids})) return fail(m, ZC_EINVAL, "buffers must be 16-byte aligned");
    DeviceGuard guard(m->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const Call c = make_call(m, layer, x, tokens, out);
    int n, total = 0;
    if ((n = launch_router_partial(m, c, s)) < 0) return n; total += n;          // the scores of the recorded experts, and the shared gate
    if ((n = launch_forced_weights(m, c, ids, s)) < 0) return n; total += n;
    if ((n = launch_route_permute(m, c, s, false, true)) < 0) return n; total += n;
    const bool wide = tokens >= 64 && uint64_t(tokens) * m->d.top_k >= 24ull * m->d.local_experts && m->pf_tiles;
    if ((n = launch_experts(m, c, s, wide ? 1 : 0)) < 0) return n; total += n;
    if ((n = launch_combine(m, c, s)) < 0) return n; total += n;
    m->launches += total;
    return ZC_OK;
}

int zc_moe_decode(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, void* out, void* stream) {
    return forward_family(m, layer, x, tokens, out, stream, 0);
}

int zc_moe_prefill(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, void* out, void* stream) {
    if (m && !m->pf_tiles) return fail(m, ZC_EINVAL, "prefill kernels need BF16 activations, FP32 arithmetic, hidden and ffn multiples of 512 and max_tokens above 64");
    return forward_family(m, layer, x, tokens, out, stream, 1);
}

int zc_moe_forward(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, void* out, void* stream) {
    return forward_family(m, layer, x, tokens, out, stream, -1);
}

// ---- expert parallelism -------------------------------------------------------------------------
int zc_moe_ep_dispatch(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, void* rows, int32_t* row_experts, void* stream) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (layer >= m->d.layers) return fail(m, ZC_ERANGE, "layer outside the model");
    if (!tokens || tokens > m->d.max_tokens || !x || !rows || !row_experts) return fail(m, ZC_EINVAL, "token count outside 1..max_tokens or missing buffer");
    if (!aligned16({x, rows, row_experts})) return fail(m, ZC_EINVAL, "buffers must be 16-byte aligned");
    DeviceGuard guard(m->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const Call c = make_call(m, layer, x, tokens, nullptr);
    int n, total = 0;
    if ((n = launch_router_partial(m, c, s)) < 0) return n; total += n;
    if ((n = launch_route_permute(m, c, s, true, true)) < 0) return n; total += n;
    if ((n = launch_ep_gather(m, c, rows, row_experts, s)) < 0) return n; total += n;
    m->launches += total;
    return ZC_OK;
}

int zc_moe_ep_experts(zc_moe* m, uint32_t layer, const void* rows, const int32_t* row_experts, uint32_t n_rows, float* y, void* stream) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (layer >= m->d.layers) return fail(m, ZC_ERANGE, "layer outside the model");
    if (!m->ep_rows_cap) return fail(m, ZC_EINVAL, "the handle holds every expert: expert parallelism needs local_experts < experts");
    if (n_rows > m->ep_rows_cap) return fail(m, ZC_EINVAL, "more rows than max_tokens x top_k x ranks");
    if (!n_rows) return ZC_OK;
    if (!rows || !row_experts || !y) return fail(m, ZC_EINVAL, "missing buffer");
    if (!aligned16({rows, row_experts, y})) return fail(m, ZC_EINVAL, "buffers must be 16-byte aligned");
    DeviceGuard guard(m->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    Call c = m->ep;
    const LayerMem& L = m->layers[layer];
    c.x = rows; c.records = L.records; c.ids = const_cast<int32_t*>(row_experts); c.expert_out = y; c.T = n_rows; c.layer = layer;
    c.status = m->scratch.status;
    int n, total = 0;
    if ((n = launch_route_permute(m, c, s, false, true)) < 0) return n; total += n;
    if ((n = launch_experts_decode(m, c, s)) < 0) return n; total += n;
    m->launches += total;
    return ZC_OK;
}

int zc_moe_ep_combine(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, const float* y_sorted, void* out, void* stream) {
    int rc = check_call(m, layer, x, tokens, out);
    if (rc != ZC_OK) return rc;
    if (!y_sorted) return fail(m, ZC_EINVAL, "missing buffer");
    if (!aligned16({y_sorted})) return fail(m, ZC_EINVAL, "buffers must be 16-byte aligned");
    DeviceGuard guard(m->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    Call c = make_call(m, layer, x, tokens, out);
    int n, total = 0;
    if ((n = launch_ep_scatter(m, c, y_sorted, s)) < 0) return n; total += n;
    if (c.has_shared) {
        Call sh = c;
        sh.items = m->empty_items;
        sh.counters = m->zero_counters;          // no routed items: only the shared expert's blocks find work
        if ((n = launch_experts_decode(m, sh, s)) < 0) return n; total += n;
    }
    if ((n = launch_combine(m, c, s)) < 0) return n; total += n;
    m->launches += total;
    return ZC_OK;
}

// ---- expert parallelism over peer memory ------------------------------------------------------------
namespace {

int ep_ready(zc_moe* m, uint32_t layer) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (layer >= m->d.layers) return fail(m, ZC_ERANGE, "layer outside the model");
    if (!m->ep_window) return fail(m, ZC_EINVAL, "the handle has no expert-parallel window: it needs local_experts < experts, dividing experts evenly");
    if (!m->ep_world) return fail(m, ZC_EINVAL, "zc_moe_ep_attach has not been called");
    return ZC_OK;
}

// Sender side, first half: routing of the local tokens, rows and tags into the owners' windows, flags; then the
// shared expert (it depends on nothing that travels, so it runs while the rows are in flight).
int ep_send_phase(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, cudaStream_t s) {
    const Call c = make_call(m, layer, x, tokens, nullptr);
    int n, total = 0;
    if ((n = launch_router_partial(m, c, s)) < 0) return n; total += n;
    if ((n = launch_route_permute(m, c, s, true, true)) < 0) return n; total += n;
    if ((n = launch_ep_send(m, c, s)) < 0) return n; total += n;
    if (c.has_shared) {
        Call sh = c;
        sh.items = m->empty_items;
        sh.counters = m->zero_counters;          // no routed items: only the shared expert's blocks find work
        if ((n = launch_experts_decode(m, sh, s)) < 0) return n; total += n;
    }
    return total;
}

// Owner side: wait for every source's rows, regroup them by expert, run the experts in place, store the results
// into the senders' windows and publish the return flags.
int ep_process_phase(zc_moe* m, uint32_t layer, cudaStream_t s) {
    int n, total = 0;
    Call q = m->ep;
    const LayerMem& L = m->layers[layer];
    q.x = m->ep_window + m->ep_layout.rows; q.records = L.records; q.ids = m->ep_row_ids;
    q.T = m->ep_world * m->ep_layout.cap; q.layer = layer; q.status = m->scratch.status; q.quiet_drop = 1;
    if ((n = launch_ep_receive_permute(m, q, s)) < 0) return n;
    if (n == 0) {                           // a receive area too large for one sorting CTA: two launches
        if ((n = launch_ep_receive(m, s)) < 0) return n; total += n;
        if ((n = launch_route_permute(m, q, s, false, true)) < 0) return n;
    }
    total += n;
    if ((n = launch_experts_decode(m, q, s)) < 0) return n; total += n;
    if ((n = launch_ep_return(m, s)) < 0) return n; total += n;
    return total;
}

// Sender side, second half: wait for every owner's results (they sit at their router slots in this rank's
// window), then the fixed-order combine; with `next` also the normalised input of the following layer.
int ep_finish_phase(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, void* out, cudaStream_t s, void* next) {
    int n, total = 0;
    Call c = make_call(m, layer, x, tokens, out);
    c.expert_out = reinterpret_cast<float*>(m->ep_window + m->ep_layout.out);
    // the combine's CTAs wait themselves for the owners' return flags (no launch that only waits)
    c.ep_ret_flags = reinterpret_cast<const unsigned long long*>(m->ep_window + m->ep_layout.ret_flags);
    c.ep_ctl = m->ep_ctl; c.ep_world = m->ep_world; c.ep_wait_ns = (unsigned long long)(m->ep_wait_ms) * 1000000ull;
    n = next ? launch_combine_norm(m, c, next, m->d.act_dtype, s) : launch_combine(m, c, s);
    if (n < 0) return n; total += n;
    return total;
}

int ep_layer_launches(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, void* out, cudaStream_t s, void* next) {
    int n, total = 0;
    if ((n = ep_send_phase(m, layer, x, tokens, s)) < 0) return n; total += n;
    if ((n = ep_process_phase(m, layer, s)) < 0) return n; total += n;
    if ((n = ep_finish_phase(m, layer, x, tokens, out, s, next)) < 0) return n; total += n;
    return total;
}

}  // namespace

int zc_moe_ep_export(zc_moe* m, void* handle64, void** window) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (!m->ep_window) return fail(m, ZC_EINVAL, "the handle has no expert-parallel window: it needs local_experts < experts, dividing experts evenly");
    DeviceGuard guard(m->device);
    if (window) *window = m->ep_window;
    if (handle64) {
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the IPC handle is exchanged as 64 bytes");
        cudaIpcMemHandle_t h;
        const cudaError_t e = cudaIpcGetMemHandle(&h, m->ep_window);
        if (e != cudaSuccess) return cuda_fail(m, e, "cudaIpcGetMemHandle");
        std::memcpy(handle64, &h, 64);
    }
    return ZC_OK;
}

int zc_moe_ep_attach(zc_moe* m, uint32_t rank, uint32_t world, const void* peers, int kind) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (!m->ep_window) return fail(m, ZC_EINVAL, "the handle has no expert-parallel window: it needs local_experts < experts, dividing experts evenly");
    if (world != m->ep_layout.world || rank >= world || rank != m->d.first_expert / m->d.local_experts)
        return fail(m, ZC_EINVAL, "rank / world do not match the handle's expert range (world = experts / local_experts, rank = first_expert / local_experts)");
    if (!peers || (kind != 0 && kind != 1)) return fail(m, ZC_EINVAL, "missing peer table");
    DeviceGuard guard(m->device);
    for (uint32_t r = 0; r < world; ++r) {
        if (r == rank) { m->ep_peers.base[r] = m->ep_window; continue; }
        if (kind == 1) { m->ep_peers.base[r] = static_cast<uint8_t* const*>(peers)[r]; continue; }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const uint8_t*>(peers) + size_t(r) * 64, 64);
        void* p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess || !p) { cudaGetLastError(); return cuda_fail(m, e, "cudaIpcOpenMemHandle (peer access between the GPUs of this node is required)"); }
        m->ep_opened[r] = p;
        m->ep_peers.base[r] = static_cast<uint8_t*>(p);
    }
    m->ep_rank = rank; m->ep_world = world;
    drop_graphs(m);
    return ZC_OK;
}

int zc_moe_ep_send(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, void* stream) {
    int rc = ep_ready(m, layer);
    if (rc != ZC_OK) return rc;
    if (!tokens || tokens > m->d.max_tokens || !x) return fail(m, ZC_EINVAL, "token count outside 1..max_tokens or missing buffer");
    if (!aligned16({x})) return fail(m, ZC_EINVAL, "buffers must be 16-byte aligned");
    DeviceGuard guard(m->device);
    const int n = ep_send_phase(m, layer, x, tokens, static_cast<cudaStream_t>(stream));
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

int zc_moe_ep_process(zc_moe* m, uint32_t layer, void* stream) {
    int rc = ep_ready(m, layer);
    if (rc != ZC_OK) return rc;
    DeviceGuard guard(m->device);
    const int n = ep_process_phase(m, layer, static_cast<cudaStream_t>(stream));
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

int zc_moe_ep_finish(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, void* out, void* stream) {
    int rc = ep_ready(m, layer);
    if (rc != ZC_OK) return rc;
    if ((rc = check_call(m, layer, x, tokens, out)) != ZC_OK) return rc;
    DeviceGuard guard(m->device);
    const int n = ep_finish_phase(m, layer, x, tokens, out, static_cast<cudaStream_t>(stream), nullptr);
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

int zc_moe_ep_layer(zc_moe* m, uint32_t layer, const void* x, uint32_t tokens, void* out, void* stream) {
    int rc = ep_ready(m, layer);
    if (rc != ZC_OK) return rc;
    if ((rc = check_call(m, layer, x, tokens, out)) != ZC_OK) return rc;
    DeviceGuard guard(m->device);
    const int n = ep_layer_launches(m, layer, x, tokens, out, static_cast<cudaStream_t>(stream), nullptr);
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

// ---- host-buffer entry points and the chained stack ----------------------------------------------------
static int forward_host(zc_moe* m, uint32_t layer, const void* x_host, uint32_t tokens, void* out_host, void* stream, bool wait) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (!tokens || tokens > m->d.max_tokens || !x_host || !out_host) return fail(m, ZC_EINVAL, "token count outside 1..max_tokens or missing buffer");
    const size_t xb = size_t(tokens) * m->d.hidden * elem_bytes(m->d.act_dtype), ob = size_t(tokens) * m->d.hidden * elem_bytes(m->d.out_dtype);
    DeviceGuard guard(m->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if ((e = cudaMemcpyAsync(m->dev_x, x_host, xb, cudaMemcpyHostToDevice, s)) != cudaSuccess) return cuda_fail(m, e, "host to device copy");
    int rc = zc_moe_forward(m, layer, m->dev_x, tokens, m->dev_out, s);
    if (rc != ZC_OK) return rc;
    if ((e = cudaMemcpyAsync(out_host, m->dev_out, ob, cudaMemcpyDeviceToHost, s)) != cudaSuccess) return cuda_fail(m, e, "device to host copy");
    if (wait && (e = cudaStreamSynchronize(s)) != cudaSuccess) return cuda_fail(m, e, "MoE execution");
    return ZC_OK;
}

int zc_moe_forward_host(zc_moe* m, uint32_t layer, const void* x_host, uint32_t tokens, void* out_host, void* stream) {
    return forward_host(m, layer, x_host, tokens, out_host, stream, true);
}

int zc_moe_forward_host_async(zc_moe* m, uint32_t layer, const void* x_host, uint32_t tokens, void* out_host, void* stream) {
    return forward_host(m, layer, x_host, tokens, out_host, stream, false);
}

// Launches the chained stack on `s`: layer l reads `in` (l = 0) or the normalised previous output. With `ep` the
// layers are expert-parallel layers over peer memory. The cancel flag is read before every layer.
static int stack_launches(zc_moe* m, const void* x, uint32_t tokens, void* out, cudaStream_t s, bool ep = false) {
    const zc_moe_desc& d = m->d;
    int total = 0;
    const void* in = x;
    for (uint32_t l = 0; l < d.layers; ++l) {
        if (cancelled(m)) return fail(m, ZC_ECANCELLED, "generation cancelled");
        const bool last = l + 1 == d.layers;
        void* next = last ? nullptr : m->act[l & 1];
        int n = ep ? ep_layer_launches(m, l, in, tokens, last ? out : m->dev_out, s, next) : run_layer(m, l, in, tokens, last ? out : m->dev_out, s, next);
        if (n < 0) return n;
        total += n;
        in = next;
    }
    return total;
}

// One CUDA graph per (kind of stack, tokens, x, out): the launch sequence is fixed - routing only changes which
// blocks find work - so replaying the graph removes the per-launch host cost of ~6 kernels a layer.
static int stack_graph(zc_moe* m, const void* x, uint32_t tokens, void* out, cudaStream_t s, bool ep) {
    const auto key = std::make_tuple(ep ? 1 : 0, tokens, x, static_cast<const void*>(out));
    auto found = m->graphs.find(key);
    if (found == m->graphs.end()) {
        cudaStream_t cs = m->own_stream;
        cudaError_t e;
        // First use of each kernel outside capture, so that function attributes are set once. The input
        // may still be in flight on the caller's stream, so wait for that stream first.
        if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return cuda_fail(m, e, "MoE stack execution");
        int n = stack_launches(m, x, tokens, out, cs, ep);
        if (n < 0) return n;
        if ((e = cudaStreamSynchronize(cs)) != cudaSuccess) return cuda_fail(m, e, "MoE stack execution");
        if ((e = cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal)) != cudaSuccess) return cuda_fail(m, e, "graph capture");
        n = stack_launches(m, x, tokens, out, cs, ep);
        cudaGraph_t graph = nullptr;
        e = cudaStreamEndCapture(cs, &graph);
        if (n < 0) { if (graph) cudaGraphDestroy(graph); return n; }
        if (e != cudaSuccess) return cuda_fail(m, e, "graph capture");
        cudaGraphExec_t exec = nullptr;
        e = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) return cuda_fail(m, e, "graph instantiation");
        if (m->graphs.size() >= zc_moe::GRAPH_CACHE) {              // drop the least recently used capture
            auto oldest = m->graphs.begin();
            for (auto it = m->graphs.begin(); it != m->graphs.end(); ++it) if (it->second.last_use < oldest->second.last_use) oldest = it;
            cudaGraphExecDestroy(oldest->second.exec);
            m->graphs.erase(oldest);
        }
        found = m->graphs.emplace(key, zc_moe::Graph{exec, uint64_t(n), 0}).first;
    }
    found->second.last_use = ++m->graph_clock;
    const cudaError_t e = cudaGraphLaunch(found->second.exec, s);
    if (e != cudaSuccess) return cuda_fail(m, e, "graph launch");
    m->launches += found->second.nodes;
    return ZC_OK;
}

int zc_moe_stack(zc_moe* m, const void* x, uint32_t tokens, void* out, void* stream) {
    int rc = check_call(m, 0, x, tokens, out);
    if (rc != ZC_OK) return rc;
    DeviceGuard guard(m->device);
    return stack_graph(m, x, tokens, out, static_cast<cudaStream_t>(stream), false);
}

int zc_moe_ep_stack(zc_moe* m, const void* x, uint32_t tokens, void* out, void* stream) {
    int rc = ep_ready(m, 0);
    if (rc != ZC_OK) return rc;
    if ((rc = check_call(m, 0, x, tokens, out)) != ZC_OK) return rc;
    DeviceGuard guard(m->device);
    return stack_graph(m, x, tokens, out, static_cast<cudaStream_t>(stream), true);
}

int zc_moe_ep_stack_eager(zc_moe* m, const void* x, uint32_t tokens, void* out, void* stream) {
    int rc = ep_ready(m, 0);
    if (rc != ZC_OK) return rc;
    if ((rc = check_call(m, 0, x, tokens, out)) != ZC_OK) return rc;
    DeviceGuard guard(m->device);
    const int n = stack_launches(m, x, tokens, out, static_cast<cudaStream_t>(stream), true);
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

int zc_moe_stack_host(zc_moe* m, const void* x_host, uint32_t tokens, void* out_host, void* stream) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (!tokens || tokens > m->d.max_tokens || !x_host || !out_host) return fail(m, ZC_EINVAL, "token count outside 1..max_tokens or missing buffer");
    const size_t xb = size_t(tokens) * m->d.hidden * elem_bytes(m->d.act_dtype), ob = size_t(tokens) * m->d.hidden * elem_bytes(m->d.out_dtype);
    DeviceGuard guard(m->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if ((e = cudaMemcpyAsync(m->dev_x, x_host, xb, cudaMemcpyHostToDevice, s)) != cudaSuccess) return cuda_fail(m, e, "host to device copy");
    int rc = zc_moe_stack(m, m->dev_x, tokens, m->dev_final, s);
    if (rc != ZC_OK) return rc;
    if ((e = cudaMemcpyAsync(out_host, m->dev_final, ob, cudaMemcpyDeviceToHost, s)) != cudaSuccess) return cuda_fail(m, e, "device to host copy");
    if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return cuda_fail(m, e, "MoE stack execution");
    if (cancelled(m)) return fail(m, ZC_ECANCELLED, "generation cancelled");
    return ZC_OK;
}

int zc_moe_set_cancel(zc_moe* m, const int32_t* flag) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    m->cancel = flag;
    return ZC_OK;
}

int zc_moe_last_routing(zc_moe* m, const int32_t** ids, const float** weights, const int32_t** offsets, const int32_t** perm, const float** logits) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (ids) *ids = m->scratch.ids;
    if (weights) *weights = m->scratch.weights;
    if (offsets) *offsets = m->scratch.offsets;
    if (perm) *perm = m->scratch.perm;
    if (logits) *logits = m->scratch.logits;
    return ZC_OK;
}

int zc_moe_active_counts(zc_moe* m, int32_t* host_counts) {
    if (!m || !host_counts) return fail(m, ZC_EINVAL, "null handle or buffer");
    DeviceGuard guard(m->device);
    const cudaError_t e = cudaMemcpy(host_counts, m->scratch.counters + 16, size_t(m->d.layers) * 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(m, e, "device read");
    return ZC_OK;
}

int zc_moe_ep_active_counts(zc_moe* m, int32_t* host_counts) {
    if (!m || !host_counts) return fail(m, ZC_EINVAL, "null handle or buffer");
    if (!m->ep.counters) return fail(m, ZC_EINVAL, "the handle holds every expert: expert parallelism needs local_experts < experts");
    DeviceGuard guard(m->device);
    const cudaError_t e = cudaMemcpy(host_counts, m->ep.counters + 16, size_t(m->d.layers) * 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(m, e, "device read");
    return ZC_OK;
}

int zc_moe_read_device(zc_moe* m, void* host_dst, const void* device_src, uint64_t bytes) {
    if (!m || !host_dst || !device_src) return fail(m, ZC_EINVAL, "null handle or buffer");
    DeviceGuard guard(m->device);
    const cudaError_t e = cudaMemcpy(host_dst, device_src, bytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(m, e, "device read");
    return ZC_OK;
}

int zc_moe_status(zc_moe* m, void* stream, uint32_t* status) {
    if (!m || !status) return fail(m, ZC_EINVAL, "null handle or status");
    DeviceGuard guard(m->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaStreamSynchronize(s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->own_stream);
    if (e != cudaSuccess) return cuda_fail(m, e, "MoE execution");
    if ((e = cudaMemcpy(status, m->scratch.status, 4, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail(m, e, "status read");
    if ((e = cudaMemset(m->scratch.status, 0, 4)) != cudaSuccess) return cuda_fail(m, e, "status clear");
    return ZC_OK;
}

int zc_moe_wait_selftest(zc_moe* m, uint32_t polls, uint32_t* report, void* stream) {
    if (!m || !report) return fail(m, ZC_EINVAL, "null handle or report");
    if (polls == 0 || polls > 100000) return fail(m, ZC_EINVAL, "wait self-test: polls must be in 1..100000");
    DeviceGuard guard(m->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint32_t* dev = nullptr;
    cudaError_t e = cudaMalloc(&dev, 16);
    if (e != cudaSuccess) return cuda_fail(m, e, "wait self-test scratch");
    e = cudaMemsetAsync(dev, 0xff, 16, s);
    int rc = e == cudaSuccess ? launch_wait_selftest(m, polls, dev, s) : cuda_fail(m, e, "wait self-test scratch");
    if (rc >= 0) {
        if ((e = cudaStreamSynchronize(s)) == cudaSuccess) e = cudaMemcpy(report, dev, 16, cudaMemcpyDeviceToHost);
        rc = e == cudaSuccess ? ZC_OK : cuda_fail(m, e, "wait self-test");
    }
    cudaFree(dev);
    if (rc == ZC_OK) ++m->launches;
    return rc;
}

int zc_moe_stack_eager(zc_moe* m, const void* x, uint32_t tokens, void* out, void* stream) {
    int rc = check_call(m, 0, x, tokens, out);
    if (rc != ZC_OK) return rc;
    DeviceGuard guard(m->device);
    const int n = stack_launches(m, x, tokens, out, static_cast<cudaStream_t>(stream));
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

int zc_moe_set_option(zc_moe* m, const char* name, int value) {
    if (!m || !name) return fail(m, ZC_EINVAL, "null handle or option name");
    const bool fold = !std::strcmp(name, "fold_q4"), pdl = !std::strcmp(name, "pdl"), exact_h = !std::strcmp(name, "exact_h");
    const bool wide = !std::strcmp(name, "prefill_wide");
    if (!std::strcmp(name, "prefill_small_rows")) {
        if (value < 0 || value > 64) return fail(m, ZC_EINVAL, "prefill_small_rows must be 0..64");
        DeviceGuard guard(m->device);
        drop_graphs(m);
        m->prefill_small_rows = uint32_t(value);
        return ZC_OK;
    }
    if (!std::strcmp(name, "few_tiles_gate_up") || !std::strcmp(name, "few_tiles_down")) {
        if (value < 1 || value > 4) return fail(m, ZC_EINVAL, "few_tiles_* must be 1..4");
        DeviceGuard guard(m->device);
        drop_graphs(m);
        (name[10] == 'g' ? m->few_tiles_gate_up : m->few_tiles_down) = uint32_t(value);
        return ZC_OK;
    }
    if (!std::strcmp(name, "router_db")) {
        if (value != 0 && value != 1) return fail(m, ZC_EINVAL, "router_db must be 0 or 1");
        DeviceGuard guard(m->device);
        drop_graphs(m);
        m->router_db = uint32_t(value);
        return ZC_OK;
    }
    if (!std::strcmp(name, "meta_blocks")) {
        if (value < 0 || value > 3) return fail(m, ZC_EINVAL, "meta_blocks must be 0..3");
        DeviceGuard guard(m->device);
        drop_graphs(m);
        m->meta_blocks = uint32_t(value);
        return ZC_OK;
    }
    if (!std::strcmp(name, "ep_wait_ms")) {
        if (value < 1 || value > 60000) return fail(m, ZC_EINVAL, "ep_wait_ms must be 1..60000");
        DeviceGuard guard(m->device);
        drop_graphs(m);
        m->ep_wait_ms = uint32_t(value);
        return ZC_OK;
    }
    if (fold || pdl || exact_h || wide) {
        DeviceGuard guard(m->device);
        drop_graphs(m);                                                      // captured launches hold the old choice
        if (wide) m->prefill_wide = value != 0;
        else if (exact_h) m->exact_h = value != 0;
        else if (fold) m->fold_q4 = value != 0; else m->pdl = value == 0 ? 0u : value == 1 ? 0xffffffffu : uint32_t(value);
        return ZC_OK;
    }
    return fail(m, ZC_EINVAL, std::string("unknown option: ") + name);
}

const char* zc_moe_kernel_name(int kind) {
    static const char* names[KERNEL_KINDS] = {"router", "route", "permute", "gate_up", "down", "combine", "ep",
                                              "prefill_prep", "prefill_gate_up", "prefill_down"};
    return kind >= 0 && kind < KERNEL_KINDS ? names[kind] : nullptr;
}

int zc_moe_profile_begin(zc_moe* m) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    m->profiling = true;
    return ZC_OK;
}

int zc_moe_profile_end(zc_moe* m, double* ms_per_kind, uint64_t* launches_per_kind) {
    if (!m || !ms_per_kind || !launches_per_kind) return fail(m, ZC_EINVAL, "null handle or output");
    m->profiling = false;
    DeviceGuard guard(m->device);
    cudaError_t e = cudaDeviceSynchronize();
    for (int k = 0; k < KERNEL_KINDS; ++k) { ms_per_kind[k] = 0; launches_per_kind[k] = 0; }
    for (auto& sp : m->spans) {
        float ms = 0;
        if (e == cudaSuccess && cudaEventElapsedTime(&ms, sp.start, sp.stop) == cudaSuccess) { ms_per_kind[sp.kind] += ms; ++launches_per_kind[sp.kind]; }
        cudaEventDestroy(sp.start); cudaEventDestroy(sp.stop);
    }
    m->spans.clear();
    if (e != cudaSuccess) return cuda_fail(m, e, "MoE execution");
    return ZC_OK;
}

int zc_synth_fill_layer(zc_moe* m, uint32_t layer, uint64_t seed, void* stream) {
    if (!m) return fail(nullptr, ZC_EINVAL, "null handle");
    if (layer >= m->d.layers) return fail(m, ZC_ERANGE, "layer outside the model");
    DeviceGuard guard(m->device);
    const int n = launch_synth_layer(m, layer, seed, static_cast<cudaStream_t>(stream));
    if (n < 0) return n;
    m->launches += n;
    return ZC_OK;
}

}  // extern "C"
