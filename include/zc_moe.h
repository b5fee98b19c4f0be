/* zc_moe.h — C ABI of the B200 (sm_100a) Mixture-of-Experts layer.
 *
 * This is the boundary a ZeroCool-style engine binds instead of its Metal operator calls for the MoE
 * layer. The reference has no FFI layer of its own: the layer is `Buf Model::moe(const Buf& x, int layer,
 * uint32_t tokens, const std::atomic<bool>* cancel, const Buf& predict)` (include/engine/model.hpp:156,
 * src/engine/model.cpp:431-557) built from `class Metal` operators (include/engine/metal.hpp:101-119).
 * Each entry point below names the reference interface it replaces.
 *
 * Conventions
 *  - Plain C, no exceptions: every call returns ZC_OK or a negative code; zc_moe_last_error() gives the
 *    text the reference would have thrown (invalid_argument -> ZC_EINVAL, out_of_range -> ZC_ERANGE,
 *    runtime_error -> ZC_EEXEC).
 *  - The handle owns the HBM-resident expert records and all scratch. x / out belong to the caller.
 *  - Calls taking a stream are stream-ordered and do not block the host. `stream` is a cudaStream_t
 *    passed as void* (NULL = the legacy default stream).
 *  - One host thread drives a handle at a time (the reference's single-coordinator rule,
 *    include/engine/metal.hpp:45-47).
 *  - All arguments are validated on the host before anything is launched: ranges, shapes, overlap of input
 *    and output, and 16-byte alignment of every caller buffer (the kernels use 16-byte accesses; a misaligned
 *    pointer is ZC_EINVAL, never a device fault). Conditions only the device can see (a token whose router
 *    scores select fewer than top_k experts, a value outside the FP16 operand range, a peer that never
 *    answered) set a status word read by zc_moe_status(), like the reference's sparse_status_
 *    (src/engine/model.cpp:118-120).
 *  - A handle belongs to the device given to zc_moe_create. Every call makes that device current for its own
 *    duration and restores the caller's current device before it returns; x / out / stream must belong to the
 *    handle's device. One process may own handles on several devices.
 *  - Value range: activations and the internal SwiGLU rows enter the tensor-core products as FP16. For a Q4
 *    projection of the short-batch kernels a value must satisfy |v| < 4094, otherwise |v| <= 65504; in the
 *    long-batch kernels additionally the sum of 64 consecutive values must stay within 65504 in magnitude.
 *    Beyond that the affected output rows are not meaningful and ZC_STATUS_RANGE is raised. Scales and biases
 *    stored as BF16 must be representable in FP16 for the long-batch kernels (|s| >= 6.1e-5 or zero).
 *  - There is no CPU fallback: without a CUDA device zc_moe_create fails with ZC_EEXEC.
 */
#ifndef ZC_MOE_H
#define ZC_MOE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZC_OK          0
#define ZC_EINVAL     -1   /* std::invalid_argument in the reference */
#define ZC_ERANGE     -2   /* std::out_of_range */
#define ZC_EEXEC      -3   /* std::runtime_error ("Metal execution: ..." / CUDA error) */
#define ZC_ECANCELLED -4   /* "generation cancelled", src/engine/model.cpp:15 */
#define ZC_ENOMEM     -5

/* Element types. Numbering follows Resident::dtype (src/engine/metal.mm:1100-1102). */
#define ZC_BF16 0
#define ZC_F32  1
#define ZC_F16  2

/* Arithmetic contract.
 * ZC_ARITH_FP32:      fp32 accumulation everywhere, no intermediate rounding.
 * ZC_ARITH_REFERENCE: every BF16 rounding boundary of kernels/metal/qwen.metal (gate/up, activation,
 *                     down, combine) and the BF16 sum-of-four that multiplies the Q4 bias (:46-62). */
#define ZC_ARITH_FP32      0
#define ZC_ARITH_REFERENCE 1

/* Bits of the device status word. */
#define ZC_STATUS_INVALID_ROUTE 1u   /* "invalid router output", src/engine/model.cpp:459 */
#define ZC_STATUS_TIMEOUT       2u   /* a bounded device-side wait (prefill pipeline, expert-parallel flags) ran out */
#define ZC_STATUS_RANGE         4u   /* a value left the FP16 range of the tensor-core operands (see "Value range") */

typedef struct zc_moe zc_moe;

/* Layer geometry and formats. The reference fixes these at compile time
 * (include/engine/storage.hpp:26-34: hidden 2560, ffn 640, 512 experts, top-10, Q4 group 64, BF16
 * metadata); here they are parameters. Expert record layout: see zc_moe_load_layer. */
typedef struct zc_moe_desc {
    uint32_t hidden;         /* H, multiple of 128, at most 4096 */
    uint32_t ffn;            /* F, expert intermediate width, multiple of 128 */
    uint32_t experts;        /* E, routed experts seen by the router (multiple of 32, <= 1024) */
    uint32_t top_k;          /* K <= 32 */
    uint32_t layers;
    uint32_t group;          /* quantisation group, 64 */
    uint32_t max_tokens;     /* largest `tokens` any call will pass; sizes the scratch */
    uint32_t first_expert;   /* expert parallelism: first routed expert whose record this handle holds */
    uint32_t local_experts;  /* number of records held (0 = all E) */
    uint32_t reserved0;
    uint8_t  gate_bits, up_bits, down_bits;  /* 4 or 8 per projection */
    uint8_t  q8_signed;      /* 8-bit codes are int8 (1) or uint8 (0; the reference's Q8, qwen.metal:112-125) */
    uint8_t  meta_dtype;     /* scales / biases: ZC_BF16 or ZC_F16 */
    uint8_t  act_dtype;      /* x: ZC_BF16 or ZC_F32 */
    uint8_t  out_dtype;      /* out: ZC_BF16 or ZC_F32 */
    uint8_t  router_dtype;   /* router weight and shared-gate vector: ZC_F32 or ZC_BF16 */
    uint8_t  has_shared;     /* layer has a shared expert with a sigmoid gate */
    uint8_t  arith;          /* ZC_ARITH_* */
    uint8_t  shared_gate_bits, shared_up_bits, shared_down_bits;   /* shared expert's record: 4 or 8 per projection; 0 = as the routed
                                * experts. The reference's mixed artifact keeps routed experts Q4 and the shared expert Q8
                                * (src/engine/metal.mm:1103-1123, docs/qwen_engine.md:261-266). */
    uint8_t  reserved[3];
    uint64_t record_bytes;   /* payload of one record = sum over projections of codes+scales+biases */
    uint64_t record_stride;  /* distance between records in a layer file (>= record_bytes) */
} zc_moe_desc;

/* Fills record_bytes / record_stride (stride = payload rounded up to 16 KiB, as
 * scripts/qwen/prepare_storage.py:140-160 lays records out) from the other fields. */
int zc_moe_desc_finalize(zc_moe_desc* desc);

/* Replaces Model::Model's Metal + Resident + ExpertCache construction for this path
 * (src/engine/model.cpp:47-117): allocates HBM for every layer's records, router and shared-expert
 * tensors, and the scratch for max_tokens. On failure *out is NULL and zc_last_error() has the text. */
int zc_moe_create(const zc_moe_desc* desc, int device, zc_moe** out);
void zc_moe_destroy(zc_moe* moe);
const char* zc_moe_last_error(const zc_moe* moe);
const char* zc_last_error(void);

/* Replaces ExpertStore::read / ExpertCache::acquire (src/engine/storage.cpp:507-516, 631-674): records
 * are copied once into HBM instead of being streamed per use. `records` holds `count` records at
 * desc.record_stride for experts [first_expert, first_expert+count) and may be host or device memory.
 * Record layout (expert_linear, src/engine/metal.mm:1124-1129, generalised): projections gate, up, down
 * in that order, each [codes | scales | biases]; codes row-major [N, K*bits/8] (Q4: uint32 words of 8
 * nibbles, k ascending from the least significant nibble); scales/biases [N, K/group] 16-bit.
 * router_w: [E, H]; shared_record: one record in the same layout with the shared expert's own bit widths
 * (shared_*_bits) or NULL; shared_gate_w: [1, H] or NULL.
 * Any pointer may be NULL to leave that tensor as it is. */
int zc_moe_load_layer(zc_moe* moe, uint32_t layer, const void* records, uint32_t first_expert, uint32_t count,
                      const void* router_w, const void* shared_record, const void* shared_gate_w);

/* Optional per-expert additive bias on the router logits of a layer (fp32 [E], host or device; NULL removes
 * it), added after the partition sum. The reference's router has none; the benchmark's skewed-load
 * configuration (Zipf bias on the logits) needs it. */
int zc_moe_set_router_bias(zc_moe* moe, uint32_t layer, const float* bias);

/* Device addresses of a layer's resident tensors, for producers that fill HBM in place. */
int zc_moe_layer_buffers(zc_moe* moe, uint32_t layer, void** records, void** router_w,
                         void** shared_record, void** shared_gate_w);

/* Replaces Metal::linear(router gate, x, tokens, float_output=true) (src/engine/model.cpp:434 ->
 * src/engine/metal.mm:818-822, router_mm + router_accumulate): logits [tokens, E] fp32 with the
 * reference's sixteen-partition accumulation order. x, logits: device memory. */
int zc_moe_router(zc_moe* moe, uint32_t layer, const void* x, uint32_t tokens, float* logits, void* stream);

/* Router logits without any allocation. No counterpart in the reference: it exists for callers that cannot
 * call cudaMalloc (so cannot create a handle) — code running while the host engine's allocator owns all of
 * HBM, while another thread captures a CUDA graph, or in a loop that may not take the allocator lock.
 * Same arithmetic and results as zc_moe_router. x [tokens, hidden] (act_dtype), router_w [experts, hidden]
 * (router_dtype) and logits [tokens, experts] fp32 are device memory of the current device.
 * Limits (rejected with ZC_EINVAL beyond them): tokens <= 64, experts <= 512 (multiple of 32), hidden <= 3072
 * (multiple of 128); x, router_w and logits 16-byte aligned, logits overlapping neither input. The scratch is a 2 MiB + 4 KiB array inside the library image, held by every GPU that
 * loads the library until the process exits. The first call on a device looks up that array's device address
 * (cudaGetSymbolAddress); make that first call before any stream capture begins. All calls share the array,
 * which keeps the previous call's contents: the call clears the counters it needs at zero itself, and two
 * calls that overlap on the GPU (different streams, or different threads) race — serialise them.
 * Calls no cudaMalloc, cudaFree or allocating library routine. */
int zc_router_logits_noalloc(const void* x, int act_dtype, const void* router_w, int router_dtype,
                             uint32_t tokens, uint32_t hidden, uint32_t experts, float* logits, void* stream);

/* Replaces Metal::route (include/engine/metal.hpp:112, src/engine/metal.mm:261-266, route_simd
 * qwen.metal:768-795): ids [tokens, K] int32 in rank order (unfilled ranks -1), weights [tokens, K]
 * fp32 = softmax over the selected scores. Device memory. */
int zc_moe_route(zc_moe* moe, const float* logits, uint32_t tokens, int32_t* ids, float* weights, void* stream);

/* Replaces the host-side dispatch of Model::moe (src/engine/model.cpp:449-461, 473-474) and the row
 * lists of encode_expert_rows (src/engine/pipeline.cpp:18-23), on the device: a stable counting sort of
 * the flat slots p = t*K + j by expert id. offsets [E+1], perm [tokens*K]; the tokens routed to expert e
 * are perm[offsets[e] .. offsets[e+1]) / K. Slots with an id outside [0, E) are dropped and flagged. */
int zc_moe_permute(zc_moe* moe, const int32_t* ids, uint32_t tokens, int32_t* offsets, int32_t* perm, void* stream);

/* Replaces the moe_sum dispatch (kernels/metal/qwen.metal:804-816, src/engine/model.cpp:553-555) on caller tensors
 * (parity hook, like zc_moe_route): out[t, :] = sum over slots in the reference's fixed order of weights[t, j] *
 * expert_out[t, j, :] (slots with ids[t, j] < 0 count as zero) + sigmoid(gate_logit[t]) * shared[t, :], with the
 * handle's arithmetic mode and output dtype. expert_out [tokens, K, H] fp32, weights [tokens, K] fp32, ids
 * [tokens, K] int32, shared [tokens, H] fp32 and gate_logit [tokens] fp32 (both or neither), device memory. */
int zc_moe_combine(zc_moe* moe, const float* expert_out, const float* weights, const int32_t* ids, const float* shared,
                   const float* gate_logit, uint32_t tokens, void* out, void* stream);

/* The BF16-staged sigmoid and SiLU of the reference arithmetic (sigmoid_bf, kernels/metal/qwen.metal:33-35, and the
 * activation of q4_gate_up :71-81), element by element on n fp32 device values (parity hook for the reference's
 * 64-point activation tables, tests/test_qwen.cpp:876-897). Either output may be NULL. Runs on the current device. */
int zc_activation_bf16(const float* x, uint32_t n, float* sigmoid_out, float* silu_out, void* stream);

/* Replaces Buf Model::moe(x, layer, tokens, ...) (src/engine/model.cpp:431-557) for short batches —
 * the reference's decode / short-append branch (encode_expert_rows with q4_gate_mv_r2 / q4_mv_r*,
 * src/engine/pipeline.cpp:24-25): memory-bound kernels that stream each selected record once.
 * x [tokens, H] in act_dtype, out [tokens, H] in out_dtype, device memory, must not overlap. */
int zc_moe_decode(zc_moe* moe, uint32_t layer, const void* x, uint32_t tokens, void* out, void* stream);

/* Same contract for long batches — the reference's prefill panels (src/engine/prefill.cpp:66,
 * pipeline.cpp:18-30: gathered q4_gate_up + q4_mm + scatter_experts per expert): one grouped
 * GEMM over all experts' row groups on the tensor cores. */
int zc_moe_prefill(zc_moe* moe, uint32_t layer, const void* x, uint32_t tokens, void* out, void* stream);

/* Model::moe with the family chosen from `tokens`. */
int zc_moe_forward(zc_moe* moe, uint32_t layer, const void* x, uint32_t tokens, void* out, void* stream);

/* The steps either side of Model::moe in the layer loop (src/engine/model.cpp:653, 659-662): the reference keeps four
 * residual streams of width H ("hyper connections").
 *   zc_moe_hc_mix replaces the hc_mix dispatch of Model::hyper (src/engine/model.cpp:343, kernels/metal/qwen.metal:582-588):
 *     x[t, d] = bf(bf(bf(bf(p0 + p1) + p2) + p3) / 4) with p_h = bf(normed[t, h, d] * mix[t, h, d]); normed and mix are
 *     fp32 [tokens, 4, H] device memory, x [tokens, H] is written in the handle's activation dtype (what zc_moe_forward reads).
 *   zc_moe_forward_hc is zc_moe_forward with hc_add (qwen.metal:589-595, dispatched at model.cpp:660-662) as the combine's
 *     epilogue: hyper_out[t, h, d] = bf(hyper[t, h, d] + bf(m[t, d] * inject[t, h])), m = the layer's output, which is not
 *     written anywhere (the roundings apply under ZC_ARITH_REFERENCE; otherwise the sum is plain fp32 on m rounded to the
 *     handle's output dtype). hyper, hyper_out: fp32 [tokens, 4, H] (may be the same buffer); inject: fp32 [tokens, 4]. */
int zc_moe_hc_mix(zc_moe* moe, const float* normed, const float* mix, uint32_t tokens, void* x, void* stream);
int zc_moe_forward_hc(zc_moe* moe, uint32_t layer, const void* x, uint32_t tokens, const float* hyper, const float* inject,
                      float* hyper_out, void* stream);

/* Model::moe with the expert selection given instead of searched: the replay of a recorded route
 * (include/engine/route_trace.hpp:44-49 records the ids of every layer; src/engine/bench.cpp:43-104 replays them).
 * ids [tokens, K] int32 device memory, in rank order; the router still runs (its scores of the given experts give
 * the weights, renormalised over the selection exactly as Metal::route does; row E gives the shared gate), the top-k
 * search does not. With the ids a normal call selected, the output equals that call's bit for bit. */
int zc_moe_forward_routed(zc_moe* moe, uint32_t layer, const void* x, uint32_t tokens, const int32_t* ids, void* out, void* stream);

/* Expert parallelism over the ranks of one node (no counterpart in the reference, a single-GPU engine).
 * A handle created with first_expert / local_experts holds one contiguous range of every layer's experts;
 * router, shared expert and shared gate are replicated. Per layer and rank:
 *   zc_moe_ep_dispatch: router + route + permutation of the local tokens over ALL experts; writes the token
 *     rows in expert order (rows [tokens*K, H], act dtype) and their expert ids (row_experts [tokens*K]).
 *     Rows for one owner rank are contiguous; the split sizes are differences of the permutation offsets
 *     (zc_moe_last_routing) at the ranks' expert boundaries. The caller exchanges rows and ids (all-to-all).
 *   zc_moe_ep_experts: the routed experts of this handle on n_rows received rows (any order, each tagged with
 *     its global expert id inside this handle's range); y [n_rows, H] fp32 in the same row order.
 *     n_rows <= max_tokens * top_k * ranks.
 *   zc_moe_ep_combine: y_sorted [tokens*K, H] fp32 — the results of this rank's own rows, returned by the
 *     reverse all-to-all in the order zc_moe_ep_dispatch wrote them — is scattered to the router slots and
 *     reduced in fixed slot order with the locally computed shared expert into out. */
int zc_moe_ep_dispatch(zc_moe* moe, uint32_t layer, const void* x, uint32_t tokens, void* rows, int32_t* row_experts, void* stream);
int zc_moe_ep_experts(zc_moe* moe, uint32_t layer, const void* rows, const int32_t* row_experts, uint32_t n_rows, float* y, void* stream);
int zc_moe_ep_combine(zc_moe* moe, uint32_t layer, const void* x, uint32_t tokens, const float* y_sorted, void* out, void* stream);

/* Expert parallelism without a collective library and without any host value in the loop: every rank's handle
 * owns a window of device memory that the other ranks of the node map over NVLink; rows, results and flags
 * travel as plain peer stores issued by this library's kernels (no TMA, no multicast). No counterpart in the
 * reference.
 *   zc_moe_ep_export: the window's address (ranks inside one process) and / or its 64-byte inter-process handle
 *     (cudaIpcGetMemHandle) — either output may be NULL.
 *   zc_moe_ep_attach: peers = world x 64-byte handles (kind 0; the entry of `rank` is ignored) or world device
 *     pointers (kind 1). world must equal experts / local_experts and rank first_expert / local_experts; every
 *     rank uses the same descriptor apart from first_expert. All ranks must have attached (a host barrier)
 *     before any of them issues a layer.
 *   zc_moe_ep_layer: Model::moe for this rank's tokens: routing, rows to their owners, the local experts on
 *     whatever arrived, results back to the router slots of their senders, fixed-order combine. Stream-ordered,
 *     no host synchronisation. Every rank must issue the same sequence of expert-parallel layer calls (a layer
 *     call on one rank waits for the matching call of every other rank). Device-side waits are bounded (option
 *     "ep_wait_ms", default 2000): when a peer does not answer, ZC_STATUS_TIMEOUT is raised, the layer finishes
 *     with whatever arrived, and later waits give up at once until zc_moe_status has cleared the word.
 *   zc_moe_ep_send / _process / _finish: the three phases of zc_moe_ep_layer as separate calls (sender first
 *     half, owner, sender second half), for hosts that emulate several ranks on one device: all ranks' sends,
 *     then all ranks' processing, then all ranks' finishes.
 *   zc_moe_ep_stack: the chained stack of zc_moe_stack with expert-parallel layers, replayed from a CUDA graph. */
int zc_moe_ep_export(zc_moe* moe, void* handle64, void** window);
int zc_moe_ep_attach(zc_moe* moe, uint32_t rank, uint32_t world, const void* peers, int kind);
int zc_moe_ep_layer(zc_moe* moe, uint32_t layer, const void* x, uint32_t tokens, void* out, void* stream);
int zc_moe_ep_send(zc_moe* moe, uint32_t layer, const void* x, uint32_t tokens, void* stream);
int zc_moe_ep_process(zc_moe* moe, uint32_t layer, void* stream);
int zc_moe_ep_finish(zc_moe* moe, uint32_t layer, const void* x, uint32_t tokens, void* out, void* stream);
int zc_moe_ep_stack(zc_moe* moe, const void* x, uint32_t tokens, void* out, void* stream);
int zc_moe_ep_stack_eager(zc_moe* moe, const void* x, uint32_t tokens, void* out, void* stream);

/* Model::moe for callers that hold HOST tensors (the reference's Buf is CPU-visible unified memory):
 * on `stream`, copies x in, runs zc_moe_forward, copies out back, then waits for the stream.
 * x_host/out_host: host memory (pinned memory makes the copies asynchronous to other streams).
 * The _async form returns after enqueueing; out_host is valid once the caller has waited for `stream`
 * (cudaStreamSynchronize, an event, or zc_moe_status, which also returns the device status word) — the
 * counterpart of the reference's asynchronous encode followed by one finish() (src/engine/metal.mm:442). */
int zc_moe_forward_host(zc_moe* moe, uint32_t layer, const void* x_host, uint32_t tokens, void* out_host, void* stream);
int zc_moe_forward_host_async(zc_moe* moe, uint32_t layer, const void* x_host, uint32_t tokens, void* out_host, void* stream);

/* The reference's cancel flag (const std::atomic<bool>* cancel of Model::moe, include/engine/model.hpp:156; read at
 * the stage boundaries of src/engine/pipeline.cpp:160-208). `flag` points to host memory another thread may set to
 * non-zero (NULL removes it). It is read on the host when a layer call is validated, before every layer of a stack
 * that is issued launch by launch, and once more by zc_moe_stack_host after its wait; the call then returns
 * ZC_ECANCELLED ("generation cancelled", src/engine/model.cpp:15) and issues nothing further. Work already
 * enqueued (a graph replay is one unit) runs to completion. */
int zc_moe_set_cancel(zc_moe* moe, const int32_t* flag);

/* The whole stack of `layers` MoE layers chained on one stream, layer l+1 reading
 * act_dtype((out_l - mean(out_l)) / std(out_l)) per token — the stand-in for the residual + norm between
 * MoE layers that the measurement uses so that no cross-layer overlap is credited. out receives the last
 * layer's output. */
int zc_moe_stack(zc_moe* moe, const void* x, uint32_t tokens, void* out, void* stream);
int zc_moe_stack_host(zc_moe* moe, const void* x_host, uint32_t tokens, void* out_host, void* stream);

/* Kernel policy switches, the counterpart of KernelConfig (include/engine/metal.hpp:17-43). Options:
 *   "fold_q4" (default 1): Q4 codes enter the tensor-core product as 1024+q / 1024+16q and the offset is
 *   removed from the FP32 group sum; 0 removes it in FP16 before the product (exact, more instructions).
 *   "pdl" (default 1; environment ZC_MOE_PDL=0 at create time): the kernels of a layer are launched with
 *   programmatic stream serialization, so that each one's set-up and weight prefetch overlap the tail of the
 *   kernel before it; results are identical either way.
 *   "exact_h" (default 0): the decode family's down product reads the FP32 SwiGLU rows as two FP16 terms (nothing
 *   below FP32 is rounded) instead of one FP16 term (11 significant bits; the reference rounds these rows to BF16).
 *   "ep_wait_ms" (default 2000): limit of one device-side wait for a peer's flag in the expert-parallel layer.
 *   "prefill_wide" (default 1): long batches use the wide-tile grouped GEMM (accumulators and weights in tensor memory);
 *   0 selects the earlier per-group-drain kernel.
 *   "prefill_small_rows" (default 16, 0..64): in a long batch, experts with at most this many rows run on the streaming
 *   kernels and the grouped GEMM takes the others (0: the grouped GEMM takes every expert).
 *   "few_tiles_gate_up" (default 1), "few_tiles_down" (default 2), 1..4: 16-row tiles per warp of those streaming
 *   launches (few experts have work there: fewer tiles per warp mean more, shorter CTAs per expert).
 *   "meta_blocks" (default 1): the streaming kernels fetch scales and biases eight groups at a time (16-byte copies)
 *   for gate/up at hidden >= 4096; 2 does so wherever the layout allows, 3 uses four-group blocks for gate/up, 0 never
 *   (each ring stage's own halves, 4- or 8-byte copies). Results are identical.
 *   "router_db" (default 1): long batches with FP32 router rows and BF16 activations use the double-buffered router
 *   tiles; 0 selects the single-buffer form. Results are identical.
 * Changing an option drops the cached graphs of zc_moe_stack. */
int zc_moe_set_option(zc_moe* moe, const char* name, int value);

/* zc_moe_stack without graph replay: the same launches issued one by one (used with the profiler below). */
int zc_moe_stack_eager(zc_moe* moe, const void* x, uint32_t tokens, void* out, void* stream);

/* Per-kernel device timing, the counterpart of KernelConfig.profile / Metal::take_profile
 * (include/engine/metal.hpp:31, 93; src/engine/metal.mm:510-557): between begin and end every kernel
 * launched outside a graph is bracketed by CUDA events on its stream. end waits for the device and returns,
 * per kernel kind k < 16, the summed milliseconds and the number of launches; zc_moe_kernel_name(k) names it. */
int zc_moe_profile_begin(zc_moe* moe);
int zc_moe_profile_end(zc_moe* moe, double* ms_per_kind, uint64_t* launches_per_kind);
const char* zc_moe_kernel_name(int kind);

/* Device buffers holding the last call's routing (the reference exposes the same tensors through
 * --trace-dir: route_l, .weights, src/engine/model.cpp:447-448, 549-552). Valid until the next call. */
int zc_moe_last_routing(zc_moe* moe, const int32_t** ids, const float** weights,
                        const int32_t** offsets, const int32_t** perm, const float** logits);

/* Number of routed experts that received work in the most recent call of each layer, host_counts[layers]
 * (the reference reports the same through its route trace, include/engine/route_trace.hpp). Blocking. */
int zc_moe_active_counts(zc_moe* moe, int32_t* host_counts);
/* The same for the owner side of expert parallelism: experts of this handle's range that received rows (from any
 * rank) in the most recent expert-parallel call of each layer. Blocking. */
int zc_moe_ep_active_counts(zc_moe* moe, int32_t* host_counts);

/* Blocking copy of handle-owned device memory (a resident tensor or the routing buffers above) to the host;
 * waits for all earlier work on the device. The reference reads the same tensors in place (unified memory). */
int zc_moe_read_device(zc_moe* moe, void* host_dst, const void* device_src, uint64_t bytes);

/* Waits for the handle's work on `stream` and returns the device status word (then clears it). */
int zc_moe_status(zc_moe* moe, void* stream, uint32_t* status);

/* Runs the give-up path of the tensor-core kernels on its own (a diagnostic; nothing in the reference corresponds to it:
 * its Metal command buffers have no device-side waits). One CTA allocates tensor memory, then two of its roles wait -
 * with the bounded waits the kernels use - on an mbarrier that nothing arrives on: after `polls` attempts (1..100000,
 * about a microsecond each) the wait gives up, raises the CTA's abort flag and ZC_STATUS_TIMEOUT in the handle's status
 * word (read and cleared by zc_moe_status), the other role leaves on the flag, and the CTA returns its tensor memory.
 * report[0..3] = {suspending wait's result, polling wait's result (0 = gave up), abort flag, TMEM base}. Synchronous. */
int zc_moe_wait_selftest(zc_moe* moe, uint32_t polls, uint32_t report[4], void* stream);

/* Number of kernel launches the handle has issued since creation (graph replays count their nodes). */
uint64_t zc_moe_launch_count(const zc_moe* moe);

/* Seeded synthetic tensors written straight into a layer's HBM buffers (benchmark and test inputs;
 * the definition of the generator is zerocool_b200/synth.py). No counterpart in the reference, which
 * measures on a real checkpoint. */
int zc_synth_fill_layer(zc_moe* moe, uint32_t layer, uint64_t seed, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ZC_MOE_H */
