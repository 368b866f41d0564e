/*
 * turbofieldfare_cuda.h — C ABI of the B200 (sm_100a) routed-expert library.
 *
 * One entry point per reference operator on the routed-expert path. The
 * reference (drumih/turbo-fieldfare) has no FFI for this path: its operators
 * are Swift classes that encode Metal compute passes onto a command buffer.
 * Each function below names the Swift method it replaces (path relative to the
 * reference repository root) and keeps that method's argument meaning:
 *
 *   (MTLBuffer, byteOffset)  ->  (device pointer, byte offset)
 *   MTLCommandBuffer         ->  cudaStream_t (void* here; work is enqueued,
 *                                the call returns immediately)
 *   precondition / throw     ->  non-zero tf_status + tf_last_error()
 *
 * Conventions
 *   - every data pointer is a DEVICE pointer unless its name says host;
 *   - *_off are byte offsets added to the pointer before use;
 *   - the caller owns every buffer, scratch included, and keeps it alive until
 *     the stream has passed the call (as with a committed command buffer);
 *   - no entry point allocates device memory except the *_create functions;
 *   - there is no CPU fallback: without a CUDA device every call fails.
 *
 * Weight format (unchanged from the .gturbo files): MLX affine, group 64.
 *   int4: N/2 bytes per row, low nibble = even column; int8: N bytes per row;
 *   one 16-bit scale and one 16-bit bias per group, w = q * scale + bias.
 *   The planes are BF16 in the format (TF_BF16); TF_FP16 planes are accepted
 *   by the stand-alone GEMVs only.
 */
#ifndef TURBOFIELDFARE_CUDA_H
#define TURBOFIELDFARE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TF_ABI_VERSION 1
#define TF_GROUP_SIZE 64
#define TF_MAX_TOP_K 8          /* MoE.maxStreamedExperts, Kernels/MoE/MoE.swift:32 */
#define TF_MAX_ROUTER_EXPERTS 256
#define TF_MAX_TILE_EXPERTS 16  /* PrefillMoEGrouping.swift:113 */

typedef int tf_status;
enum {
    TF_OK = 0,
    TF_ERR_INVALID_ARGUMENT = 1,   /* a Swift precondition would have trapped */
    TF_ERR_UNSUPPORTED = 2,
    TF_ERR_CUDA = 3,               /* a CUDA runtime call failed; see tf_last_error */
    TF_ERR_ALIGNMENT = 4,
    TF_ERR_OUT_OF_MEMORY = 5,      /* PrefillGroupedRoutedMoEError.allocationFailed */
    TF_ERR_SCRATCH_TOO_SMALL = 6,  /* SharedExpertError.scratchTooSmall */
    TF_ERR_DIMENSION_MISMATCH = 7, /* SharedExpertError.dimensionMismatch */
    TF_ERR_NO_DEVICE = 8,          /* MetalError.noDevice */
    /* PrefillMoEGroupingError cases, in declaration order
       (Kernels/Prefill/MoE/PrefillMoEGrouping.swift:52-62) */
    TF_ERR_GROUPING_INVALID_QUERY_COUNT = 101,
    TF_ERR_GROUPING_INVALID_TOP_K = 102,
    TF_ERR_GROUPING_INVALID_NUM_EXPERTS = 103,
    TF_ERR_GROUPING_INVALID_TILE_EXPERT_COUNT = 104,
    TF_ERR_GROUPING_PAIR_COUNT_MISMATCH = 105,
    TF_ERR_GROUPING_TOKEN_OUT_OF_RANGE = 106,
    TF_ERR_GROUPING_RANK_OUT_OF_RANGE = 107,
    TF_ERR_GROUPING_EXPERT_OUT_OF_RANGE = 108,
    TF_ERR_GROUPING_DUPLICATE_TOKEN_RANK = 109,
    TF_ERR_GROUPING_SORT_KEY_COUNT_MISMATCH = 110,
    /* GTurboFormatError cases (Sources/TurboFieldfareFormat/GTurboFormatV1.swift:25-38) and the
       ModelError cases the .gturbo readers throw */
    TF_ERR_FORMAT_INVALID = 201,
    TF_ERR_FORMAT_OVERFLOW = 202,
    TF_ERR_FORMAT_TRUNCATED = 203,
    TF_ERR_IO = 204,               /* ModelError.posixFailed / missingFile */
    TF_ERR_NOT_FOUND = 205         /* ModelError.tensorNotFound */
};

typedef enum { TF_BF16 = 0, TF_FP16 = 1 } tf_dtype;

/* Nine byte offsets into one expert blob: gate{W,S,B} | up{W,S,B} | down{W,S,B}.
 * Replaces MoEExpertOffsets (Kernels/MoE/MoE.swift:4-29) and the MSL
 * ExpertOffsets (Metal/MoE/moe.metal:62-72); same field order, 36 bytes. */
typedef struct tf_expert_offsets {
    uint32_t gate_w_off, gate_s_off, gate_b_off;
    uint32_t up_w_off, up_s_off, up_b_off;
    uint32_t down_w_off, down_s_off, down_b_off;
} tf_expert_offsets;

/* One quantised projection: three planes + shape. Replaces
 * SharedExpertProjection (Kernels/MoE/SharedExpertInt8.swift:9-31). */
typedef struct tf_projection {
    const void* weights; uint64_t weights_off;
    const void* scales;  uint64_t scales_off;
    const void* biases;  uint64_t biases_off;
    uint32_t rows, cols;
} tf_projection;

/* 16-byte route pair. Replaces PrefillTokenExpertPair
 * (Kernels/Prefill/MoE/PrefillRouter.swift:5-28); layout pinned by
 * Tests/TurboFieldfare/Core/Kernels/Prefill/PrefillRouterTests.swift:12-19. */
typedef struct tf_pair {
    uint32_t token, expert, rank, weight_bits_and_reserved;
} tf_pair;

/* PrefillMoEGroup / PrefillMoETile (PrefillMoEGrouping.swift:4-31). */
typedef struct tf_group { uint32_t expert, pair_start, pair_count; } tf_group;
typedef struct tf_tile { uint32_t group_start, group_count, pair_start, pair_count; } tf_tile;

/* Device-resident routing metadata produced by tf_group_routes_device and
 * consumed by tf_grouped_moe_batched. All pointers are DEVICE buffers the
 * caller owns: sorted_pairs [T*K]; per_expert_offsets, per_expert_counts,
 * groups, chunk_start [E]; chunk_group [T*K/8 + E]; counters [4] =
 * {group count, chunk count, pair count, grouped pairs (less than the pair count when
 * slots of an exchange buffer were empty)}. A chunk is up to 8
 * consecutive sorted pairs of one expert (one pass of the grouped kernels).
 * Replaces PrefillMoEGroupedRoutes (PrefillMoEGrouping.swift:33-50), which the
 * reference builds on the CPU after reading the router output back. */
typedef struct tf_device_routes {
    tf_pair* sorted_pairs;
    uint32_t* per_expert_offsets;
    uint32_t* per_expert_counts;
    tf_group* groups;
    uint32_t* chunk_group;
    uint32_t* chunk_start;
    uint32_t* counters;
} tf_device_routes;

typedef struct tf_context tf_context;

/* ---- context: replaces MetalContext (Infrastructure/Metal/MetalContext.swift:51-214) ---- */
tf_status tf_context_create(int device, tf_context** out);
void tf_context_destroy(tf_context* ctx);
/* Message of the last failing call on this context (or of the last failing
 * context-less call when ctx is NULL). Never NULL. */
const char* tf_last_error(tf_context* ctx);
int tf_abi_version(void);
/* Number of kernels this context has enqueued since creation (for callers that
 * need to show that work ran on the GPU). */
uint64_t tf_launch_count(tf_context* ctx);
/* Block forwards (tf_moe_block_forward, tf_stack_forward) of at least `tokens` tokens run their expert
 * GEMMs on the tcgen05 tensor cores, smaller ones on the CUDA-core streaming kernels. Default 256. Set it
 * before creating the workspaces that should be able to take the tensor-core path. The reference picks its
 * prefill kernels by chunk size in the same way (RealForwardRunner.swift:902-1186). */
tf_status tf_context_set_tensorcore_min_tokens(tf_context* ctx, uint32_t tokens);
/* The same threshold for the shared expert of a block alone (a dense GEMM over all tokens of the block).
 * Default 256, like the routed experts: measured at 8, 16, 32 and 64 tokens the streaming kernels were faster
 * (1.07 ms against 1.22 ms for six layers at 64 tokens). */
tf_status tf_context_set_shared_tensorcore_min_tokens(tf_context* ctx, uint32_t tokens);
/* Router calls over at least `rows` rows (default 256) take two launches: every logit on the tensor cores with a bound
 * on its distance from the canonical fp32 value, then the canonical logit (the reference's order of operations,
 * Metal/MoE/moe.metal:135-185) of the experts that can still reach the top k, typically top_k + 1 or 2 of them.
 * Indices and weights are those of the one-launch kernels bit for bit. UINT32_MAX keeps the one-launch kernel. Calls
 * that ask for the logits (out_logits) always take the one-launch kernel. */
tf_status tf_context_set_router_tensorcore_min_rows(tf_context* ctx, uint32_t rows);
/* Expert parallelism with fixed-capacity exchanges (decode steps): when ranks * tokens * top_k / (experts of a rank), the
 * expected rows per local expert, reaches `rows`, the owner's expert phase runs on the tensor cores instead of the
 * streaming kernels. Off by default (UINT32_MAX): at eight ranks x 64 tokens (32 rows per expert) the tensor-core phase
 * with its gather and copy-back launches took 6.62 ms per step against 5.98 ms. Read by tf_ep_buffers_create. */
tf_status tf_context_set_ep_tensorcore_min_rows_per_expert(tf_context* ctx, uint32_t rows);
/* Profiling aid with no counterpart in the reference: when a device buffer of `capacity` 64-bit words is set, the
 * single-launch one-token step of tf_stack_forward stamps the GPU's global nanosecond timer at every phase boundary
 * (eight stamps per layer: start, norm, router + shared gate/up, barrier, routed gate/up, barrier, down + combine,
 * barrier). NULL switches it off (the default). */
tf_status tf_context_set_step_trace(tf_context* ctx, void* device_u64, uint32_t capacity);
/* Chooses how tf_stack_forward runs a ONE-token step: as one persistent launch that walks all layers with grid
 * barriers between the phases of a layer (enabled != 0), or layer by layer with the kernels of the block forward
 * (0). New entry point: the reference has no equivalent of either (its decode step is one command buffer per
 * phase, RealForwardRunner.swift:1449-1693). */
tf_status tf_context_set_single_launch_step(tf_context* ctx, int enabled);
/* Synchronises the device and reports whether any kernel abandoned one of its bounded waits
 * (mbarrier / flag polls never spin for ever: on expiry the kernel records a code and returns).
 * Replaces the command-buffer error check (Infrastructure/Metal/MetalContext.swift:22-26).
 * *code_out is 0 when healthy; a non-zero code also returns TF_ERR_CUDA and clears the word. */
tf_status tf_device_status(tf_context* ctx, uint32_t* code_out);

/* ---- stand-alone GEMVs ---- */
/* y[m] = deq4(W[m,n]) . x[n]; x, y fp16; fp32 accumulation.
 * Replaces DequantInt4GEMV.encode (Kernels/Quant/DequantInt4GEMV.swift:44-87):
 * requires n % 64 == 0 and an even weights offset (:57-62). */
tf_status tf_int4_gemv(tf_context* ctx, void* stream,
                       const void* weights, uint64_t weights_off,
                       const void* scales, uint64_t scales_off,
                       const void* biases, uint64_t biases_off,
                       const void* x, uint64_t x_off, void* y, uint64_t y_off,
                       uint32_t m, uint32_t n, tf_dtype sb_dtype);
/* `count` such GEMVs in ONE launch over matrices of one shape whose three planes repeat every matrix_stride_bytes
 * (e.g. the gate tensor of consecutive expert blobs: stride = the blob stride): y[b] = deq4(W[b]) . x[b]. x and y
 * advance by their strides in elements per matrix; x_stride_elements 0 multiplies every matrix with the same vector.
 * New entry point: the reference encodes one DequantInt4GEMV per matrix (DequantInt4GEMV.swift:44-87); this is
 * how a sweep of expert-sized GEMVs reaches HBM speed. Same preconditions as tf_int4_gemv. */
tf_status tf_int4_gemv_batched(tf_context* ctx, void* stream,
                               const void* weights, uint64_t weights_off,
                               const void* scales, uint64_t scales_off,
                               const void* biases, uint64_t biases_off,
                               uint64_t matrix_stride_bytes,
                               const void* x, uint64_t x_off, uint32_t x_stride_elements,
                               void* y, uint64_t y_off, uint32_t y_stride_elements,
                               uint32_t m, uint32_t n, uint32_t count, tf_dtype sb_dtype);
/* Replaces DequantInt8GEMV.encode (Kernels/Quant/DequantInt8GEMV.swift:50-81). */
tf_status tf_int8_gemv(tf_context* ctx, void* stream,
                       const void* weights, uint64_t weights_off,
                       const void* scales, uint64_t scales_off,
                       const void* biases, uint64_t biases_off,
                       const void* x, uint64_t x_off, void* y, uint64_t y_off,
                       uint32_t m, uint32_t n, tf_dtype sb_dtype);

/* ---- router ---- */
/* logits = deq8(W) . (hidden * effective_scale); top-8, ties to the lower
 * index; weights = softmax(top-8 logits) * per_expert_scale -> fp16. The ids
 * stay on the device. Replaces MoE.encodeRouterGemma4
 * (Kernels/MoE/MoE.swift:109-159): d % 64 == 0, num_experts <= 256, top_k == 8.
 * out_logits (fp32 [num_experts], device) may be NULL. */
tf_status tf_router_gemma4(tf_context* ctx, void* stream,
                           const void* weights, uint64_t weights_off,
                           const void* scales, uint64_t scales_off,
                           const void* biases, uint64_t biases_off,
                           const void* hidden,
                           const void* effective_scale, uint64_t effective_scale_off,
                           const void* per_expert_scale, uint64_t per_expert_scale_off,
                           uint32_t* out_indices, void* out_weights, float* out_logits,
                           uint32_t num_experts, uint32_t d, uint32_t top_k);
/* The same for query_count rows with a row stride. Replaces
 * PrefillRouter.encodeGemma4Block (Kernels/Prefill/MoE/PrefillRouter.swift:37-89):
 * query_count > 0, num_experts <= 256, 1 <= top_k <= 64 (this library: <= 8),
 * hidden_stride_elements >= d. hidden_dtype selects fp16 or bf16 rows.
 * logit_bias (fp32 [num_experts], device, may be NULL) is added to the logits
 * before selection (used to skew synthetic routing); out_logits may be NULL. */
tf_status tf_router_gemma4_block(tf_context* ctx, void* stream,
                                 const void* weights, uint64_t weights_off,
                                 const void* scales, uint64_t scales_off,
                                 const void* biases, uint64_t biases_off,
                                 const void* hidden, uint64_t hidden_off, tf_dtype hidden_dtype,
                                 const void* effective_scale, uint64_t effective_scale_off,
                                 const void* per_expert_scale, uint64_t per_expert_scale_off,
                                 const float* logit_bias,
                                 uint32_t* out_indices, uint64_t out_indices_off,
                                 void* out_weights, uint64_t out_weights_off, float* out_logits,
                                 uint32_t query_count, uint32_t num_experts, uint32_t d,
                                 uint32_t top_k, uint32_t hidden_stride_elements);

/* ---- decode routed experts ---- */
/* acts[k*f + j] = half(gelu_tanh(gate_k[j,:].x) * (up_k[j,:].x)) for the top_k
 * blobs in the DEVICE table blobs[top_k]. Replaces
 * MoE.encodeRoutedPersistentPhase1U16Load (Kernels/MoE/MoE.swift:180-213). */
tf_status tf_moe_phase1(tf_context* ctx, void* stream,
                        const void* const* blobs, const tf_expert_offsets* offsets,
                        const void* x, void* acts, uint32_t d, uint32_t f, uint32_t top_k);
/* Same over active_slots[active_count] (device u32). Replaces
 * MoE.encodeRoutedPersistentPhase1SubsetU16Load (MoE.swift:215-258). */
tf_status tf_moe_phase1_subset(tf_context* ctx, void* stream,
                               const void* const* blobs, const tf_expert_offsets* offsets,
                               const void* x, void* acts, uint32_t d, uint32_t f, uint32_t top_k,
                               const uint32_t* active_slots, uint32_t active_count);
/* y[d] = half(residual[d] + sum_k w_k * (down_k[d,:] . acts_k)), slot order.
 * Replaces MoE.encodeRoutedPersistentPhase2Reduce (MoE.swift:260-295). */
tf_status tf_moe_phase2_reduce(tf_context* ctx, void* stream,
                               const void* const* blobs, const tf_expert_offsets* offsets,
                               const void* acts, const void* routing_weights,
                               const void* residual, void* y,
                               uint32_t d, uint32_t f, uint32_t top_k);
/* Fills the device table blobs[t*top_k + r] = pool_base + indices[t*top_k+r] * stride
 * without a host round trip. Replaces Model.routedExpertBuffers /
 * routedExpertOffsets (Runtime/Inference/ModelExpertIO.swift:21-142), whose
 * CPU read-back of the ids exists only because experts lived on SSD. */
tf_status tf_expert_table_from_indices(tf_context* ctx, void* stream,
                                       const void* pool_layer_base, uint64_t expert_stride,
                                       const uint32_t* indices, uint32_t count, uint32_t num_experts,
                                       const void** blobs_out);

/* ---- shared expert ---- */
/* y = down(half(gelu(half(gate.x)) * half(up.x))). Replaces
 * SharedExpertInt4.encode (Kernels/MoE/SharedExpertInt4.swift:30-93). The
 * *_bytes arguments are the sizes of the buffers behind x, y and the three
 * scratch pointers, checked as the reference checks MTLBuffer.length. */
tf_status tf_shared_expert_int4(tf_context* ctx, void* stream,
                                const void* x, uint64_t x_off, uint64_t x_bytes,
                                const tf_projection* gate, const tf_projection* up,
                                const tf_projection* down,
                                void* y, uint64_t y_off, uint64_t y_bytes,
                                void* scratch_gate, uint64_t scratch_gate_off, uint64_t scratch_gate_bytes,
                                void* scratch_up, uint64_t scratch_up_off, uint64_t scratch_up_bytes,
                                void* scratch_act, uint64_t scratch_act_off, uint64_t scratch_act_bytes);

/* ---- routing metadata (host) ---- */
/* Replaces PrefillRouter.makeTokenExpertPairs (PrefillRouter.swift:91-111). HOST arrays. */
tf_status tf_make_token_expert_pairs(const uint32_t* host_indices, const uint16_t* host_weights_f16,
                                     uint32_t query_count, uint32_t top_k, tf_pair* host_pairs_out);
/* Validate, sort by (sort key, expert, token, rank), build offsets (UINT32_MAX
 * when unused), counts, groups and tiles. HOST arrays; outputs sized
 * pair_count / num_experts / pair_count / pair_count. Replaces
 * PrefillMoEGrouping.groupTokenExpertPairs (PrefillMoEGrouping.swift:91-193). */
tf_status tf_group_pairs(const tf_pair* host_pairs, uint32_t pair_count,
                         int32_t query_count, int32_t top_k, int32_t num_experts,
                         int32_t tile_expert_count,
                         const uint64_t* host_expert_sort_keys, uint32_t sort_key_count,
                         tf_pair* sorted_out, uint32_t* per_expert_offsets, uint32_t* per_expert_counts,
                         tf_group* groups_out, uint32_t* group_count_out,
                         tf_tile* tiles_out, uint32_t* tile_count_out);

/* ---- batched routing on the device ---- */
/* Device form of groupTokenExpertPairs for router output that never leaves the
 * GPU: order (expert, token, rank), ids clamped to num_experts-1 as the caller
 * does (Runtime/Inference/RealForwardRunner.swift:955); an id of UINT32_MAX marks an
 * empty slot and is skipped. No sort keys and no
 * tiles: tiles exist in the reference only to bound SSD slots. Replaces the
 * CPU stage PrefillRouter.makeTokenExpertPairs + PrefillMoEGrouping
 * (RealForwardRunner.swift:945-979). From 4096 pairs on the call is three
 * launches that share a scratch area of the context, so such calls on one
 * context must not overlap (use one stream, or a context per stream). */
tf_status tf_group_routes_device(tf_context* ctx, void* stream,
                                 const uint32_t* indices, const void* weights_f16,
                                 uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                                 const tf_device_routes* routes);
/* tf_router_gemma4_block followed by tf_group_routes_device. Blocks of at most 64 rows do both in ONE launch: the
 * thread block that finishes the last row also sorts the pairs (decode steps are bound by launch latency, and the
 * grouping of a few hundred pairs is a fraction of a launch). Results are identical to the two calls. */
tf_status tf_router_gemma4_block_grouped(tf_context* ctx, void* stream, const void* weights, uint64_t weights_off,
                                         const void* scales, uint64_t scales_off, const void* biases, uint64_t biases_off,
                                         const void* hidden, uint64_t hidden_off, tf_dtype hidden_dtype,
                                         const void* effective_scale, uint64_t effective_scale_off,
                                         const void* per_expert_scale, uint64_t per_expert_scale_off,
                                         const float* logit_bias, uint32_t* out_indices, void* out_weights,
                                         uint32_t query_count, uint32_t num_experts, uint32_t d, uint32_t top_k,
                                         uint32_t hidden_stride_elements, const tf_device_routes* routes);
/* Per pair: act = half(gelu(gate.x) * (up.x)) into acts_scratch[pair, F] (sorted
 * pair order), then down -> route_partials[(token*top_k + rank)*D + d], fp16
 * (the reference) or fp32 when partials_f32 != 0. Experts are read from the
 * HBM-resident pool: blob(e) = pool_layer_base + e * expert_stride. Replaces
 * PrefillGroupedRoutedMoE.encodeStreamedBatched over all tiles
 * (Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:386-461). */
tf_status tf_grouped_moe_batched(tf_context* ctx, void* stream,
                                 const void* hidden, uint64_t hidden_off, uint32_t hidden_stride_elements,
                                 const void* pool_layer_base, uint64_t expert_stride,
                                 const tf_expert_offsets* offsets, const tf_device_routes* routes,
                                 void* acts_scratch, void* route_partials, int partials_f32,
                                 uint32_t query_count, uint32_t d, uint32_t f, uint32_t top_k);
/* The reference's streamed form of the batched routed experts: one tile of at most 16 live experts bound to blob
 * base addresses, and the 128-byte parameter block whose layout its tests pin
 * (PrefillGroupedRoutedMoEStreamedParams, Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:104-183;
 * Tests/.../Prefill/PrefillGroupedRoutedMoETests+Layout.swift:7-28). */
#define TF_STREAMED_MAX_EXPERTS 16
typedef struct tf_streamed_params {
    uint32_t pair_start;                 /* first sorted pair of the tile */
    uint32_t pair_count;
    uint32_t d;
    uint32_t routed_intermediate;        /* F */
    uint32_t top_k;
    uint32_t hidden_stride_elements;
    uint32_t live_expert_count;
    uint32_t local_expert[TF_STREAMED_MAX_EXPERTS];   /* expert id of local slot i; UINT32_MAX when unused */
    uint32_t gate_w_off, gate_s_off, gate_b_off, up_w_off, up_s_off, up_b_off, down_w_off, down_s_off, down_b_off;
} tf_streamed_params;
/* Replaces PrefillGroupedRoutedMoE.encodeStreamedBatched (PrefillGroupedRoutedMoE.swift:386-461) for the sorted pairs
 * [pair_start, pair_start + pair_count): per pair gate, up, act = half(gelu(g) * u), down, written to
 * route_partials[(token * top_k + rank) * d] as fp16. `blobs` is a HOST array of blob_count device addresses, blob i
 * holding expert params->local_expert[i] (the views of PrefillStreamedTileBinding, :185-214); every expert of the pair
 * range must be bound (a pair of an unbound expert is skipped and tf_device_status reports 0x7F000031).
 * gate_up_act_scratch holds pair_count * F fp16; the reference's second scratch is not needed. The call does all pairs
 * at once; pair_microbatch_rows only sets *microbatches_out (the reference's return value) and must be positive.
 * As there, pair_count == 0, live_expert_count != blob_count or pair_microbatch_rows == 0 do nothing and return TF_OK
 * with *microbatches_out = 0. At most 65536 pairs per call. */
tf_status tf_grouped_moe_streamed(tf_context* ctx, void* stream,
                                  const void* hidden, uint64_t hidden_off,
                                  const void* sorted_pairs, uint64_t sorted_pairs_off,
                                  void* route_partials, uint64_t route_partials_off,
                                  void* gate_up_act_scratch, uint64_t gate_up_act_scratch_off,
                                  const void* const* blobs, uint32_t blob_count, const tf_streamed_params* params,
                                  uint32_t pair_microbatch_rows, uint32_t* microbatches_out);
/* h2[t,d] = half(sum_r w[t,r] * partial[t,r,d] (+ residual[t,d])), rank order.
 * Replaces PrefillMoE.encodeReduceTokenMajor (Kernels/Prefill/MoE/PrefillMoE.swift:11-39);
 * residual may be NULL (the reference has none); with fp32 partials the order is
 * the decode kernel's (Metal/MoE/moe.metal:473-480). */
tf_status tf_moe_reduce_token_major(tf_context* ctx, void* stream,
                                    const void* route_partials, int partials_f32,
                                    const void* route_weights,
                                    const void* residual, uint32_t residual_stride_elements,
                                    void* h2, uint32_t h2_stride_elements,
                                    uint32_t query_count, uint32_t top_k, uint32_t d);
/* Shared expert for `rows` tokens at once (weights read from HBM once; one pass per 8 tokens).
 * Replaces PrefillSharedExpert.encodeBlock (Kernels/Prefill/MoE/PrefillSharedExpert.swift:11-59),
 * which loops SharedExpertInt4.encode over the rows. scratch_act: [rows, gate.rows] fp16. */
tf_status tf_shared_expert_int4_block(tf_context* ctx, void* stream,
                                      const void* x, uint64_t x_off, uint32_t x_stride_elements,
                                      const tf_projection* gate, const tf_projection* up,
                                      const tf_projection* down,
                                      void* y, uint64_t y_off, uint32_t y_stride_elements,
                                      void* scratch_act, uint32_t rows);

/* The 8-bit shared expert for a block of rows: fused gate/up projection with act = half(gelu(half(gate)) * half(up)),
 * then the 8-bit down projection. Replaces SharedExpertInt8.encode (Kernels/MoE/SharedExpertInt8.swift:55-210;
 * shared_int8_gate_up_act_simd, Metal/Quant/dequant_int8.metal:98-154) and its row loop in
 * PrefillSharedExpert.encodeBlock. scratch_act holds rows * gate.rows fp16. Dimension errors as there
 * (TF_ERR_DIMENSION_MISMATCH). Packed planes may sit at any byte offset, 16-bit planes at even offsets. */
tf_status tf_shared_expert_int8_block(tf_context* ctx, void* stream,
                                      const void* x, uint64_t x_off, uint32_t x_stride_elements,
                                      const tf_projection* gate, const tf_projection* up, const tf_projection* down,
                                      void* y, uint64_t y_off, uint32_t y_stride_elements,
                                      void* scratch_act, uint32_t rows);
/* The shared expert block for callers that cannot allocate device memory. It has no counterpart in the
 * reference. Who needs it: a serving process that hands all of the GPU's memory to its own pool at start-up and
 * never calls cudaMalloc again (a later cudaMalloc would fail, or stall the device while the driver maps
 * memory); a plugin loaded into such a process; code that runs while another thread captures a CUDA graph,
 * where an allocation is an error. Everything else in this header needs a tf_context, a workspace or a
 * caller-provided scratch buffer, and each of those is a device allocation by somebody.
 * This call takes no context and no scratch: x, the three projections and y are the caller's buffers, and the
 * fp16 activations between the gate/up kernel and the down kernel go to an array that is part of the library
 * image (1 MiB per GPU that loads the library, held until the process exits). It calls no cudaMalloc, cudaFree
 * or other allocating routine.
 *   - Limit: rows * gate->rows * 2 bytes <= 1 MiB (248 rows at the Gemma-4 shared width 2112); a larger block
 *     returns TF_ERR_SCRATCH_TOO_SMALL and the message names tf_shared_expert_int4_block as the way out.
 *   - The first call on a device looks up the array's device address and the SM count and sets the kernels'
 *     shared-memory attribute; make that first call with the device current and before any stream capture.
 *   - All calls on a device share the one array, which still holds the previous call's activations. Nothing in
 *     it has to start at zero; the status word is cleared by every call. Two calls that overlap on the GPU
 *     (different streams, or graphs replayed concurrently) race on the array and corrupt each other.
 *   - device_status: optional DEVICE word owned by the caller; it is cleared, and a kernel that gives up a
 *     bounded wait writes its code there. NULL uses a word inside the library that cannot be read back.
 *   - Errors: the status is returned and tf_last_error(NULL) holds the text. Arithmetic, alignment rules and
 *     arguments otherwise as tf_shared_expert_int4_block. */
tf_status tf_shared_expert_int4_block_noalloc(void* stream,
                                              const void* x, uint64_t x_off, uint32_t x_stride_elements,
                                              const tf_projection* gate, const tf_projection* up,
                                              const tf_projection* down,
                                              void* y, uint64_t y_off, uint32_t y_stride_elements, uint32_t rows,
                                              uint32_t* device_status);

/* ---- tensor-core (tcgen05 / TMEM) kernels for prefill-sized batches ---- */
/* Y[M,N] = X[M,K] . dequant(W[N,K])^T, fp16 in/out, fp32 accumulation; the weight tile is staged as
 * half(q*s+b) and multiplied on the matrix unit. Replaces MPPPrefillInt4QMM.encode
 * (Kernels/TensorCore/MPPPrefillInt4QMM.swift:34-78; Metal/TensorCore/tensorops.metal:13-105).
 * K % 64 == 0 as there; M and N are free. With N % 8 == 0 and 16-byte aligned planes the tcgen05 kernel runs;
 * any other N, any byte offset of the packed plane and any even offset of the 16-bit planes (all accepted by the
 * reference) run a CUDA-core kernel with the arithmetic of the reference's scalar QMM
 * (Metal/Prefill/prefill.metal:672-709). */
tf_status tf_int4_qmm(tf_context* ctx, void* stream,
                      const void* weights, uint64_t weights_off,
                      const void* scales, uint64_t scales_off,
                      const void* biases, uint64_t biases_off,
                      const void* x, uint64_t x_off, void* y, uint64_t y_off,
                      uint32_t m, uint32_t n, uint32_t k);
/* The same call reporting which kernel ran, as MPPPrefillInt4QMM.encode returns its Path
 * (MPPPrefillInt4QMM.swift:5-8). Inputs outside the reference's guard (K % 64 != 0, odd offsets of a 16-bit plane,
 * an empty shape) launch nothing, set TF_QMM_PATH_UNAVAILABLE and return TF_OK: the caller falls back, as there. */
typedef enum tf_qmm_path {
    TF_QMM_PATH_UNAVAILABLE = 0,
    TF_QMM_PATH_TENSORCORE = 1,    /* tcgen05 / TMEM (the reference's .affineThreadgroupF16) */
    TF_QMM_PATH_CUDA_CORES = 2     /* unaligned planes or N % 8 != 0 */
} tf_qmm_path;
tf_status tf_int4_qmm_with_path(tf_context* ctx, void* stream,
                                const void* weights, uint64_t weights_off,
                                const void* scales, uint64_t scales_off,
                                const void* biases, uint64_t biases_off,
                                const void* x, uint64_t x_off, void* y, uint64_t y_off,
                                uint32_t m, uint32_t n, uint32_t k, tf_qmm_path* path_out);
/* Gathers the hidden row of every (token, expert) pair into x_sorted[T*top_k, D] in the order of
 * routes->sorted_pairs, with every eight columns stored in the order (0,4,1,5,2,6,3,7) that
 * tf_grouped_moe_tensorcore reads, and records inverse_perm[token*top_k + rank] = sorted row.
 * row_expert_ids[T*top_k] receives each row's expert. Replaces the per-pair hidden gather inside
 * prefill_grouped_routed_moe_batched_phase1 (Metal/Prefill/prefill.metal:598-640). */
tf_status tf_pack_sorted_rows(tf_context* ctx, void* stream, const void* hidden, uint32_t hidden_stride_elements,
                              const tf_device_routes* routes, uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                              uint32_t d, void* x_sorted, uint32_t* row_expert_ids, uint32_t* inverse_perm);
/* Routed experts over expert-sorted rows: x_sorted[x_rows, D] from tf_pack_sorted_rows;
 * acts_scratch[x_rows, F] = half(gelu(gate.x) * (up.x)) (scratch, same permuted column order);
 * out_rows[x_rows, D] = half(down.act) in natural column order, still in sorted row order
 * (tf_ep_combine folds them back per token). Same mathematics as tf_grouped_moe_batched with
 * the weights rounded to half(q*s+b) first, the matrix-unit convention of tensorops.metal:60-75. Replaces
 * PrefillGroupedRoutedMoE.encodeStreamedBatched (Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:386-461)
 * for batches large enough to fill 128-token tiles. */
tf_status tf_grouped_moe_tensorcore(tf_context* ctx, void* stream,
                                    const void* x_sorted, uint32_t x_rows,
                                    const void* pool_layer_base, uint64_t expert_stride, uint32_t num_experts,
                                    const tf_expert_offsets* offsets, const tf_device_routes* routes,
                                    void* acts_scratch, void* out_rows, uint32_t d, uint32_t f);
/* Shared expert for `rows` tokens on the matrix unit; gate and up are rounded to fp16 before the activation
 * like the row kernel (Kernels/MoE/SharedExpertInt4.swift:62-93). Replaces PrefillSharedExpert.encodeBlock
 * (Kernels/Prefill/MoE/PrefillSharedExpert.swift:11-59) for prefill-sized blocks. */
tf_status tf_shared_expert_int4_tensorcore(tf_context* ctx, void* stream,
                                           const void* x, uint32_t x_stride_elements,
                                           const tf_projection* gate, const tf_projection* up,
                                           const tf_projection* down,
                                           void* y, uint32_t y_stride_elements,
                                           void* scratch_act, uint32_t rows);

/* ---- HBM-resident expert pool (replaces SSD streaming) ---- */
/* One allocation of layers * experts blobs of `stride` bytes in the .gturbo blob
 * layout. Replaces PreadExpertStreamer and its LFU slot cache
 * (Infrastructure/Streaming/PreadExpertStreamer.swift:57-414) and
 * Model.routedExpertOffsets / planRoutedExperts / fetchRoutedExperts
 * (Runtime/Inference/ModelExpertIO.swift:21-142): every expert is resident, so a
 * "fetch" is tf_expert_pool_ptr(). tf_expert_pool_create allocates device memory. */
typedef struct tf_pool tf_pool;
tf_status tf_expert_pool_create(tf_context* ctx, uint32_t layers, uint32_t experts, uint64_t stride,
                                const tf_expert_offsets* offsets, tf_pool** out);
void tf_expert_pool_destroy(tf_pool* pool);
/* Device address of a blob; NULL when out of range. */
const void* tf_expert_pool_ptr(const tf_pool* pool, uint32_t layer, uint32_t expert);
uint64_t tf_expert_pool_bytes(const tf_pool* pool);
void tf_expert_pool_dims(const tf_pool* pool, uint32_t* layers_out, uint32_t* experts_out, uint64_t* stride_out);
/* Copy one blob (as stored in packed_experts/layer_XX.bin) from HOST memory. */
tf_status tf_expert_pool_upload(tf_pool* pool, void* stream, uint32_t layer, uint32_t expert,
                                const void* host_blob, uint64_t bytes);
/* Seeded synthetic weights generated on the device: uniform codes, per-group
 * scale |N(0,1)| * 0.004 (8-bit: / 16), bias -zero_point * scale + N(0, 1e-4), bf16. */
tf_status tf_fill_affine_synthetic(tf_context* ctx, void* stream, void* weights, void* scales, void* biases,
                                   uint32_t rows, uint32_t cols, uint32_t bits, uint64_t seed);
/* The pool may be a shard [expert_offset, expert_offset + experts) of global_experts experts (0 = not
 * sharded); blobs are seeded by the global expert id, so shards hold the bytes of the whole pool. */
tf_status tf_expert_pool_fill_synthetic(tf_pool* pool, void* stream, uint64_t seed, uint32_t d, uint32_t f,
                                        uint32_t global_experts, uint32_t expert_offset);
/* The same for a shard that holds an arbitrary selection of the experts: slot e of layer l gets the bytes of expert
 * original_ids[l * experts + e] (HOST array, layers * experts entries, each < global_experts) of the whole pool. */
tf_status tf_expert_pool_fill_synthetic_placed(tf_pool* pool, void* stream, uint64_t seed, uint32_t d, uint32_t f,
                                               uint32_t global_experts, const uint32_t* original_ids);

/* ---- .gturbo model directory -> HBM ----
 * Reader of the installed model format: manifest.json, packed_experts/layout.json, packed_experts/<layer files>
 * and model_weights.bin (24-byte header, 72-byte entries, names, padding to 16 KiB, then the resident tensors).
 * Replaces ManifestReader.decode (Infrastructure/ModelIO/ManifestReader.swift:89-152),
 * PackedExpertsLayoutReader.decode (Infrastructure/ModelIO/PackedExpertsLayout.swift:82-119),
 * ResidentIndexReader.load (Infrastructure/ModelIO/ResidentIndex.swift:49-140) with the validation rules of
 * Sources/TurboFieldfareFormat (GTurboManifestV1.swift:172-268, GTurboPackedExpertsLayoutV1.swift:86-211,
 * GTurboResidentIndexV1.swift:40-158). Architecture fields are reported, not compared with a compiled-in
 * configuration; SHA-256 verification of the payload files is left to the installer. Errors: the status is
 * returned and tf_last_error(NULL) holds the text. None of the parsing calls needs a GPU. */
typedef struct tf_gturbo tf_gturbo;
typedef struct tf_gturbo_info {
    uint32_t version_major, version_minor;
    uint32_t num_layers, experts_per_layer, top_k;
    uint32_t hidden_size, moe_intermediate_size, ffn_intermediate;
    uint32_t shared_expert_bits;      /* manifest.quant.sharedExpert.weightBits; 0 when the manifest has no quant table */
    uint32_t reserved;
    uint64_t expert_stride;
    uint64_t index_size, resident_size, entry_count;   /* header of model_weights.bin */
} tf_gturbo_info;
/* One resident tensor; offsets are relative to the resident payload (file offset minus index_size), as in
 * Model.resident(name:) (Runtime/Inference/Model.swift:195-233). dtype: 0 u32, 1 bf16, 2 fp16, 3 fp32. */
typedef struct tf_gturbo_tensor {
    uint64_t offset, size;
    uint64_t scale_offset, scale_size;
    uint64_t bias_offset, bias_size;
    uint32_t shape[4];
    uint8_t dtype;
    uint8_t reserved[7];
} tf_gturbo_tensor;
tf_status tf_gturbo_open(const char* directory, tf_gturbo** out);
/* The same from memory: the two JSON documents and (at least) the index region of model_weights.bin. */
tf_status tf_gturbo_parse(const void* manifest_json, uint64_t manifest_bytes, const void* layout_json, uint64_t layout_bytes,
                          const void* resident_index, uint64_t resident_index_bytes, tf_gturbo** out);
void tf_gturbo_close(tf_gturbo* g);
tf_status tf_gturbo_get_info(const tf_gturbo* g, tf_gturbo_info* out);
/* Model.routedExpertOffsets (Runtime/Inference/ModelExpertIO.swift:21-40). */
tf_status tf_gturbo_expert_offsets(const tf_gturbo* g, uint32_t layer, tf_expert_offsets* out);
/* PackedExpertsLayout.expert(layer:expert:) by LOGICAL expert id; outputs may be NULL. */
tf_status tf_gturbo_expert_location(const tf_gturbo* g, uint32_t layer, uint32_t expert, const char** file_out,
                                    uint64_t* offset_out, uint64_t* size_out, uint32_t* physical_rank_out);
tf_status tf_gturbo_resident(const tf_gturbo* g, const char* name, tf_gturbo_tensor* out);
tf_status tf_gturbo_resident_name(const tf_gturbo* g, uint64_t position, const char** name_out);
/* Reads every layer file and copies each blob to its logical slot of the pool; a pool that holds a shard
 * takes experts [expert_offset, expert_offset + pool experts). Replaces the pread streamer
 * (Infrastructure/Streaming/PreadExpertStreamer.swift:57-414). Allocates two pinned staging buffers. */
tf_status tf_expert_pool_load_gturbo(tf_pool* pool, void* stream, const tf_gturbo* g, uint32_t expert_offset);

/* ---- fused MoE block and layer stack (new entry points; the reference spreads
 * this over RealForwardRunner with two CPU round trips per layer) ---- */
typedef struct tf_moe_layer {
    tf_projection router;            /* 8-bit affine [num_experts, d] */
    const void* effective_scale;     /* bf16 [d]  (RealForwardRunner.swift:352-376) */
    const void* per_expert_scale;    /* bf16 [num_experts] */
    const float* logit_bias;         /* fp32 [num_experts] or NULL */
    const void* pool_layer_base;     /* tf_expert_pool_ptr(pool, layer, 0) */
    uint64_t expert_stride;
    tf_expert_offsets offsets;
    tf_projection shared_gate, shared_up, shared_down;   /* 4-bit affine */
    uint32_t num_experts, d, f, fs, top_k;
    uint32_t shared_bits;            /* 8: the shared expert is 8-bit affine (SharedExpertInt8); 0 or 4: 4-bit */
} tf_moe_layer;

/* Uploads the resident payload of model_weights.bin and builds one tf_moe_layer per layer from the checkpoint's
 * tensor names (router.proj.weight, router.scale with 1/sqrt(D) folded in as in RealForwardRunner.swift:352-376,
 * router.per_expert_scale, mlp.{gate,up,down}_proj.weight; Runtime/Inference/Model.swift:89-188). `pool` must
 * hold every expert of the model. Allocates device memory; the layers stay valid until the model is destroyed. */
typedef struct tf_gturbo_model tf_gturbo_model;
tf_status tf_gturbo_model_load(tf_context* ctx, void* stream, const tf_gturbo* g, const tf_pool* pool, tf_gturbo_model** out);
void tf_gturbo_model_destroy(tf_gturbo_model* model);
const tf_moe_layer* tf_gturbo_model_layers(const tf_gturbo_model* model, uint32_t* count_out);
const void* tf_gturbo_model_resident_base(const tf_gturbo_model* model);

/* Device scratch for up to max_tokens tokens (router output, routes, activations,
 * partials). Replaces the runner-owned scratch buffers
 * (RealForwardRunner.swift:176-199; Runtime/Prefill/PrefillChunkScratch.swift:79-152).
 * Partials are fp32 when max_tokens <= 64 (decode arithmetic), fp16 otherwise
 * (the prefill kernels' rounding). tf_workspace_create allocates device memory. */
typedef struct tf_workspace tf_workspace;
tf_status tf_workspace_create(tf_context* ctx, uint32_t max_tokens, uint32_t d, uint32_t f, uint32_t fs,
                              uint32_t top_k, uint32_t num_experts, tf_workspace** out);
void tf_workspace_destroy(tf_workspace* ws);
uint64_t tf_workspace_bytes(const tf_workspace* ws);
const uint32_t* tf_workspace_indices(const tf_workspace* ws);   /* device [tokens, top_k] of the last forward */
const void* tf_workspace_weights(const tf_workspace* ws);        /* device fp16 [tokens, top_k] */
const tf_device_routes* tf_workspace_routes(const tf_workspace* ws);

/* y[t] = half(shared(x[t]) + sum_r w[t,r] * routed_{idx[t,r]}(x[t])) for `tokens`
 * fp16 rows: router + top-8 + softmax, device grouping, grouped gate/up + GeGLU,
 * grouped down, shared expert, weighted combine. No host synchronisation. */
tf_status tf_moe_block_forward(tf_context* ctx, void* stream, const tf_moe_layer* layer,
                               const void* x, uint32_t x_stride_elements,
                               void* y, uint32_t y_stride_elements, uint32_t tokens, tf_workspace* ws);
/* The same block on bf16 activation rows (the prefill configuration that names bf16 tiles): x is converted to fp16 on
 * entry -- exact for every bf16 value that is zero or inside fp16's normal range, 6.1e-5 ... 65504 in magnitude, which
 * normalised activations are -- the block runs as above (its fp16 weight tiles carry three more significant bits than
 * bf16 tiles would), and y is rounded to bf16 on exit. Uses the workspace's stack scratch for the fp16 copies. */
tf_status tf_moe_block_forward_bf16(tf_context* ctx, void* stream, const tf_moe_layer* layer,
                                    const void* x_bf16, uint32_t x_stride_elements,
                                    void* y_bf16, uint32_t y_stride_elements, uint32_t tokens, tf_workspace* ws);
/* dst = src converted between fp16 and bf16, row by row (16-byte aligned rows, D a multiple of 8). */
tf_status tf_convert_rows(tf_context* ctx, void* stream, const void* src, tf_dtype src_dtype, uint32_t src_stride_elements,
                          void* dst, tf_dtype dst_dtype, uint32_t dst_stride_elements, uint32_t rows, uint32_t d);

/* A stack of MoE blocks with RMSNorm between layers and a residual stream:
 * x = rmsnorm(h) * w_l; h = h + block_l(x). hidden is fp16 [tokens, d], in place. */
typedef struct tf_stack tf_stack;
tf_status tf_stack_create(tf_context* ctx, const tf_moe_layer* layers, const void* const* norm_weights_bf16,
                          uint32_t layer_count, float eps, tf_stack** out);
void tf_stack_destroy(tf_stack* stack);
tf_status tf_stack_forward(tf_stack* stack, void* stream, void* hidden, uint32_t tokens, tf_workspace* ws);

/* h += y (one fp16 rounding; y may be NULL), then x_out = half(rmsnorm(h) * w) (x_out may be NULL).
 * The residual add of one stack layer fused with the norm of the next; contiguous fp16 rows. */
tf_status tf_residual_rmsnorm(tf_context* ctx, void* stream, void* hidden, const void* y, const void* weight_bf16,
                              void* x_out, uint32_t rows, uint32_t d, float eps);

/* ---- expert parallelism (new; the reference is single-GPU: MetalContext.swift:51-71) ---- */
/* Gather each sorted pair's activation row into the send buffer in (destination rank, expert, token,
 * rank) order, with the expert id local to its owner, and record inverse_perm[token*top_k + rank] = slot.
 * capacity == 0: exact layout, slot = sorted pair index (split sizes come from per_expert_counts).
 * capacity > 0: fixed layout [ranks][capacity] with unused slots marked id = UINT32_MAX (no host
 * synchronisation; an overflowing destination sets the context's device error word).
 * send_row_stride_elements: 0 or D for plain rows; D + 8 or more (a multiple of 8) makes every send row carry its
 * expert id in the four bytes after the D activations, so that one exchange moves rows and ids together. */
tf_status tf_ep_pack(tf_context* ctx, void* stream, const void* hidden, uint64_t hidden_off, uint32_t hidden_stride_elements,
                     const tf_device_routes* routes, uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                     uint32_t experts_per_rank, uint32_t capacity, uint32_t d,
                     void* send_rows, uint32_t* send_expert_ids, uint32_t* inverse_perm, uint32_t send_row_stride_elements);
/* ids[slot] = the expert id that a row of row_stride_elements > D elements carries after its D activations. */
tf_status tf_ep_extract_ids(tf_context* ctx, void* stream, const void* rows, uint32_t row_stride_elements, uint32_t d,
                            uint32_t slots, uint32_t* ids);
/* The three phases of one expert-parallel layer; the caller runs the all-to-all exchanges between them
 * (rows and expert ids out, result rows back).
 *   tf_ep_dispatch: router + top-k + device grouping over the GLOBAL experts + tf_ep_pack;
 *   tf_ep_experts:  on the owner: group the received rows by local expert and run gate/up/GeGLU/down;
 *                   out_rows[slot] is the fp16 expert output of the row received in that slot; with
 *                   recv_row_stride_elements > D the ids are read from the row tails into recv_expert_ids first;
 *   tf_ep_finish:   shared expert on the local tokens + tf_ep_combine of the returned rows. */
tf_status tf_ep_dispatch(tf_context* ctx, void* stream, const tf_moe_layer* layer, const void* x, uint32_t tokens,
                         tf_workspace* ws, uint32_t experts_per_rank, uint32_t capacity,
                         void* send_rows, uint32_t* send_expert_ids, uint32_t* inverse_perm, uint32_t send_row_stride_elements);
tf_status tf_ep_experts(tf_context* ctx, void* stream, const void* pool_layer_base, uint64_t expert_stride,
                        const tf_expert_offsets* offsets, const void* recv_rows, const uint32_t* recv_expert_ids,
                        uint32_t recv_slots, uint32_t local_experts, const tf_device_routes* recv_routes,
                        const void* zero_weights, void* acts_scratch, void* out_rows, uint32_t d, uint32_t f,
                        uint32_t recv_row_stride_elements);
/* tf_ep_experts for prefill-sized exchanges (every received slot holds a row): the same result through the tcgen05
 * grouped GEMMs. Extra scratch: x_sorted and out_sorted [recv_slots, D] fp16, row_ids and inverse_perm [recv_slots],
 * one_weights [recv_slots] fp16 holding 1.0. */
tf_status tf_ep_experts_tensorcore(tf_context* ctx, void* stream, const void* pool_layer_base, uint64_t expert_stride,
                                   const tf_expert_offsets* offsets, const void* recv_rows, const uint32_t* recv_expert_ids,
                                   uint32_t recv_slots, uint32_t local_experts, const tf_device_routes* recv_routes,
                                   const void* zero_weights, const void* one_weights, void* x_sorted, uint32_t* row_ids,
                                   uint32_t* inverse_perm, void* acts_scratch, void* out_sorted, void* out_rows,
                                   uint32_t d, uint32_t f);
tf_status tf_ep_finish(tf_context* ctx, void* stream, const tf_moe_layer* layer, const void* x, uint32_t tokens,
                       tf_workspace* ws, const void* returned_rows, const uint32_t* inverse_perm, void* y);
/* out[t] = half(sum_r w[t,r] * returned_rows[inverse_perm[t*top_k + r]] + residual[t]), rank order. */
tf_status tf_ep_combine(tf_context* ctx, void* stream, const void* returned_rows, const void* route_weights,
                        const uint32_t* inverse_perm, const void* residual, uint32_t residual_stride_elements,
                        void* out, uint32_t out_stride_elements, uint32_t query_count, uint32_t top_k, uint32_t d);

/* ---- expert-parallel exchange over peer memory (decode steps; no reference counterpart: the reference runs on
 * one device) ----
 * A rank allocates one exchange buffer (tf_peer_buffer_create), hands its 64-byte handle to the other ranks' processes
 * (any host channel), and maps theirs (tf_peer_buffer_import: CUDA IPC, peer access over NVLink). tf_ep_peer_push
 * copies the used slots of a [world][capacity] block array into the owners' buffers (block `rank` of each), and
 * tf_ep_peer_barrier is a flag barrier between the ranks with bounded waits: a wait that gives up sets the context's
 * device error word (tf_device_status) and later barriers stop waiting. Plain kernels only, so a decode step with
 * its exchanges can be captured in a CUDA graph. One process per GPU; every rank must issue the same sequence of
 * barriers. */
#define TF_PEER_HANDLE_BYTES 64
typedef struct tf_peer_buffer tf_peer_buffer;
tf_status tf_peer_buffer_create(tf_context* ctx, uint64_t bytes, tf_peer_buffer** out);      /* zero-filled */
void tf_peer_buffer_destroy(tf_peer_buffer* buffer);
void* tf_peer_buffer_ptr(const tf_peer_buffer* buffer);
tf_status tf_peer_buffer_export(const tf_peer_buffer* buffer, void* handle_out_64_bytes);
tf_status tf_peer_buffer_import(tf_context* ctx, const void* handle_64_bytes, void** ptr_out);
tf_status tf_peer_buffer_release(tf_context* ctx, void* imported_ptr);
/* peer_bases_device: device array of `world` base addresses (own buffer at index `rank`). Slot (s, j) of src_rows
 * goes to peer s at dst_offset_bytes + ((rank * capacity + j) * dst_stride_elements) * 2 when its expert id is not
 * 0xFFFFFFFF; the id comes from slot_ids[s * capacity + j], or, when slot_ids is NULL, from the 32 bits at element
 * tail_at_element of the row (then an unused slot still gets its 16-byte tail written, so the owner sees it empty).
 * epoch_and_ticket_device: NULL, or two zero-initialised words of this rank; then the thread block that finishes last
 * runs the flag barrier of tf_ep_peer_barrier in the same launch (word 0 is the epoch counter that call takes). */
tf_status tf_ep_peer_push(tf_context* ctx, void* stream, const void* src_rows, uint32_t src_stride_elements,
                          const void* const* peer_bases_device, uint64_t dst_offset_bytes, uint32_t dst_stride_elements,
                          uint32_t copy_elements, const uint32_t* slot_ids, uint32_t tail_at_element,
                          uint32_t world, uint32_t rank, uint32_t capacity,
                          uint64_t flags_offset_bytes, uint32_t* epoch_and_ticket_device);
/* tf_ep_pack + tf_ep_peer_push in one launch, for a block whose routes are already grouped (tf_router_gemma4_block_grouped):
 * the row of pair p goes from hidden[token] straight into its owner's buffer at dst_offset_bytes +
 * ((rank * capacity + position) * dst_stride_elements) * 2, with the local expert id in the 16-byte tail at element d;
 * unused slots get an empty tail; inverse_perm[token * top_k + r] = owner * capacity + position. Ends with the flag
 * barrier like tf_ep_peer_push. */
tf_status tf_ep_pack_push(tf_context* ctx, void* stream, const void* hidden, uint32_t hidden_stride_elements,
                          const tf_device_routes* routes, uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                          uint32_t experts_per_rank, uint32_t d, const void* const* peer_bases_device, uint64_t dst_offset_bytes,
                          uint32_t dst_stride_elements, uint32_t* inverse_perm, uint32_t world, uint32_t rank, uint32_t capacity,
                          uint64_t flags_offset_bytes, uint32_t* epoch_and_ticket_device);
/* flags: `world` 32-bit words at flags_offset_bytes of every buffer; epoch_counter_device: one zero-initialised word
 * of this rank, advanced by the kernel. */
tf_status tf_ep_peer_barrier(tf_context* ctx, void* stream, const void* const* peer_bases_device, uint64_t flags_offset_bytes,
                             uint32_t* epoch_counter_device, uint32_t world, uint32_t rank);

/* ---- greedy LM head ---- */
/* out_token = argmax_row deq4(W[vocab, d]) . half(rms(hidden) * norm_weight): RMSNorm to fp16, the int4 GEMV with
 * UNROUNDED fp32 logits, the maximum over the finite ones, ties to the lowest row, 0 when none is finite.
 * Replaces LMHeadChainInt4.encodeGreedyDecode (Kernels/Fusions/LMHeadChainInt4.swift:53-135) and
 * lm_head_greedy_int4_rows_chunk_raw / lm_head_greedy_int4_rows_reduce (Metal/Sampling/logit.metal:688-787).
 * hidden_off selects a row of a larger buffer, as hiddenOffset does. Scales and biases are bf16. The context owns the
 * scratch (normed row, fp32 logits), as the Swift wrapper does; it grows, with an allocation, the first time a
 * larger d or vocab is seen. Calls on one context must not overlap on different streams. */
tf_status tf_lm_head_greedy_int4(tf_context* ctx, void* stream, const void* hidden, uint64_t hidden_off,
                                 const void* norm_weight_bf16, uint64_t norm_off,
                                 const void* weights, uint64_t weights_off, const void* scales, uint64_t scales_off,
                                 const void* biases, uint64_t biases_off, uint32_t* out_token,
                                 uint32_t d, uint32_t vocab, float rms_eps);

/* ---- norms ---- */
/* y = half(x * rsqrt(mean(x^2) + eps) * w_bf16); weight NULL = no-scale form.
 * Replaces RMSNorm.encode and the block form PrefillRMSNorm
 * (Metal/Primitives/rmsnorm.metal:32-93,153-175; Metal/Prefill/prefill.metal:54-111). */
tf_status tf_rmsnorm(tf_context* ctx, void* stream,
                     const void* x, uint64_t x_off, const void* weight_bf16, uint64_t weight_off,
                     void* y, uint64_t y_off, uint32_t rows, uint32_t d,
                     uint32_t stride_elements, float eps, tf_dtype act_dtype);
/* The three-way norm in front of the feed-forward block, per row and in fp16:
 *   hidden += rms(attn) * w_post_attn (written back); h = rms_no_scale(hidden);
 *   dense_x = h * w_pre_ffn; routed_x = h * w_pre_ffn2; router_x = h,
 * every stage rounded to fp16 where the reference rounds, so the result equals the chain of tf_rmsnorm calls bit
 * for bit. Replaces FusedPostAttentionSetup.encode (rows = 1; Kernels/Fusions/FusedPostAttentionSetup.swift:26-60,
 * Metal/Fusions/fused.metal:190-269) and PrefillPostAttentionSetup.encode with its five row strides
 * (Kernels/Prefill/Epilogues/PrefillPostAttentionSetup.swift; Metal/Prefill/prefill.metal:178-254). */
tf_status tf_post_attn_setup(tf_context* ctx, void* stream, void* hidden, uint32_t hidden_stride_elements,
                             const void* attn, uint32_t attn_stride_elements, void* dense_x, uint32_t dense_stride_elements,
                             void* routed_x, uint32_t routed_stride_elements, void* router_x, uint32_t router_stride_elements,
                             const void* w_post_attn_bf16, const void* w_pre_ffn_bf16, const void* w_pre_ffn2_bf16,
                             uint32_t rows, uint32_t d, float eps);
/* hidden = (hidden + rms(h1 + rms(h2) * w2) * w) * layer_scalar with fp16
 * rounding at each stage. Replaces FusedLayerTail / PrefillLayerTail
 * (Metal/Fusions/fused.metal:271-375; Metal/Prefill/prefill.metal:255-334). */
tf_status tf_layer_tail(tf_context* ctx, void* stream,
                        const void* h2, const void* h1, void* hidden,
                        const void* w_postffn2_bf16, const void* w_postffn_bf16,
                        uint32_t rows, uint32_t d, uint32_t stride_elements,
                        float eps, float layer_scalar);

/* ---- expert parallelism behind the C ABI (new: the reference is single-GPU,
 * Infrastructure/Metal/MetalContext.swift:51-71). One process per GPU; experts sharded num_experts / world per rank
 * (tf_moe_layer.pool_layer_base is the rank's shard, num_experts the global count); tokens stay with their rank. The
 * calls below replace, per layer, the MoE section of the reference's forward runner
 * (Runtime/Inference/RealForwardRunner.swift:902-1186 prefill, :1449-1693 decode) with the collectives inside. NCCL is
 * bound at run time (libnccl.so.2). ---- */
#define TF_EP_UNIQUE_ID_BYTES 128
typedef struct tf_ep tf_ep;
typedef struct tf_ep_buffers tf_ep_buffers;
typedef enum tf_ep_mode {
    TF_EP_EXACT = 0,        /* exact row counts over NCCL send/recv; one host synchronisation per layer (prefill) */
    TF_EP_FIXED_NCCL = 1,   /* fixed capacity per destination, no host synchronisation, NCCL send/recv */
    TF_EP_FIXED_PEER = 2    /* fixed capacity, rows pushed over peer memory by a kernel with flag barriers: plain
                             * kernels only, capturable in a CUDA graph; becomes TF_EP_FIXED_NCCL on every rank together
                             * when a peer mapping fails */
} tf_ep_mode;
/* Rank 0 makes the 128-byte id (ncclGetUniqueId) and hands it to the other ranks over any host channel. */
tf_status tf_ep_unique_id(void* out_128_bytes);
/* Collective over the ranks: ncclCommInitRank on ctx's device. world 1 needs no id and no NCCL. */
tf_status tf_ep_create(tf_context* ctx, const void* unique_id_128_bytes, int rank, int world, tf_ep** out);
/* The same over a communicator the host already has (an ncclComm_t); it is not destroyed by tf_ep_destroy. */
tf_status tf_ep_create_from_comm(tf_context* ctx, void* nccl_comm, int rank, int world, tf_ep** out);
void tf_ep_destroy(tf_ep* ep);
int tf_ep_rank(const tf_ep* ep);
int tf_ep_world(const tf_ep* ep);
/* Expert placement by measured load (host only, no device work). The library shards experts contiguously: rank r owns
 * ids [r * E / world, (r + 1) * E / world). A host that wants the ranks equally loaded renumbers the experts of a layer
 * when it loads the weights: placement[l * E + new_id] = original id, the router's rows (weights, scales, biases,
 * per-expert scale, logit bias) and the pool slots stored in the new order. Outputs do not change (the router only
 * reports other ids for the same experts; exactly equal logits may break their tie the other way).
 * counts[l * E + e]: routed (token, rank) pairs that expert e of layer l received on a calibration batch, summed over
 * all ranks' tokens. Per layer, experts are taken by descending count (ties by id) and each goes to the least loaded
 * rank that still has a free slot (ties to the lowest rank); a rank's slots are filled in that order. */
tf_status tf_ep_balanced_placement(const uint64_t* counts, uint32_t layers, uint32_t num_experts, uint32_t world,
                                   uint32_t* placement);
/* Exchange buffers and scratch for up to max_tokens LOCAL tokens. Collective: every rank asks for the same buffers in
 * the same order (the peer mode maps the ranks' buffers into one another). Allocates device memory. */
tf_status tf_ep_buffers_create(tf_ep* ep, uint32_t max_tokens, uint32_t d, uint32_t f, uint32_t fs, uint32_t top_k,
                               uint32_t num_experts, tf_ep_mode mode, tf_ep_buffers** out);
void tf_ep_buffers_destroy(tf_ep_buffers* buffers);                 /* collective in the peer mode */
tf_ep_mode tf_ep_buffers_mode(const tf_ep_buffers* buffers);       /* the mode in use (after a fallback) */
tf_workspace* tf_ep_buffers_workspace(const tf_ep_buffers* buffers);   /* router output of the last forward */
/* y[tokens, d] = shared(x) + sum_r w_r * routed_r(x) with the routed experts on their owner ranks. Collective: every
 * rank calls it for the same layer (its own tokens; tokens may differ per rank, 0 included only in the fixed modes). In
 * TF_EP_EXACT the call synchronises the stream once (to read the row counts) and may grow its receive buffers, so it
 * cannot be captured in a CUDA graph; the fixed modes only enqueue. */
tf_status tf_moe_block_forward_ep(tf_ep* ep, void* stream, const tf_moe_layer* layer, const void* x, void* y, uint32_t tokens,
                                  tf_ep_buffers* buffers);
/* hidden [tokens, d] fp16, updated in place: for each layer x = rmsnorm(h) * w_l; h = h + block_l(x). */
tf_status tf_stack_forward_ep(tf_ep* ep, void* stream, const tf_moe_layer* layers, const void* const* norm_weights_bf16,
                              uint32_t layer_count, float eps, void* hidden, uint32_t tokens, tf_ep_buffers* buffers);

#ifdef __cplusplus
}
#endif
#endif /* TURBOFIELDFARE_CUDA_H */
