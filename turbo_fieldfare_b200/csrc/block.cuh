// Host-side objects behind the pool, workspace and stack handles of the C ABI.
#pragma once

#include <vector>

#include "tf_common.cuh"

struct tf_pool {
    tf_context* ctx;
    uint8_t* base;
    uint32_t layers, experts;
    uint64_t stride;
    tf_expert_offsets offsets;
};

struct tf_workspace {
    tf_context* ctx;
    uint32_t max_tokens, d, f, fs, top_k, num_experts;
    uint8_t* base;          // one allocation
    uint32_t* indices;      // [T, K]
    uint16_t* weights;      // [T, K] fp16
    tf_device_routes routes;
    uint16_t* acts;         // [T*K, F] fp16
    void* partials;         // [T, K, D] fp32 (T <= f32_tokens) or fp16
    uint16_t* shared_act;   // [T, Fs]
    uint16_t* shared_y;     // [T, D]
    uint16_t* x_norm;       // [T, D] (stack)
    uint16_t* y_block;      // [T, D] (stack)
    uint16_t* x_sorted;     // [T*K, D] expert-sorted activation rows (tensor-core path; NULL for small workspaces)
    uint32_t* inverse_perm; // [T*K] sorted row of every (token, rank)
    uint32_t* pack_ids;     // [T*K]
    uint64_t bytes;
};

struct tf_stack {
    tf_context* ctx;
    std::vector<tf_moe_layer> layers;
    std::vector<const void*> norm_weights;   // bf16 [D] per layer
    float eps;
    // device copy of the per-layer pointers for the single-launch one-token step (decode_step.cu)
    void* device_layers = nullptr;
    bool decode_step_ok = false;
    bool decode_step_bulk_scales = false;
};

namespace tf {
struct PeerWait;
bool decode_step_eligible(const tf_stack* st, const tf_workspace* ws);
tf_status decode_step_prepare(tf_context* ctx, tf_stack* st);
tf_status launch_decode_step(tf_context* ctx, void* stream, tf_stack* st, void* hidden, tf_workspace* ws);
// grouped.cu: tf_group_routes_device over ids read at a stride (and optionally written out densely)
tf_status group_routes_strided(tf_context* ctx, void* stream, const uint32_t* indices, uint32_t idx_stride, uint32_t* ids_out,
                               const void* weights_f16, uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                               const tf_device_routes* routes, const char* name, const struct PeerWait* peer_wait);
// block.cu / ep.cu: tf_ep_experts and tf_ep_combine whose first kernel waits (bounded) for the peers' flags
tf_status ep_experts_waiting(tf_context* ctx, void* stream, const void* pool_layer_base, uint64_t expert_stride,
                             const tf_expert_offsets* offsets, const void* recv_rows, const uint32_t* recv_expert_ids,
                             uint32_t recv_slots, uint32_t local_experts, const tf_device_routes* recv_routes,
                             const void* zero_weights, void* acts_scratch, void* out_rows, uint32_t d, uint32_t f,
                             uint32_t recv_row_stride_elements, const struct PeerWait* peer_wait);
tf_status ep_experts_tensorcore_waiting(tf_context* ctx, void* stream, const void* pool_layer_base, uint64_t expert_stride,
                                        const tf_expert_offsets* offsets, const void* recv_rows, const uint32_t* recv_expert_ids,
                                        uint32_t recv_slots, uint32_t local_experts, const tf_device_routes* recv_routes,
                                        const void* zero_weights, const void* one_weights, void* x_sorted, uint32_t* row_ids,
                                        uint32_t* inverse_perm, void* acts_scratch, void* out_sorted, void* out_rows,
                                        uint32_t d, uint32_t f, uint32_t recv_row_stride_elements, const struct PeerWait* peer_wait);
tf_status combine_rows_residual_rmsnorm(tf_context* ctx, void* stream, void* hidden, const void* rows, const void* route_weights,
                                        const uint32_t* inverse_perm, const void* shared_y, const void* norm_weight_bf16, void* x,
                                        uint32_t tokens, uint32_t top_k, uint32_t d, float eps, const struct PeerWait* peer_wait);
tf_status ep_combine_waiting(tf_context* ctx, void* stream, const void* returned_rows, const void* route_weights,
                             const uint32_t* inverse_perm, const void* residual, uint32_t residual_stride_elements,
                             void* out, uint32_t out_stride_elements, uint32_t query_count, uint32_t top_k, uint32_t d,
                             const struct PeerWait* peer_wait, const uint32_t* skip_ids = nullptr);
}  // namespace tf

