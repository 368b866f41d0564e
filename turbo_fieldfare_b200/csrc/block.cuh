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
bool decode_step_eligible(const tf_stack* st, const tf_workspace* ws);
tf_status decode_step_prepare(tf_context* ctx, tf_stack* st);
tf_status launch_decode_step(tf_context* ctx, void* stream, tf_stack* st, void* hidden, tf_workspace* ws);
// grouped.cu: tf_group_routes_device over ids read at a stride (and optionally written out densely)
tf_status group_routes_strided(tf_context* ctx, void* stream, const uint32_t* indices, uint32_t idx_stride, uint32_t* ids_out,
                               const void* weights_f16, uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                               const tf_device_routes* routes, const char* name);
}  // namespace tf

