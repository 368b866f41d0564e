// Device functions shared by the router kernels and the single-launch decode step: the canonical logit of an
// expert row staged in shared memory, and the warp-parallel top-k + softmax.
#pragma once

#include "tf_common.cuh"

namespace tf {

// Top-k of a row of scores (highest first, ties to the lower expert index) and the softmax over the selected scores
// times the per-expert gain, rounded to fp16: the first k entries of the order (score desc, index asc), which is the
// result of the reference's insertion scan (Metal/MoE/moe.metal:152-184). Every lane keeps its experts' scores in registers as
// order-preserving integer keys; a round is one warp-wide integer maximum followed by a warp-wide minimum over the
// indices that hold it; a selected expert drops to -inf, so it can only come back when nothing greater is left (fewer
// comparable candidates than top_k). NaN scores never win. The exponentials are taken by top_k lanes at once and summed
// in rank order. `scores` is only read.
__device__ __forceinline__ uint32_t topk_score_key(float v) {
    if (v != v) return 0u;
    const uint32_t b = __float_as_uint(v + 0.0f);             // -0 and +0 compare equal: one key for both
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);       // -inf maps to 0x007FFFFF, above the NaN key
}
__device__ __forceinline__ float topk_key_score(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}
__device__ __forceinline__ void warp_select_topk(const float* scores /*shared*/, uint32_t num_experts, uint32_t top_k,
                                                 const uint16_t* __restrict__ per_expert_scale,
                                                 uint32_t* __restrict__ out_idx, uint16_t* __restrict__ out_w, int lane) {
    constexpr int kPerLane = TF_MAX_ROUTER_EXPERTS / kWarp;
    uint32_t key[kPerLane];
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
        const uint32_t e = lane + j * kWarp;
        key[j] = e < num_experts ? topk_score_key(scores[e]) : 0u;
    }
    const uint32_t neg_inf_key = 0x007FFFFFu;
    float my_score = 0.0f, max_s = 0.0f;
    uint32_t my_idx = 0;
    for (uint32_t r = 0; r < top_k; ++r) {
        uint32_t best = 0u, best_e = 0xFFFFFFFFu;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
            const uint32_t e = lane + j * kWarp;
            if (e < num_experts && key[j] > best) { best = key[j]; best_e = e; }      // ascending e: ties keep the lower index
        }
        const uint32_t top = __reduce_max_sync(kFullMask, best);
        uint32_t winner = __reduce_min_sync(kFullMask, (best == top && top != 0u) ? best_e : 0xFFFFFFFFu);
        float top_score = topk_key_score(top);
        if (winner == 0xFFFFFFFFu) { winner = 0u; top_score = -INFINITY; }            // no comparable candidate at all
        if (r == 0) max_s = top_score;
        if ((uint32_t)lane == r) { my_score = top_score; my_idx = winner; }
        if (winner < num_experts && (winner % kWarp) == (uint32_t)lane) {
#pragma unroll
            for (int j = 0; j < kPerLane; ++j)
                if ((uint32_t)j == winner / kWarp) key[j] = neg_inf_key;
        }
    }
    const float ex = (uint32_t)lane < top_k ? expf(my_score - max_s) : 0.0f;
    float sum_exp = 0.0f;
    for (uint32_t r = 0; r < top_k; ++r) sum_exp += __shfl_sync(kFullMask, ex, (int)r);
    if ((uint32_t)lane < top_k) {
        const float w = ex / sum_exp * bf16_bits_to_float(per_expert_scale[my_idx]);
        out_idx[lane] = my_idx;
        out_w[lane] = __half_as_ushort(__float2half_rn(w));
    }
}

// Canonical logit of one expert row whose bytes, scales and biases sit in shared memory
// (same arithmetic and order as router_row_logit; only the operand source differs).
__device__ __forceinline__ float router_row_logit_smem(const uint8_t* Wrow, const uint16_t* s_row, const uint16_t* b_row,
                                                       const float* xf, uint32_t groups, int lane) {
    float acc = 0.0f;
#pragma unroll 4
    for (uint32_t g = 0; g < groups; ++g) {
        const uint32_t i0 = g * kGroup + lane * 2;
        const uint32_t w = *reinterpret_cast<const uint16_t*>(Wrow + i0);
        const float q0 = (float)(w & 0xFFu), q1 = (float)(w >> 8);
        const float2 xv = *reinterpret_cast<const float2*>(xf + i0);
        const float s = bf16_bits_to_float(s_row[g]);
        const float b = bf16_bits_to_float(b_row[g]);
        const float p = __fmaf_rn(q1, xv.y, __fmul_rn(q0, xv.x));
        acc = __fmaf_rn(s, p, acc);
        acc = __fmaf_rn(b, __fadd_rn(xv.x, xv.y), acc);
    }
    return warp_sum(acc);
}

}  // namespace tf
