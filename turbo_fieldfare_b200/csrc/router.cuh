// Device functions shared by the router kernels and the single-launch decode step: the canonical logit of an
// expert row staged in shared memory, and the warp-parallel top-k + softmax.
#pragma once

#include "tf_common.cuh"

namespace tf {

// Warp-parallel top-k over logits in shared memory: k rounds of arg-max with
// ties to the lower index, i.e. the first k entries of the order
// (score desc, index asc) — the result of the reference's insertion scan
// (moe.metal:152-166). Then softmax over the selected scores times the
// per-expert gain, rounded to fp16 (moe.metal:168-184). Called by warp 0.
__device__ __forceinline__ void warp_select_topk(float* scores /*shared, clobbered*/, uint32_t num_experts, uint32_t top_k,
                                                 const uint16_t* __restrict__ per_expert_scale,
                                                 uint32_t* __restrict__ out_idx, uint16_t* __restrict__ out_w, int lane) {
    float sel_score[TF_MAX_TOP_K];
    uint32_t sel_idx[TF_MAX_TOP_K];
    for (uint32_t r = 0; r < top_k; ++r) {
        float best = -INFINITY;
        uint32_t best_e = 0xFFFFFFFFu;
        for (uint32_t e = lane; e < num_experts; e += kWarp) {
            const float s = scores[e];
            if (s > best || (s == best && e < best_e)) { best = s; best_e = e; }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float os = __shfl_xor_sync(kFullMask, best, off);
            const uint32_t oe = __shfl_xor_sync(kFullMask, best_e, off);
            if (os > best || (os == best && oe < best_e)) { best = os; best_e = oe; }
        }
        if (best_e == 0xFFFFFFFFu) best_e = 0;   // fewer finite candidates than top_k
        sel_score[r] = best;
        sel_idx[r] = best_e;
        if (lane == 0 && best_e < num_experts) scores[best_e] = -INFINITY;   // NaN-free inputs: -inf never wins again before real scores
        __syncwarp();
    }
    if (lane == 0) {
        const float max_s = sel_score[0];
        float exps[TF_MAX_TOP_K];
        float sum_exp = 0.0f;
        for (uint32_t r = 0; r < top_k; ++r) { exps[r] = expf(sel_score[r] - max_s); sum_exp += exps[r]; }
        for (uint32_t r = 0; r < top_k; ++r) {
            const float w = exps[r] / sum_exp * bf16_bits_to_float(per_expert_scale[sel_idx[r]]);
            out_idx[r] = sel_idx[r];
            out_w[r] = __half_as_ushort(__float2half_rn(w));
        }
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
