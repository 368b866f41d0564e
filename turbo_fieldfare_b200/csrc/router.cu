// Router: 8-bit affine GEMV + top-k + softmax in ONE launch, ids stay on the device.
// Replaces router_gemv_gemma4_r4 + router_topk_select_k8 (Metal/MoE/moe.metal:78-185)
// and prefill_router_gemma4_block (Metal/Prefill/prefill.metal:478-573).
//
// Logit arithmetic is canonical so that a CPU emulation reproduces every bit
// (top-k indices must match exactly):
//   xf[i]  = fmul(float(hidden[i]), float(effective_scale[i]))
//   lane l, group g: i0 = 64 g + 2 l
//     p   = fma(q1, xf[i0+1], fmul(q0, xf[i0]))
//     acc = fma(s, p, acc);  acc = fma(b, fadd(xf[i0], xf[i0+1]), acc)
//   logit = xor-butterfly sum over the 32 lanes (offsets 16, 8, 4, 2, 1)
// which is the reference kernel's per-lane element assignment with the
// contraction and reduction order fixed.
#include "router.cuh"
#include "router_tensor.cuh"

namespace tf {

constexpr int kSplitExpertsPerBlock = 4;
constexpr int kSplitThreads = kSplitExpertsPerBlock * kWarp;
constexpr int kBlockRouterThreads = 256;

template <bool X_BF16>
__device__ __forceinline__ void stage_router_x(const uint16_t* __restrict__ hidden, const uint16_t* __restrict__ eff,
                                               float* xf, uint32_t d) {
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        const float h = X_BF16 ? bf16_bits_to_float(hidden[i]) : f16_bits_to_float(hidden[i]);
        xf[i] = __fmul_rn(h, bf16_bits_to_float(eff[i]));
    }
    __syncthreads();
}

__device__ __forceinline__ float router_row_logit(const uint8_t* __restrict__ Wrow, const uint16_t* __restrict__ s_row,
                                                  const uint16_t* __restrict__ b_row, const float* xf,
                                                  uint32_t groups, int lane, bool a2) {
    float acc = 0.0f;
    for (uint32_t g = 0; g < groups; ++g) {
        const uint32_t i0 = g * kGroup + lane * 2;
        uint32_t w;
        if (a2) w = *reinterpret_cast<const uint16_t*>(Wrow + i0);
        else w = (uint32_t)Wrow[i0] | ((uint32_t)Wrow[i0 + 1] << 8);
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

// Grouping of a small block's routes inside the router launch (the work of group_routes_kernel for at most
// kRouterSplitRows rows): the block that finishes the last row sorts the (token, rank) pairs by expert, stably in
// token-major order, and writes offsets, counts, groups and the 8-token chunk table. A pair's place is its expert's
// offset plus the number of earlier pairs of that expert, counted on a per-expert bitmap over the pairs.
struct RouterGroupOut {
    tf_pair* sorted_pairs;          // nullptr: no grouping
    uint32_t* per_expert_offsets;
    uint32_t* per_expert_counts;
    tf_group* groups;
    uint32_t* chunk_group;
    uint32_t* chunk_start;
    uint32_t* counters;
};

__host__ __device__ inline size_t router_group_smem_bytes(uint32_t n_pairs, uint32_t num_experts) {
    const uint32_t nw = (n_pairs + 31) / 32;
    // mask, hist + offs, expert ids, warp totals (3 x 32), weights
    return (size_t)num_experts * nw * 4 + (size_t)num_experts * 2 * 4 + (size_t)n_pairs * 4 + 96 * 4 + (size_t)((n_pairs + 1) / 2) * 4;
}

__device__ void group_routes_in_block(const uint32_t* __restrict__ idx, const uint16_t* __restrict__ w, uint32_t T, uint32_t K,
                                      uint32_t E, const RouterGroupOut& out, uint8_t* smem) {
    const uint32_t n = T * K, nw = (n + 31) / 32;
    uint32_t* mask = reinterpret_cast<uint32_t*>(smem);          // [E][nw]
    uint32_t* hist = mask + (size_t)E * nw;                      // [E]
    uint32_t* offs = hist + E;                                   // [E]
    uint32_t* exs = offs + E;                                    // [n]
    uint32_t* wtot = exs + n;                                    // [3][32]: per-warp totals of the scan
    uint16_t* wts = reinterpret_cast<uint16_t*>(wtot + 96);      // [n]
    const uint32_t lane = threadIdx.x % kWarp, warp = threadIdx.x / kWarp, nwarps = blockDim.x / kWarp;
    // ids and weights (written by other blocks of this launch) travel while the bitmaps are cleared
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        uint32_t ex = __ldcg(idx + i);
        if (ex != 0xFFFFFFFFu && ex >= E) ex = E - 1;            // min(id, E-1): Runtime/Inference/RealForwardRunner.swift:955
        exs[i] = ex;
        wts[i] = __ldcg(w + i);
    }
    for (uint32_t i = threadIdx.x; i < E * nw + E; i += blockDim.x) mask[i] = 0;      // mask and hist are adjacent
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const uint32_t ex = exs[i];
        if (ex != 0xFFFFFFFFu) {
            atomicAdd(&hist[ex], 1u);
            atomicOr(&mask[(size_t)ex * nw + i / 32], 1u << (i % 32));
        }
    }
    __syncthreads();
    // exclusive scans over the experts (pairs, non-empty groups, chunks): every warp scans 32 experts, the warps'
    // totals meet in shared memory, and rounds of nwarps * 32 experts carry the running totals.
    uint32_t off = 0, gi = 0, ch = 0;
    for (uint32_t base = 0; base < E; base += nwarps * kWarp) {
        const uint32_t e = base + warp * kWarp + lane;
        const uint32_t cnt = e < E ? hist[e] : 0u;
        const uint32_t nch = (cnt + (uint32_t)kChunkTokens - 1) / (uint32_t)kChunkTokens;
        uint32_t i_off = cnt, i_g = cnt ? 1u : 0u, i_ch = nch;
#pragma unroll
        for (int o = 1; o < kWarp; o <<= 1) {
            const uint32_t a = __shfl_up_sync(kFullMask, i_off, o), b2 = __shfl_up_sync(kFullMask, i_g, o),
                           c = __shfl_up_sync(kFullMask, i_ch, o);
            if ((int)lane >= o) { i_off += a; i_g += b2; i_ch += c; }
        }
        if (lane == kWarp - 1) { wtot[warp] = i_off; wtot[32 + warp] = i_g; wtot[64 + warp] = i_ch; }
        __syncthreads();
        uint32_t p_off = off, p_g = gi, p_ch = ch;
        for (uint32_t v = 0; v < nwarps; ++v) {
            const uint32_t a = wtot[v], b2 = wtot[32 + v], c = wtot[64 + v];
            if (v < warp) { p_off += a; p_g += b2; p_ch += c; }
            off += a; gi += b2; ch += c;
        }
        const uint32_t my_off = p_off + i_off - cnt, my_g = p_g + i_g - (cnt ? 1u : 0u), my_ch = p_ch + i_ch - nch;
        if (e < E) {
            offs[e] = my_off;
            out.per_expert_counts[e] = cnt;
            out.per_expert_offsets[e] = cnt ? my_off : 0xFFFFFFFFu;
            if (cnt) {
                out.groups[my_g] = tf_group{e, my_off, cnt};
                out.chunk_start[my_g] = my_ch;
                for (uint32_t j = 0; j < nch; ++j) out.chunk_group[my_ch + j] = my_g;
            }
        }
        __syncthreads();                                          // wtot is reused by the next round; offs is read below
    }
    if (threadIdx.x == 0) {
        out.counters[0] = gi;
        out.counters[1] = ch;
        out.counters[2] = n;
        out.counters[3] = off;
    }
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const uint32_t ex = exs[i];
        if (ex == 0xFFFFFFFFu) continue;
        const uint32_t* m = mask + (size_t)ex * nw;
        uint32_t pos = offs[ex];
        for (uint32_t q = 0; q < i / 32; ++q) pos += __popc(m[q]);
        pos += __popc(m[i / 32] & ((1u << (i % 32)) - 1u));
        out.sorted_pairs[pos] = tf_pair{i / K, ex, i % K, (uint32_t)wts[i]};
    }
}

// Few rows (decode): grid (rows, experts/4); the block first copies its four expert rows into
// shared memory with coalesced loads (the per-lane access pattern of the canonical order would
// otherwise be a chain of 2-byte global loads); the last block to finish a row (self-resetting
// ticket) runs the selection, so one launch does everything.
template <bool X_BF16>
__global__ void __launch_bounds__(kSplitThreads)
router_split_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ S, const uint16_t* __restrict__ B,
                    const uint16_t* __restrict__ hidden, uint32_t hidden_stride,
                    const uint16_t* __restrict__ eff, const uint16_t* __restrict__ per_expert_scale,
                    const float* __restrict__ logit_bias,
                    uint32_t* __restrict__ out_idx, uint16_t* __restrict__ out_w, float* __restrict__ out_logits,
                    float* scratch_logits, unsigned int* tickets, const RouterGroupOut grp,
                    uint32_t num_experts, uint32_t d, uint32_t top_k, bool a2) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* xf = reinterpret_cast<float*>(smem);                                   // [d]
    uint8_t* wrows = smem + (size_t)d * 4;                                        // [4][d]
    const uint32_t groups = d / kGroup;
    uint16_t* srows = reinterpret_cast<uint16_t*>(wrows + (size_t)kSplitExpertsPerBlock * d);   // [4][groups]
    uint16_t* brows = srows + kSplitExpertsPerBlock * groups;
    __shared__ float scores[TF_MAX_ROUTER_EXPERTS];
    __shared__ bool is_last;
    const uint32_t row = blockIdx.x;
    const uint32_t e0 = blockIdx.y * kSplitExpertsPerBlock;
    const uint32_t ne = num_experts - e0 < (uint32_t)kSplitExpertsPerBlock ? num_experts - e0 : (uint32_t)kSplitExpertsPerBlock;
    // the four rows are contiguous in every plane
    const uint8_t* wsrc = W + (size_t)e0 * d;
    const uint16_t* hrow = hidden + (size_t)row * hidden_stride;
    const bool a16 = (reinterpret_cast<uintptr_t>(wsrc) & 15) == 0 && (d & 15) == 0;
    const bool x16 = (reinterpret_cast<uintptr_t>(hrow) & 15) == 0 && (reinterpret_cast<uintptr_t>(eff) & 15) == 0 && (d & 7) == 0;
    pdl_launch_dependents();
    if (a16 && x16 && ne * d <= kSplitThreads * 16 * 6 && d <= kSplitThreads * 8 * 3) {
        // latency path: every load of the block is issued before the first one is consumed
        uint4 wv[6], hv[3], ev[3];
#pragma unroll
        for (int j = 0; j < 6; ++j) {
            const uint32_t i = threadIdx.x + j * kSplitThreads;
            wv[j] = i < ne * d / 16 ? ldg_nc_u4(wsrc + (size_t)i * 16) : make_uint4(0u, 0u, 0u, 0u);
        }
        pdl_wait();          // the weights above do not depend on the previous kernel; the hidden row does
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            const uint32_t i = threadIdx.x + j * kSplitThreads;
            const bool ok = i < d / 8;
            hv[j] = ok ? __ldg(reinterpret_cast<const uint4*>(hrow) + i) : make_uint4(0u, 0u, 0u, 0u);
            ev[j] = ok ? __ldg(reinterpret_cast<const uint4*>(eff) + i) : make_uint4(0u, 0u, 0u, 0u);
        }
        for (uint32_t i = threadIdx.x; i < ne * groups; i += blockDim.x) {
            srows[i] = S[(size_t)e0 * groups + i];
            brows[i] = B[(size_t)e0 * groups + i];
        }
#pragma unroll
        for (int j = 0; j < 6; ++j) {
            const uint32_t i = threadIdx.x + j * kSplitThreads;
            if (i < ne * d / 16) reinterpret_cast<uint4*>(wrows)[i] = wv[j];
        }
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            const uint32_t i = threadIdx.x + j * kSplitThreads;
            if (i < d / 8) {
                const uint32_t hw[4] = {hv[j].x, hv[j].y, hv[j].z, hv[j].w}, ew[4] = {ev[j].x, ev[j].y, ev[j].z, ev[j].w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint16_t h0 = (uint16_t)(hw[q] & 0xFFFFu), h1 = (uint16_t)(hw[q] >> 16);
                    const float f0 = X_BF16 ? bf16_bits_to_float(h0) : f16_bits_to_float(h0);
                    const float f1 = X_BF16 ? bf16_bits_to_float(h1) : f16_bits_to_float(h1);
                    xf[i * 8 + 2 * q] = __fmul_rn(f0, bf16_bits_to_float((uint16_t)(ew[q] & 0xFFFFu)));
                    xf[i * 8 + 2 * q + 1] = __fmul_rn(f1, bf16_bits_to_float((uint16_t)(ew[q] >> 16)));
                }
            }
        }
        __syncthreads();
    } else {
        if (a16) {
            for (uint32_t i = threadIdx.x; i < ne * d / 16; i += blockDim.x)
                reinterpret_cast<uint4*>(wrows)[i] = ldg_nc_u4(wsrc + (size_t)i * 16);
        } else if (a2) {
            for (uint32_t i = threadIdx.x; i < ne * d / 2; i += blockDim.x)
                reinterpret_cast<uint16_t*>(wrows)[i] = reinterpret_cast<const uint16_t*>(wsrc)[i];
        } else {
            for (uint32_t i = threadIdx.x; i < ne * d; i += blockDim.x) wrows[i] = wsrc[i];
        }
        for (uint32_t i = threadIdx.x; i < ne * groups; i += blockDim.x) {
            srows[i] = S[(size_t)e0 * groups + i];
            brows[i] = B[(size_t)e0 * groups + i];
        }
        pdl_wait();
        stage_router_x<X_BF16>(hrow, eff, xf, d);     // ends with a barrier
    }

    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t e = e0 + warp;
    if (e < num_experts) {
        float logit = router_row_logit_smem(wrows + (size_t)warp * d, srows + warp * groups, brows + warp * groups, xf, groups, lane);
        if (logit_bias) logit = __fadd_rn(logit, logit_bias[e]);
        if (lane == 0) scratch_logits[(size_t)row * TF_MAX_ROUTER_EXPERTS + e] = logit;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int tk = atomicAdd(&tickets[row], 1u);
        is_last = (tk == gridDim.y - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (uint32_t i = threadIdx.x; i < num_experts; i += blockDim.x) {
        const float v = __ldcg(&scratch_logits[(size_t)row * TF_MAX_ROUTER_EXPERTS + i]);
        scores[i] = v;
        if (out_logits) out_logits[(size_t)row * num_experts + i] = v;
    }
    if (threadIdx.x == 0) tickets[row] = 0;   // ready for the next launch on this stream
    __syncthreads();
    if (warp == 0)
        warp_select_topk(scores, num_experts, top_k, per_expert_scale, out_idx + (size_t)row * top_k,
                         out_w + (size_t)row * top_k, lane);
    if (grp.sorted_pairs == nullptr) return;
    if (gridDim.x == 1) {
        // One token: a pair's place is the number of selected experts with a smaller id; every group holds one pair
        // and one chunk. That needs distinct experts: a row with fewer than top_k selectable logits (NaN, -inf)
        // repeats expert 0, and then the general grouping below merges the repeats into one group.
        __syncthreads();                       // warp 0 has written the row's indices and weights
        int repeated = 0;
        if (threadIdx.x < top_k) {
            uint32_t mine = out_idx[threadIdx.x];
            if (mine >= num_experts) mine = num_experts - 1;
            for (uint32_t r = 0; r < top_k; ++r) {
                uint32_t other = out_idx[r];
                if (other >= num_experts) other = num_experts - 1;
                repeated |= (r != threadIdx.x && other == mine) ? 1 : 0;
            }
        }
        if (__syncthreads_or(repeated)) {
            group_routes_in_block(out_idx, out_w, 1, top_k, num_experts, grp, smem);
            return;
        }
        for (uint32_t e = threadIdx.x; e < num_experts; e += blockDim.x) {
            grp.per_expert_counts[e] = 0u;
            grp.per_expert_offsets[e] = 0xFFFFFFFFu;
        }
        __syncthreads();
        if (threadIdx.x < top_k) {
            uint32_t mine = out_idx[threadIdx.x];
            if (mine >= num_experts) mine = num_experts - 1;
            uint32_t pos = 0;
            for (uint32_t r = 0; r < top_k; ++r) {
                uint32_t other = out_idx[r];
                if (other >= num_experts) other = num_experts - 1;
                pos += other < mine ? 1u : 0u;
            }
            grp.sorted_pairs[pos] = tf_pair{0u, mine, threadIdx.x, (uint32_t)out_w[threadIdx.x]};
            grp.per_expert_counts[mine] = 1u;
            grp.per_expert_offsets[mine] = pos;
            grp.groups[pos] = tf_group{mine, pos, 1u};
            grp.chunk_start[pos] = pos;
            grp.chunk_group[pos] = pos;
        }
        if (threadIdx.x == 0) {
            grp.counters[0] = top_k;
            grp.counters[1] = top_k;
            grp.counters[2] = top_k;
            grp.counters[3] = top_k;
        }
        return;
    }
    // the block that completes the last row groups all rows (second ticket, after the row tickets)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int tk = atomicAdd(&tickets[kRouterSplitRows], 1u);
        is_last = (tk == gridDim.x - 1);
        if (is_last) tickets[kRouterSplitRows] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    group_routes_in_block(out_idx, out_w, gridDim.x, top_k, num_experts, grp, smem);
}

// A handful of rows (batched decode, 2...kRouterSplitRows): grid (rows / R, experts / 8). A block stages R activation
// rows (as fp32 x * effective_scale) and its eight expert rows in shared memory; warp w then computes the logits of
// expert e0 + w for all R rows at once, so the codes, scales and biases of a group are decoded once per R rows. The
// arithmetic and its order per (row, expert) are those of router_row_logit_smem. The last block of a row group
// (ticket) selects the top-k of its R rows, one warp per row; the block that completes the last row group builds the
// grouping tables.
constexpr int kRowsThreads = 256;
constexpr int kRowsExpertsPerBlock = kRowsThreads / kWarp;
template <bool X_BF16, int R>
__global__ void __launch_bounds__(kRowsThreads)
router_rows_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ S, const uint16_t* __restrict__ B,
                   const uint16_t* __restrict__ hidden, uint32_t hidden_stride,
                   const uint16_t* __restrict__ eff, const uint16_t* __restrict__ per_expert_scale,
                   const float* __restrict__ logit_bias,
                   uint32_t* __restrict__ out_idx, uint16_t* __restrict__ out_w, float* __restrict__ out_logits,
                   float* scratch_logits, unsigned int* tickets, const RouterGroupOut grp,
                   uint32_t rows, uint32_t num_experts, uint32_t d, uint32_t top_k) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t groups = d / kGroup;
    float* xf = reinterpret_cast<float*>(smem);                                        // [R][d]
    uint8_t* wrows = smem + (size_t)R * d * 4;                                         // [8][d]
    uint16_t* srows = reinterpret_cast<uint16_t*>(wrows + (size_t)kRowsExpertsPerBlock * d);   // [8][groups]
    uint16_t* brows = srows + kRowsExpertsPerBlock * groups;
    __shared__ float scores[R][TF_MAX_ROUTER_EXPERTS];
    __shared__ bool is_last;
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t row0 = blockIdx.x * R;
    const uint32_t e0 = blockIdx.y * kRowsExpertsPerBlock;
    const uint32_t ne = num_experts - e0 < (uint32_t)kRowsExpertsPerBlock ? num_experts - e0 : (uint32_t)kRowsExpertsPerBlock;
    pdl_launch_dependents();
    // expert rows (contiguous in every plane; d is a multiple of 64 and the planes are 16-byte aligned by contract)
    {
        const uint8_t* wsrc = W + (size_t)e0 * d;
        for (uint32_t i = threadIdx.x; i < ne * d / 16; i += kRowsThreads)
            reinterpret_cast<uint4*>(wrows)[i] = ldg_nc_u4(wsrc + (size_t)i * 16);
        for (uint32_t i = threadIdx.x; i < ne * groups; i += kRowsThreads) {
            srows[i] = S[(size_t)e0 * groups + i];
            brows[i] = B[(size_t)e0 * groups + i];
        }
    }
    pdl_wait();          // the weights above do not depend on the previous kernel; the hidden rows do
    for (uint32_t i = threadIdx.x; i < d / 8; i += kRowsThreads) {
        const uint4 ev = __ldg(reinterpret_cast<const uint4*>(eff) + i);
        const uint32_t ew[4] = {ev.x, ev.y, ev.z, ev.w};
        uint4 hv[R];
#pragma unroll
        for (int r = 0; r < R; ++r)
            hv[r] = row0 + r < rows ? __ldg(reinterpret_cast<const uint4*>(hidden + (size_t)(row0 + r) * hidden_stride) + i)
                                    : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t hw[4] = {hv[r].x, hv[r].y, hv[r].z, hv[r].w};
            float o[8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint16_t h0 = (uint16_t)(hw[q] & 0xFFFFu), h1 = (uint16_t)(hw[q] >> 16);
                const float f0 = X_BF16 ? bf16_bits_to_float(h0) : f16_bits_to_float(h0);
                const float f1 = X_BF16 ? bf16_bits_to_float(h1) : f16_bits_to_float(h1);
                o[2 * q] = __fmul_rn(f0, bf16_bits_to_float((uint16_t)(ew[q] & 0xFFFFu)));
                o[2 * q + 1] = __fmul_rn(f1, bf16_bits_to_float((uint16_t)(ew[q] >> 16)));
            }
            float4* dst = reinterpret_cast<float4*>(xf + (size_t)r * d + i * 8);
            dst[0] = make_float4(o[0], o[1], o[2], o[3]);
            dst[1] = make_float4(o[4], o[5], o[6], o[7]);
        }
    }
    __syncthreads();

    if ((uint32_t)warp < ne) {
        const uint8_t* wr = wrows + (size_t)warp * d;
        const uint16_t* sr = srows + warp * groups;
        const uint16_t* br = brows + warp * groups;
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = 0.0f;
#pragma unroll 2
        for (uint32_t g = 0; g < groups; ++g) {
            const uint32_t i0 = g * kGroup + lane * 2;
            const uint32_t w = *reinterpret_cast<const uint16_t*>(wr + i0);
            // byte -> float through the 2^23 mantissa trick (exact for 0...255)
            const float q0 = __uint_as_float(0x4B000000u | (w & 0xFFu)) - 8388608.0f;
            const float q1 = __uint_as_float(0x4B000000u | (w >> 8)) - 8388608.0f;
            const float sc = bf16_bits_to_float(sr[g]);
            const float bi = bf16_bits_to_float(br[g]);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float2 xv = *reinterpret_cast<const float2*>(xf + (size_t)r * d + i0);
                const float p = __fmaf_rn(q1, xv.y, __fmul_rn(q0, xv.x));
                acc[r] = __fmaf_rn(sc, p, acc[r]);
                acc[r] = __fmaf_rn(bi, __fadd_rn(xv.x, xv.y), acc[r]);
            }
        }
        const uint32_t e = e0 + warp;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float logit = warp_sum(acc[r]);
            if (logit_bias) logit = __fadd_rn(logit, logit_bias[e]);
            if (lane == 0 && row0 + r < rows) scratch_logits[(size_t)(row0 + r) * TF_MAX_ROUTER_EXPERTS + e] = logit;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int tk = atomicAdd(&tickets[blockIdx.x], 1u);
        is_last = (tk == gridDim.y - 1);
        if (is_last) tickets[blockIdx.x] = 0;            // ready for the next launch on this stream
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (uint32_t i = threadIdx.x; i < R * num_experts; i += kRowsThreads) {
        const uint32_t r = i / num_experts, e = i % num_experts;
        if (row0 + r < rows) {
            const float v = __ldcg(&scratch_logits[(size_t)(row0 + r) * TF_MAX_ROUTER_EXPERTS + e]);
            scores[r][e] = v;
            if (out_logits) out_logits[(size_t)(row0 + r) * num_experts + e] = v;
        }
    }
    __syncthreads();
    if (warp < R && row0 + warp < rows)
        warp_select_topk(scores[warp], num_experts, top_k, per_expert_scale, out_idx + (size_t)(row0 + warp) * top_k,
                         out_w + (size_t)(row0 + warp) * top_k, lane);
    if (grp.sorted_pairs == nullptr) return;
    // the block that completes the last row group groups all rows (second ticket, after the row tickets)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int tk = atomicAdd(&tickets[kRouterSplitRows], 1u);
        is_last = (tk == gridDim.x - 1);
        if (is_last) tickets[kRouterSplitRows] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    group_routes_in_block(out_idx, out_w, rows, top_k, num_experts, grp, smem);
}

// Many rows (batched decode, prefill): one block per row.
template <bool X_BF16>
__global__ void __launch_bounds__(kBlockRouterThreads)
router_block_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ S, const uint16_t* __restrict__ B,
                    const uint16_t* __restrict__ hidden, uint32_t hidden_stride,
                    const uint16_t* __restrict__ eff, const uint16_t* __restrict__ per_expert_scale,
                    const float* __restrict__ logit_bias,
                    uint32_t* __restrict__ out_idx, uint16_t* __restrict__ out_w, float* __restrict__ out_logits,
                    uint32_t num_experts, uint32_t d, uint32_t top_k, bool a2) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* xf = reinterpret_cast<float*>(smem);
    __shared__ float scores[TF_MAX_ROUTER_EXPERTS];
    const uint32_t row = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    stage_router_x<X_BF16>(hidden + (size_t)row * hidden_stride, eff, xf, d);
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t groups = d / kGroup;
    for (uint32_t e = warp; e < num_experts; e += kBlockRouterThreads / kWarp) {
        float logit = router_row_logit(W + (size_t)e * d, S + (size_t)e * groups, B + (size_t)e * groups, xf, groups, lane, a2);
        if (logit_bias) logit = __fadd_rn(logit, logit_bias[e]);
        if (lane == 0) {
            scores[e] = logit;
            if (out_logits) out_logits[(size_t)row * num_experts + e] = logit;
        }
    }
    __syncthreads();
    if (warp == 0)
        warp_select_topk(scores, num_experts, top_k, per_expert_scale, out_idx + (size_t)row * top_k,
                         out_w + (size_t)row * top_k, lane);
}

// Prefill-sized batches: one block per R token rows (R = 6, 7 or 8, picked by the host so that the row tiles fill whole
// rounds of the resident blocks). Same canonical arithmetic per (row, expert) as router_row_logit, but an expert's codes,
// scale and bias are decoded once per group for R rows, and a group's activations are read from shared memory once for
// four experts: the rows' scaled activations sit in shared memory as fp32 and every lane carries 4 R accumulators.
constexpr int kTileRouterRows = 8;          // most rows per block (sizes the shared memory)
constexpr int kTileExperts = 4;             // experts per warp iteration
template <bool X_BF16, int R>
__global__ void __launch_bounds__(kBlockRouterThreads, 2)
router_tile_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ S, const uint16_t* __restrict__ B,
                   const uint16_t* __restrict__ hidden, uint32_t hidden_stride,
                   const uint16_t* __restrict__ eff, const uint16_t* __restrict__ per_expert_scale,
                   const float* __restrict__ logit_bias,
                   uint32_t* __restrict__ out_idx, uint16_t* __restrict__ out_w, float* __restrict__ out_logits,
                   uint32_t rows, uint32_t num_experts, uint32_t d, uint32_t top_k) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* xf = reinterpret_cast<float*>(smem);                                   // [R][d]
    float* scores = xf + (size_t)R * d;                                           // [R][num_experts]
    const uint32_t row0 = blockIdx.x * R;
    const uint32_t nrows = rows - row0 < (uint32_t)R ? rows - row0 : (uint32_t)R;
    pdl_launch_dependents();
    pdl_wait();
    for (uint32_t c = threadIdx.x; c < d; c += blockDim.x) {
        const float es = bf16_bits_to_float(eff[c]);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float v = 0.0f;
            if ((uint32_t)r < nrows) {
                const uint16_t hb = hidden[(size_t)(row0 + r) * hidden_stride + c];
                v = __fmul_rn(X_BF16 ? bf16_bits_to_float(hb) : f16_bits_to_float(hb), es);
            }
            xf[(size_t)r * d + c] = v;
        }
    }
    __syncthreads();
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t groups = d / kGroup;
    constexpr uint32_t kWarps = kBlockRouterThreads / kWarp;
    // A warp takes four experts at a time (e, e + 8, e + 16, e + 24); experts past the end repeat the first one and
    // are not stored. The next group's codes, scales and biases are on their way while the current group is multiplied.
    for (uint32_t e0 = warp; e0 < num_experts; e0 += kTileExperts * kWarps) {
        uint32_t ex[kTileExperts];
        const uint8_t* Wp[kTileExperts];
        const uint16_t* sp[kTileExperts];
        const uint16_t* bp[kTileExperts];
#pragma unroll
        for (int j = 0; j < kTileExperts; ++j) {
            const uint32_t e = e0 + j * kWarps;
            ex[j] = e < num_experts ? e : e0;
            Wp[j] = W + (size_t)ex[j] * d + lane * 2;
            sp[j] = S + (size_t)ex[j] * groups;
            bp[j] = B + (size_t)ex[j] * groups;
        }
        float acc[kTileExperts][R];
        uint32_t wn[kTileExperts];
        uint16_t sn[kTileExperts], bn[kTileExperts];
#pragma unroll
        for (int j = 0; j < kTileExperts; ++j) {
#pragma unroll
            for (int r = 0; r < R; ++r) acc[j][r] = 0.0f;
            wn[j] = *reinterpret_cast<const uint16_t*>(Wp[j]);          // d % 64 == 0, 2-byte aligned rows
            sn[j] = sp[j][0]; bn[j] = bp[j][0];
        }
        for (uint32_t g = 0; g < groups; ++g) {
            float q0[kTileExperts], q1[kTileExperts], sc[kTileExperts], bi[kTileExperts];
#pragma unroll
            for (int j = 0; j < kTileExperts; ++j) {
                // byte -> float through the 2^23 mantissa trick (exact for 0...255)
                q0[j] = __uint_as_float(0x4B000000u | (wn[j] & 0xFFu)) - 8388608.0f;
                q1[j] = __uint_as_float(0x4B000000u | (wn[j] >> 8)) - 8388608.0f;
                sc[j] = bf16_bits_to_float(sn[j]);
                bi[j] = bf16_bits_to_float(bn[j]);
            }
            if (g + 1 < groups) {
#pragma unroll
                for (int j = 0; j < kTileExperts; ++j) {
                    wn[j] = *reinterpret_cast<const uint16_t*>(Wp[j] + (g + 1) * kGroup);
                    sn[j] = sp[j][g + 1]; bn[j] = bp[j][g + 1];
                }
            }
            const float* xg = xf + g * kGroup + lane * 2;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float2 xv = *reinterpret_cast<const float2*>(xg + (size_t)r * d);
                const float xs = __fadd_rn(xv.x, xv.y);
#pragma unroll
                for (int j = 0; j < kTileExperts; ++j) {
                    const float p = __fmaf_rn(q1[j], xv.y, __fmul_rn(q0[j], xv.x));
                    acc[j][r] = __fmaf_rn(sc[j], p, acc[j][r]);
                    acc[j][r] = __fmaf_rn(bi[j], xs, acc[j][r]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kTileExperts; ++j) {
            const bool live = e0 + j * kWarps < num_experts;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float l = warp_sum(acc[j][r]);
                if (logit_bias) l = __fadd_rn(l, logit_bias[ex[j]]);
                if (lane == 0 && live && (uint32_t)r < nrows) {
                    scores[r * num_experts + ex[j]] = l;
                    if (out_logits) out_logits[(size_t)(row0 + r) * num_experts + ex[j]] = l;
                }
            }
        }
    }
    __syncthreads();
    if ((uint32_t)warp < nrows)          // eight warps, at most eight rows
        warp_select_topk(scores + warp * num_experts, num_experts, top_k, per_expert_scale, out_idx + (size_t)(row0 + warp) * top_k,
                         out_w + (size_t)(row0 + warp) * top_k, lane);
}

// Rows per block of router_tile_kernel: the R in 6...8 whose tiles leave the fewest idle block slots in the last round
// (rounds x R is the time in units of one row's work).
static int tile_router_rows(uint32_t rows, uint32_t slots) {
    int best = kTileRouterRows;
    uint64_t best_cost = ~0ull;
    for (int r = kTileRouterRows; r >= 6; --r) {
        const uint32_t tiles = (rows + r - 1) / r;
        const uint64_t cost = (uint64_t)((tiles + slots - 1) / slots) * r;
        if (cost < best_cost) { best_cost = cost; best = r; }
    }
    return best;
}

// Scratch of the two-launch router: (approximate logit, magnitude) per (row, expert), owned by the context and grown
// on demand. Growing allocates, which a stream that is being captured must not do: the caller then takes the
// one-launch kernel.
static bool router_scratch(tf_context* ctx, cudaStream_t st, uint32_t rows, uint32_t num_experts) {
    const size_t need = (size_t)rows * num_experts * sizeof(float2);
    if (need <= ctx->router_approx_bytes) return true;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) { cudaGetLastError(); return false; }
    if (ctx->router_approx) { cudaFree(ctx->router_approx); ctx->router_approx = nullptr; ctx->router_approx_bytes = 0; }
    if (cudaMalloc(&ctx->router_approx, need) != cudaSuccess) { cudaGetLastError(); return false; }
    ctx->router_approx_bytes = need;
    return true;
}

static tf_status launch_router(tf_context* ctx, void* stream, const uint8_t* W, const uint8_t* S, const uint8_t* B,
                               const uint8_t* hidden, tf_dtype hidden_dtype, const uint8_t* eff, const uint8_t* pes,
                               const float* logit_bias, uint32_t* out_idx, uint8_t* out_w, float* out_logits,
                               uint32_t rows, uint32_t num_experts, uint32_t d, uint32_t top_k, uint32_t stride,
                               const char* name, const tf_device_routes* routes = nullptr) {
    TF_REQUIRE(ctx, aligned(S, 2) && aligned(B, 2) && aligned(hidden, 2) && aligned(eff, 2) && aligned(pes, 2) &&
                        aligned(out_w, 2) && aligned(out_idx, 4),
               TF_ERR_ALIGNMENT, "%s: 16-bit planes must be 2-byte aligned, indices 4-byte aligned", name);
    const bool a2 = aligned(W, 2);
    const size_t smem = (size_t)d * sizeof(float);
    TF_REQUIRE(ctx, smem <= 160 * 1024, TF_ERR_UNSUPPORTED, "%s: D=%u too large", name, d);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool bf = hidden_dtype == TF_BF16;
    auto Sp = reinterpret_cast<const uint16_t*>(S);
    auto Bp = reinterpret_cast<const uint16_t*>(B);
    auto hp = reinterpret_cast<const uint16_t*>(hidden);
    auto ep = reinterpret_cast<const uint16_t*>(eff);
    auto pp = reinterpret_cast<const uint16_t*>(pes);
    auto wp = reinterpret_cast<uint16_t*>(out_w);
    const bool vec16 = aligned(W, 16) && aligned(hp, 16) && aligned(ep, 16) && d % 16 == 0 && stride % 8 == 0;
    if (rows >= 2 && rows <= (uint32_t)kRouterSplitRows && vec16) {
        constexpr int R = 1;          // latency bound: a 64-token step took 4.35 ms with four rows per block, 4.28 with two, 4.16 with one
        auto k = bf ? router_rows_kernel<true, R> : router_rows_kernel<false, R>;
        size_t smem_rows = (size_t)R * d * 4 + (size_t)kRowsExpertsPerBlock * d + (size_t)kRowsExpertsPerBlock * (d / kGroup) * 4;
        RouterGroupOut grp{};
        if (routes) {
            grp = RouterGroupOut{static_cast<tf_pair*>(routes->sorted_pairs), static_cast<uint32_t*>(routes->per_expert_offsets),
                                 static_cast<uint32_t*>(routes->per_expert_counts), static_cast<tf_group*>(routes->groups),
                                 static_cast<uint32_t*>(routes->chunk_group), static_cast<uint32_t*>(routes->chunk_start),
                                 static_cast<uint32_t*>(routes->counters)};
            const size_t need = router_group_smem_bytes(rows * top_k, num_experts);
            if (need > smem_rows) smem_rows = need;
        }
        TF_REQUIRE(ctx, smem_rows <= 200 * 1024, TF_ERR_UNSUPPORTED, "%s: D=%u too large", name, d);
        static DeviceSmemCache configured_rows[2];
        if (tf_status s2 = ensure_dynamic_smem(ctx, k, configured_rows[bf ? 1 : 0], smem_rows)) return s2;
        dim3 grid((rows + R - 1) / R, (num_experts + kRowsExpertsPerBlock - 1) / kRowsExpertsPerBlock);
        launch_pdl(k, grid, dim3(kRowsThreads), smem_rows, st, W, Sp, Bp, hp, stride, ep, pp, logit_bias, out_idx, wp, out_logits,
                   ctx->router_logits, ctx->router_tickets, grp, rows, num_experts, d, top_k);
        return check_launch(ctx, name);
    }
    if (rows <= (uint32_t)kRouterSplitRows) {
        dim3 grid(rows, (num_experts + kSplitExpertsPerBlock - 1) / kSplitExpertsPerBlock);
        auto k = bf ? router_split_kernel<true> : router_split_kernel<false>;
        size_t smem_split = (size_t)d * 4 + (size_t)kSplitExpertsPerBlock * d + (size_t)kSplitExpertsPerBlock * (d / kGroup) * 4;
        RouterGroupOut grp{};
        if (routes) {
            grp = RouterGroupOut{static_cast<tf_pair*>(routes->sorted_pairs), static_cast<uint32_t*>(routes->per_expert_offsets),
                                 static_cast<uint32_t*>(routes->per_expert_counts), static_cast<tf_group*>(routes->groups),
                                 static_cast<uint32_t*>(routes->chunk_group), static_cast<uint32_t*>(routes->chunk_start),
                                 static_cast<uint32_t*>(routes->counters)};
            const size_t need = router_group_smem_bytes(rows * top_k, num_experts);
            if (need > smem_split) smem_split = need;
        }
        TF_REQUIRE(ctx, smem_split <= 200 * 1024, TF_ERR_UNSUPPORTED, "%s: D=%u too large", name, d);
        if (smem_split > 40 * 1024) TF_CUDA(ctx, cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_split));
        launch_pdl(k, grid, dim3(kSplitThreads), smem_split, st, W, Sp, Bp, hp, stride, ep, pp, logit_bias, out_idx, wp, out_logits,
                   ctx->router_logits, ctx->router_tickets, grp, num_experts, d, top_k, a2);
        return check_launch(ctx, name);
    } else if (rows >= ctx->router_tensorcore_min_rows && !out_logits && vec16 && d % kApxChunk == 0 && aligned(S, 8) && aligned(B, 8) &&
               num_experts <= TF_MAX_ROUTER_EXPERTS && top_k <= (uint32_t)kWarp && top_k <= num_experts &&
               router_recheck_smem_bytes(d, num_experts) <= 200 * 1024 && router_scratch(ctx, st, rows, num_experts)) {
        // logits on the tensor cores, then the canonical logits of the few experts that can reach the top k
        auto ka = bf ? router_approx_kernel<true> : router_approx_kernel<false>;
        constexpr int kProductionGroups = 2816 / kGroup;          // the recheck keeps an expert's 44 code words in registers
        const bool fixed = d / kGroup == (uint32_t)kProductionGroups;
        auto kr = fixed ? (bf ? router_recheck_kernel<true, kProductionGroups> : router_recheck_kernel<false, kProductionGroups>)
                        : (bf ? router_recheck_kernel<true, 0> : router_recheck_kernel<false, 0>);
        static DeviceSmemCache configured_approx[2], configured_recheck[4];
        const size_t smem_a = router_approx_smem_bytes(), smem_r = router_recheck_smem_bytes(d, num_experts);
        if (tf_status s = ensure_dynamic_smem(ctx, ka, configured_approx[bf ? 1 : 0], smem_a)) return s;
        if (tf_status s = ensure_dynamic_smem(ctx, kr, configured_recheck[(bf ? 1 : 0) + (fixed ? 2 : 0)], smem_r)) return s;
        float2* approx = reinterpret_cast<float2*>(ctx->router_approx);
        launch_pdl(ka, dim3((rows + kApxTokens - 1) / kApxTokens, (num_experts + kApxExperts - 1) / kApxExperts), dim3(kApxThreads),
                   smem_a, st, W, Sp, Bp, hp, stride, ep, approx, rows, num_experts, d);
        if (tf_status s = check_launch(ctx, name)) return s;
        launch_pdl(kr, dim3((rows + kRecheckWarps - 1) / kRecheckWarps), dim3(kRecheckWarps * kWarp), smem_r, st, W, Sp, Bp, hp, stride,
                   ep, pp, logit_bias, static_cast<const float2*>(approx), out_idx, wp, rows, num_experts, d, top_k);
    } else if (rows >= 256 && a2 && (size_t)kTileRouterRows * (d + num_experts) * 4 <= 100 * 1024) {
        const int R = tile_router_rows(rows, (uint32_t)ctx->sm_count * 2u);
        void (*k)(const uint8_t*, const uint16_t*, const uint16_t*, const uint16_t*, uint32_t, const uint16_t*, const uint16_t*, const float*,
                  uint32_t*, uint16_t*, float*, uint32_t, uint32_t, uint32_t, uint32_t);
        if (R == 6) k = bf ? router_tile_kernel<true, 6> : router_tile_kernel<false, 6>;
        else if (R == 7) k = bf ? router_tile_kernel<true, 7> : router_tile_kernel<false, 7>;
        else k = bf ? router_tile_kernel<true, 8> : router_tile_kernel<false, 8>;
        const size_t smem_tile = (size_t)R * (d + num_experts) * 4;
        static DeviceSmemCache configured[2][3];
        if (tf_status s = ensure_dynamic_smem(ctx, k, configured[bf ? 1 : 0][R - 6], smem_tile)) return s;
        launch_pdl(k, dim3((rows + R - 1) / R), dim3(kBlockRouterThreads), smem_tile, st, W, Sp, Bp, hp, stride,
                   ep, pp, logit_bias, out_idx, wp, out_logits, rows, num_experts, d, top_k);
    } else {
        auto k = bf ? router_block_kernel<true> : router_block_kernel<false>;
        if (smem > 40 * 1024) TF_CUDA(ctx, cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        launch_pdl(k, dim3(rows), dim3(kBlockRouterThreads), smem, st, W, Sp, Bp, hp, stride, ep, pp, logit_bias, out_idx, wp, out_logits,
                   num_experts, d, top_k, a2);
    }
    return check_launch(ctx, name);
}

}  // namespace tf

extern "C" {

tf_status tf_router_gemma4(tf_context* ctx, void* stream, const void* weights, uint64_t weights_off,
                           const void* scales, uint64_t scales_off, const void* biases, uint64_t biases_off,
                           const void* hidden, const void* effective_scale, uint64_t effective_scale_off,
                           const void* per_expert_scale, uint64_t per_expert_scale_off,
                           uint32_t* out_indices, void* out_weights, float* out_logits,
                           uint32_t num_experts, uint32_t d, uint32_t top_k) {
    const char* name = "tf_router_gemma4";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, weights && scales && biases && hidden && effective_scale && per_expert_scale && out_indices && out_weights,
               TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, d > 0 && d % tf::kGroup == 0, TF_ERR_INVALID_ARGUMENT, "%s: D=%u must be a multiple of 64", name, d);
    TF_REQUIRE(ctx, num_experts > 0 && num_experts <= TF_MAX_ROUTER_EXPERTS, TF_ERR_INVALID_ARGUMENT,
               "%s: numExperts=%u must be in 1...256", name, num_experts);
    TF_REQUIRE(ctx, top_k == TF_MAX_TOP_K, TF_ERR_INVALID_ARGUMENT, "%s: topK must be 8, got %u", name, top_k);
    TF_REQUIRE(ctx, num_experts >= top_k, TF_ERR_INVALID_ARGUMENT, "%s: numExperts < topK", name);
    return tf::launch_router(ctx, stream, tf::byte_ptr(weights, weights_off), tf::byte_ptr(scales, scales_off),
                             tf::byte_ptr(biases, biases_off), static_cast<const uint8_t*>(hidden), TF_FP16,
                             tf::byte_ptr(effective_scale, effective_scale_off),
                             tf::byte_ptr(per_expert_scale, per_expert_scale_off), nullptr, out_indices,
                             static_cast<uint8_t*>(out_weights), out_logits, 1, num_experts, d, top_k, d, name);
}

tf_status tf_router_gemma4_block(tf_context* ctx, void* stream, const void* weights, uint64_t weights_off,
                                 const void* scales, uint64_t scales_off, const void* biases, uint64_t biases_off,
                                 const void* hidden, uint64_t hidden_off, tf_dtype hidden_dtype,
                                 const void* effective_scale, uint64_t effective_scale_off,
                                 const void* per_expert_scale, uint64_t per_expert_scale_off,
                                 const float* logit_bias,
                                 uint32_t* out_indices, uint64_t out_indices_off,
                                 void* out_weights, uint64_t out_weights_off, float* out_logits,
                                 uint32_t query_count, uint32_t num_experts, uint32_t d,
                                 uint32_t top_k, uint32_t hidden_stride_elements) {
    const char* name = "tf_router_gemma4_block";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, weights && scales && biases && hidden && effective_scale && per_expert_scale && out_indices && out_weights,
               TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, query_count > 0, TF_ERR_INVALID_ARGUMENT, "%s: queryCount must be positive", name);
    TF_REQUIRE(ctx, num_experts > 0 && num_experts <= TF_MAX_ROUTER_EXPERTS, TF_ERR_INVALID_ARGUMENT,
               "%s: numExperts > 256 is not supported", name);
    TF_REQUIRE(ctx, top_k > 0 && top_k <= TF_MAX_TOP_K, TF_ERR_INVALID_ARGUMENT,
               "%s: topK must be in 1...%d, got %u", name, TF_MAX_TOP_K, top_k);
    TF_REQUIRE(ctx, num_experts >= top_k, TF_ERR_INVALID_ARGUMENT, "%s: numExperts < topK", name);
    TF_REQUIRE(ctx, d > 0 && d % tf::kGroup == 0, TF_ERR_INVALID_ARGUMENT, "%s: D must be a multiple of 64", name);
    TF_REQUIRE(ctx, hidden_stride_elements >= d, TF_ERR_INVALID_ARGUMENT, "%s: hidden stride is too small", name);
    TF_REQUIRE(ctx, hidden_dtype == TF_FP16 || hidden_dtype == TF_BF16, TF_ERR_INVALID_ARGUMENT, "%s: bad hidden dtype", name);
    return tf::launch_router(ctx, stream, tf::byte_ptr(weights, weights_off), tf::byte_ptr(scales, scales_off),
                             tf::byte_ptr(biases, biases_off), tf::byte_ptr(hidden, hidden_off), hidden_dtype,
                             tf::byte_ptr(effective_scale, effective_scale_off),
                             tf::byte_ptr(per_expert_scale, per_expert_scale_off), logit_bias,
                             reinterpret_cast<uint32_t*>(tf::byte_ptr(static_cast<void*>(out_indices), out_indices_off)),
                             tf::byte_ptr(out_weights, out_weights_off), out_logits, query_count, num_experts, d, top_k,
                             hidden_stride_elements, name);
}

tf_status tf_router_gemma4_block_grouped(tf_context* ctx, void* stream, const void* weights, uint64_t weights_off,
                                         const void* scales, uint64_t scales_off, const void* biases, uint64_t biases_off,
                                         const void* hidden, uint64_t hidden_off, tf_dtype hidden_dtype,
                                         const void* effective_scale, uint64_t effective_scale_off,
                                         const void* per_expert_scale, uint64_t per_expert_scale_off,
                                         const float* logit_bias, uint32_t* out_indices, void* out_weights,
                                         uint32_t query_count, uint32_t num_experts, uint32_t d, uint32_t top_k,
                                         uint32_t hidden_stride_elements, const tf_device_routes* routes) {
    const char* name = "tf_router_gemma4_block_grouped";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, routes && routes->sorted_pairs && routes->per_expert_offsets && routes->per_expert_counts && routes->groups &&
                        routes->chunk_group && routes->chunk_start && routes->counters,
               TF_ERR_INVALID_ARGUMENT, "%s: NULL routes buffer", name);
    if (query_count > (uint32_t)tf::kRouterSplitRows) {
        // larger blocks: the router kernels for many rows, then the grouping launch
        tf_status s = tf_router_gemma4_block(ctx, stream, weights, weights_off, scales, scales_off, biases, biases_off, hidden,
                                             hidden_off, hidden_dtype, effective_scale, effective_scale_off, per_expert_scale,
                                             per_expert_scale_off, logit_bias, out_indices, 0, out_weights, 0, nullptr,
                                             query_count, num_experts, d, top_k, hidden_stride_elements);
        if (s) return s;
        return tf_group_routes_device(ctx, stream, out_indices, out_weights, query_count, top_k, num_experts, routes);
    }
    TF_REQUIRE(ctx, weights && scales && biases && hidden && effective_scale && per_expert_scale && out_indices && out_weights,
               TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, query_count > 0, TF_ERR_INVALID_ARGUMENT, "%s: queryCount must be positive", name);
    TF_REQUIRE(ctx, num_experts > 0 && num_experts <= TF_MAX_ROUTER_EXPERTS, TF_ERR_INVALID_ARGUMENT,
               "%s: numExperts > 256 is not supported", name);
    TF_REQUIRE(ctx, top_k > 0 && top_k <= TF_MAX_TOP_K && num_experts >= top_k, TF_ERR_INVALID_ARGUMENT,
               "%s: topK must be in 1...%d and at most numExperts, got %u", name, TF_MAX_TOP_K, top_k);
    TF_REQUIRE(ctx, d > 0 && d % tf::kGroup == 0 && hidden_stride_elements >= d, TF_ERR_INVALID_ARGUMENT,
               "%s: D must be a multiple of 64 and the stride at least D", name);
    TF_REQUIRE(ctx, hidden_dtype == TF_FP16 || hidden_dtype == TF_BF16, TF_ERR_INVALID_ARGUMENT, "%s: bad hidden dtype", name);
    return tf::launch_router(ctx, stream, tf::byte_ptr(weights, weights_off), tf::byte_ptr(scales, scales_off),
                             tf::byte_ptr(biases, biases_off), tf::byte_ptr(hidden, hidden_off), hidden_dtype,
                             tf::byte_ptr(effective_scale, effective_scale_off),
                             tf::byte_ptr(per_expert_scale, per_expert_scale_off), logit_bias, out_indices,
                             static_cast<uint8_t*>(out_weights), nullptr, query_count, num_experts, d, top_k,
                             hidden_stride_elements, name, routes);
}

}  // extern "C"
