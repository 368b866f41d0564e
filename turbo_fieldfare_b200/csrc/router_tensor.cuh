// Router of prefill-sized batches in two launches, with the same indices and weights as the canonical fp32 router
// (Metal/MoE/moe.metal:135-185 fixes a per-logit order of fp32 operations; router_row_logit restates it).
//
//   1. router_approx_kernel: all logits on the tensor cores (mma.sync.m16n8k16, fp32 accumulation). The 8-bit codes
//      enter the A operand as exact fp16 integers; an activation x is split into two fp16 numbers hi + lo of
//      x * 2^10, so the operands carry the inputs (nearly) exactly and the only differences from the canonical value
//      are rounding errors of the sums. Beside each logit the kernel accumulates a MAGNITUDE
//      sum_g (255 |s_g| + |b_g|) * (sum_{i in g} |x_i|), an upper bound of the sum of |terms| of either evaluation.
//   2. router_recheck_kernel: per token, eps_e = kRelError * magnitude_e bounds |approximate - canonical| (derivation
//      below). With lower_e = v_e - eps_e and upper_e = v_e + eps_e, the top_k-th largest lower value LB is reached by
//      top_k canonical logits, so an expert with upper_e < LB cannot be among the canonical top_k, whatever the ties.
//      All other experts (typically top_k plus one or two) get their canonical logit computed in the canonical
//      order, and the usual top-k + softmax runs over those. Rows with a non-finite value anywhere re-check every expert.
//
// Error budget behind kRelError = 2^-13 (relative to the magnitude, which over-estimates sum |terms| by about 1.5):
//   canonical order: a term passes at most 2 + 2 * groups + 5 fp32 roundings, 95 * 2^-24 = 5.7e-6 at 44 groups;
//   tensor cores: products of fp16 numbers are exact in fp32; a k = 16 step adds 16 products and the accumulator with
//     aligned, truncated addends, at most 18 * 2^-23 of the step's magnitude; 8 steps per group: 1.7e-5;
//   the group epilogue and the 88 accumulations behind it: 5.3e-6; the group sums of x: 1e-6;
//   the fp16 split: |x * 2^10 - hi - lo| <= 2^-22 |x * 2^10| + 2^-25, the absolute part is added to the group's |x| sum.
//   Sum 2.9e-5, kRelError = 1.2e-4 leaves a factor four.
#pragma once

#include <cuda_fp16.h>

#include "router.cuh"

namespace tf {

constexpr int kApxTokens = 16;                     // tokens per block of router_approx_kernel (two n = 8 tiles)
constexpr int kApxExperts = 128;                   // experts per block: eight warps, one 16-row MMA tile each
constexpr int kApxChunk = 256;                     // columns staged at a time (four groups)
constexpr int kApxWPitch = kApxChunk + 64;         // bytes per staged weight row: the rows of a quarter-warp load fill all banks
constexpr int kApxXPitch = kApxChunk * 2 + 16;     // bytes per staged activation row (fp16): the same for the B fragments
constexpr int kApxThreads = 256;
constexpr float kApxPrescale = 1024.0f;            // activations are split as x * 2^10 = hi + lo
constexpr float kApxRelError = 1.220703125e-04f;   // 2^-13
constexpr int kRecheckWarps = 8;                   // tokens per block of router_recheck_kernel

__host__ __device__ inline size_t router_approx_smem_bytes() {
    return 2 * (size_t)kApxExperts * kApxWPitch + 2 * (size_t)kApxTokens * kApxXPitch + 2 * 4 * kApxTokens * sizeof(float);
}
__host__ __device__ inline size_t router_recheck_smem_bytes(uint32_t d, uint32_t num_experts) {
    return (size_t)kRecheckWarps * ((size_t)d + num_experts) * sizeof(float);
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* global_src) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(global_src) : "memory");
}

__device__ __forceinline__ void mma_f16_f32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two bytes of `word` (selected by `sel`) as two exact fp16 integers: the bytes become the low mantissa bits of
// 1024 + byte (0x6400 | byte), then 1024 is subtracted.
__device__ __forceinline__ uint32_t bytes_to_half2(uint32_t word, uint32_t sel) {
    const uint32_t biased = __byte_perm(word, 0x64646464u, sel);
    const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&biased), __half2half2(__ushort_as_half((unsigned short)0x6400)));
    return *reinterpret_cast<const uint32_t*>(&v);
}

// out[token][expert] = (approximate logit without the logit bias, magnitude), both in units of x (not x * 2^10).
// Grid: (ceil(rows / 16), ceil(num_experts / 128)). Column k of an MMA step is mapped to the matrix column
// 16 t + 4 step + {0, 1} (k = 2 t + {0, 1}) and 16 t + 4 step + {2, 3} (k = 2 t + 8 + {0, 1}) of the group, for both
// operands, so a thread's 16 weight bytes and 16 activation values of a group are contiguous.
template <bool X_BF16>
__global__ void __launch_bounds__(kApxThreads, 2)
router_approx_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ S, const uint16_t* __restrict__ B,
                     const uint16_t* __restrict__ hidden, uint32_t hidden_stride, const uint16_t* __restrict__ eff,
                     float2* __restrict__ out, uint32_t rows, uint32_t num_experts, uint32_t d) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* Wc0 = smem;                                                   // [2][128][kApxWPitch]
    uint8_t* Hi = Wc0 + 2 * (size_t)kApxExperts * kApxWPitch;             // [16][kApxXPitch]
    uint8_t* Lo = Hi + (size_t)kApxTokens * kApxXPitch;
    float* XS = reinterpret_cast<float*>(Lo + (size_t)kApxTokens * kApxXPitch);   // [4 groups][16 tokens]: sum of x * 2^10
    float* XA = XS + 4 * kApxTokens;                                       // the same of |x * 2^10| (+ the split's absolute part)
    const int tid = threadIdx.x, warp = tid / kWarp, lane = tid % kWarp, g = lane >> 2, t = lane & 3;
    const uint32_t tok0 = blockIdx.x * kApxTokens, e0 = blockIdx.y * kApxExperts;
    const uint32_t groups = d / kGroup;
    const uint32_t last = num_experts - 1;
    const uint32_t e_lo = min(e0 + warp * 16 + g, last), e_hi = min(e0 + warp * 16 + g + 8, last);   // rows past the end repeat the last one
    pdl_launch_dependents();
    pdl_wait();
    float acc[2][4] = {}, mag[2][4] = {};
    // The next chunk's weight codes (cp.async into the other buffer) and activation rows (registers) are requested
    // before the current chunk is multiplied.
    auto request_weights = [&](uint32_t c0, uint8_t* dst) {
#pragma unroll
        for (int i = 0; i < (kApxExperts * kApxChunk / 16) / kApxThreads; ++i) {
            const uint32_t idx = tid + kApxThreads * i, row = idx >> 4, seg = idx & 15;
            const uint32_t e = min(e0 + row, last);
            cp_async_16(dst + (size_t)row * kApxWPitch + seg * 16, W + (size_t)e * d + c0 + seg * 16);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    uint4 hreg[2], ereg;
    auto request_rows = [&](uint32_t c0) {
        ereg = *reinterpret_cast<const uint4*>(eff + c0 + lane * 8);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t tok = tok0 + warp + 8 * h;
            hreg[h] = tok < rows ? *reinterpret_cast<const uint4*>(hidden + (size_t)tok * hidden_stride + c0 + lane * 8) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    request_weights(0, Wc0);
    request_rows(0);
    uint32_t ci = 0;
    for (uint32_t c0 = 0; c0 < d; c0 += kApxChunk, ++ci) {
        uint8_t* Wc = Wc0 + (size_t)(ci & 1u) * kApxExperts * kApxWPitch;
        __syncthreads();                         // the previous chunk's fragments have been read
        // activations: a warp stages the 256 columns of tokens `warp` and `warp + 8`, eight columns per lane (zero bits
        // are +0 in fp16 and bf16: rows past the end contribute nothing)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t tl = warp + 8 * h;
            float y[8];
            const uint32_t hw[4] = {hreg[h].x, hreg[h].y, hreg[h].z, hreg[h].w}, ew[4] = {ereg.x, ereg.y, ereg.z, ereg.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint16_t h0 = (uint16_t)(hw[j] & 0xFFFFu), h1 = (uint16_t)(hw[j] >> 16);
                const float x0 = __fmul_rn(X_BF16 ? bf16_bits_to_float(h0) : f16_bits_to_float(h0), bf16_bits_to_float((uint16_t)(ew[j] & 0xFFFFu)));
                const float x1 = __fmul_rn(X_BF16 ? bf16_bits_to_float(h1) : f16_bits_to_float(h1), bf16_bits_to_float((uint16_t)(ew[j] >> 16)));
                y[2 * j] = x0 * kApxPrescale;
                y[2 * j + 1] = x1 * kApxPrescale;
            }
            uint32_t hiw[4], low[4];
            float sum = 0.0f, asum = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 hh = __floats2half2_rn(y[2 * j], y[2 * j + 1]);
                const float2 hf = __half22float2(hh);
                const __half2 ll = __floats2half2_rn(y[2 * j] - hf.x, y[2 * j + 1] - hf.y);
                hiw[j] = *reinterpret_cast<const uint32_t*>(&hh);
                low[j] = *reinterpret_cast<const uint32_t*>(&ll);
                sum += y[2 * j] + y[2 * j + 1];
                asum += fabsf(y[2 * j]) + fabsf(y[2 * j + 1]);
            }
            *reinterpret_cast<uint4*>(Hi + (size_t)tl * kApxXPitch + lane * 16) = make_uint4(hiw[0], hiw[1], hiw[2], hiw[3]);
            *reinterpret_cast<uint4*>(Lo + (size_t)tl * kApxXPitch + lane * 16) = make_uint4(low[0], low[1], low[2], low[3]);
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                sum += __shfl_xor_sync(kFullMask, sum, o);
                asum += __shfl_xor_sync(kFullMask, asum, o);
            }
            if ((lane & 7) == 0) {
                XS[(lane >> 3) * kApxTokens + tl] = sum;
                XA[(lane >> 3) * kApxTokens + tl] = asum + 0.015625f;     // 64 x 2^-25 / kApxRelError, rounded up
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (c0 + kApxChunk < d) {
            request_weights(c0 + kApxChunk, Wc0 + (size_t)((ci + 1u) & 1u) * kApxExperts * kApxWPitch);
            request_rows(c0 + kApxChunk);
        }
        // scales and biases of the chunk's four groups for this thread's two expert rows (8-byte aligned: groups % 4 == 0)
        const uint32_t gq = c0 / kGroup;
        const uint2 s_lo = *reinterpret_cast<const uint2*>(S + (size_t)e_lo * groups + gq);
        const uint2 s_hi = *reinterpret_cast<const uint2*>(S + (size_t)e_hi * groups + gq);
        const uint2 b_lo = *reinterpret_cast<const uint2*>(B + (size_t)e_lo * groups + gq);
        const uint2 b_hi = *reinterpret_cast<const uint2*>(B + (size_t)e_hi * groups + gq);
        const uint32_t slw[2] = {s_lo.x, s_lo.y}, shw[2] = {s_hi.x, s_hi.y}, blw[2] = {b_lo.x, b_lo.y}, bhw[2] = {b_hi.x, b_hi.y};
#pragma unroll
        for (int gi = 0; gi < 4; ++gi) {
            const uint4 a_lo = *reinterpret_cast<const uint4*>(Wc + (size_t)(warp * 16 + g) * kApxWPitch + gi * 64 + t * 16);
            const uint4 a_hi = *reinterpret_cast<const uint4*>(Wc + (size_t)(warp * 16 + g + 8) * kApxWPitch + gi * 64 + t * 16);
            const uint32_t alw[4] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w}, ahw[4] = {a_hi.x, a_hi.y, a_hi.z, a_hi.w};
            uint32_t af[4][4];
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                af[s][0] = bytes_to_half2(alw[s], 0x5140u); af[s][1] = bytes_to_half2(ahw[s], 0x5140u);
                af[s][2] = bytes_to_half2(alw[s], 0x7362u); af[s][3] = bytes_to_half2(ahw[s], 0x7362u);
            }
            float P[2][4] = {};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const size_t off = (size_t)(nt * 8 + g) * kApxXPitch + (size_t)(gi * 64 + t * 16) * 2;
                const uint4 h0 = *reinterpret_cast<const uint4*>(Hi + off), h1 = *reinterpret_cast<const uint4*>(Hi + off + 16);
                const uint4 l0 = *reinterpret_cast<const uint4*>(Lo + off), l1 = *reinterpret_cast<const uint4*>(Lo + off + 16);
                const uint32_t bh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
                const uint32_t bl[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    mma_f16_f32(P[nt], af[s][0], af[s][1], af[s][2], af[s][3], bh[2 * s], bh[2 * s + 1]);
                    mma_f16_f32(P[nt], af[s][0], af[s][1], af[s][2], af[s][3], bl[2 * s], bl[2 * s + 1]);
                }
            }
            const uint32_t sh = (gi & 1) * 16;
            const float sl = bf16_bits_to_float((uint16_t)(slw[gi >> 1] >> sh)), sH = bf16_bits_to_float((uint16_t)(shw[gi >> 1] >> sh));
            const float bL = bf16_bits_to_float((uint16_t)(blw[gi >> 1] >> sh)), bH = bf16_bits_to_float((uint16_t)(bhw[gi >> 1] >> sh));
            const float ml = fmaf(255.0f, fabsf(sl), fabsf(bL)), mh = fmaf(255.0f, fabsf(sH), fabsf(bH));
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float2 xs = *reinterpret_cast<const float2*>(XS + gi * kApxTokens + nt * 8 + 2 * t);
                const float2 xa = *reinterpret_cast<const float2*>(XA + gi * kApxTokens + nt * 8 + 2 * t);
                acc[nt][0] = fmaf(sl, P[nt][0], fmaf(bL, xs.x, acc[nt][0]));
                acc[nt][1] = fmaf(sl, P[nt][1], fmaf(bL, xs.y, acc[nt][1]));
                acc[nt][2] = fmaf(sH, P[nt][2], fmaf(bH, xs.x, acc[nt][2]));
                acc[nt][3] = fmaf(sH, P[nt][3], fmaf(bH, xs.y, acc[nt][3]));
                mag[nt][0] = fmaf(ml, xa.x, mag[nt][0]);
                mag[nt][1] = fmaf(ml, xa.y, mag[nt][1]);
                mag[nt][2] = fmaf(mh, xa.x, mag[nt][2]);
                mag[nt][3] = fmaf(mh, xa.y, mag[nt][3]);
            }
        }
    }
    const float unscale = 1.0f / kApxPrescale;
    const uint32_t er_lo = e0 + warp * 16 + g, er_hi = er_lo + 8;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const uint32_t tok = tok0 + nt * 8 + 2 * t + c;
            if (tok >= rows) continue;
            if (er_lo < num_experts) out[(size_t)tok * num_experts + er_lo] = make_float2(acc[nt][c] * unscale, mag[nt][c] * unscale);
            if (er_hi < num_experts) out[(size_t)tok * num_experts + er_hi] = make_float2(acc[nt][2 + c] * unscale, mag[nt][2 + c] * unscale);
        }
    }
}

// Canonical logits with the expert's codes, scales and biases read from global memory and the row's scaled activations
// from shared memory (the arithmetic and order of router_row_logit), kLogitChunk groups at a time: the loads of a chunk
// are issued together, one chunk ahead of the arithmetic (across experts too); lane i holds the scale and bias of the
// chunk's group i.
constexpr int kLogitChunk = 16;
__device__ __forceinline__ void router_logit_load(const uint8_t* __restrict__ Wrow, const uint16_t* __restrict__ s_row,
                                                  const uint16_t* __restrict__ b_row, uint32_t g0, uint32_t groups, int lane,
                                                  uint32_t (&w)[kLogitChunk], uint32_t& sb) {
#pragma unroll
    for (int i = 0; i < kLogitChunk; ++i)
        w[i] = g0 + i < groups ? (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(Wrow + (size_t)(g0 + i) * kGroup + lane * 2)) : 0u;
    sb = 0u;
    if (lane < kLogitChunk && g0 + lane < groups) sb = (uint32_t)__ldg(s_row + g0 + lane) | ((uint32_t)__ldg(b_row + g0 + lane) << 16);
}
__device__ __forceinline__ float router_logit_chunk(float acc, const uint32_t (&wv)[kLogitChunk], uint32_t sb, const float* xf,
                                                    uint32_t g0, uint32_t groups, int lane) {
#pragma unroll
    for (int i = 0; i < kLogitChunk; ++i) {
        const uint32_t sbv = __shfl_sync(kFullMask, sb, i);
        if (g0 + i < groups) {                                                          // the same for the whole warp
            const uint32_t w = wv[i];
            const float q0 = __uint_as_float(0x4B000000u | (w & 0xFFu)) - 8388608.0f;      // exact for 0...255
            const float q1 = __uint_as_float(0x4B000000u | (w >> 8)) - 8388608.0f;
            const float2 xv = *reinterpret_cast<const float2*>(xf + (size_t)(g0 + i) * kGroup + lane * 2);
            const float s = bf16_bits_to_float((uint16_t)(sbv & 0xFFFFu));
            const float b = bf16_bits_to_float((uint16_t)(sbv >> 16));
            const float p = __fmaf_rn(q1, xv.y, __fmul_rn(q0, xv.x));
            acc = __fmaf_rn(s, p, acc);
            acc = __fmaf_rn(b, __fadd_rn(xv.x, xv.y), acc);
        }
    }
    return acc;
}
// The lowest expert of the candidate masks (32 experts per word), removed from them; 0xFFFFFFFF when none is left.
template <int N>
__device__ __forceinline__ uint32_t pop_candidate(uint32_t (&masks)[N]) {
    uint32_t e = 0xFFFFFFFFu;
#pragma unroll
    for (int j = N - 1; j >= 0; --j)
        if (masks[j]) e = (uint32_t)(__ffs((int)masks[j]) - 1) + j * kWarp;
    if (e != 0xFFFFFFFFu) {
#pragma unroll
        for (int j = 0; j < N; ++j)
            if ((uint32_t)j == e / kWarp) masks[j] &= masks[j] - 1u;
    }
    return e;
}

// The same for a group count known at compile time (the production width): all of an expert's codes are requested at
// once, lane l holds the scale and bias of groups l and l + 32, and nothing in the loop is guarded.
template <int GROUPS>
struct LogitOperands {
    uint32_t w[GROUPS];
    uint32_t sb0, sb1;
};
template <int GROUPS>
__device__ __forceinline__ void router_logit_load_all(const uint8_t* __restrict__ Wrow, const uint16_t* __restrict__ s_row,
                                                      const uint16_t* __restrict__ b_row, int lane, LogitOperands<GROUPS>& r) {
    static_assert(GROUPS <= 2 * kWarp, "two scale words per lane");
    const uint8_t* wl = Wrow + lane * 2;
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) r.w[g] = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(wl + g * kGroup));
    r.sb0 = lane < GROUPS ? (uint32_t)__ldg(s_row + lane) | ((uint32_t)__ldg(b_row + lane) << 16) : 0u;
    r.sb1 = lane + kWarp < GROUPS ? (uint32_t)__ldg(s_row + lane + kWarp) | ((uint32_t)__ldg(b_row + lane + kWarp) << 16) : 0u;
}
template <int GROUPS>
__device__ __forceinline__ float router_logit_all(const LogitOperands<GROUPS>& r, const float* xf, int lane) {
    const float* xl = xf + lane * 2;
    float acc = 0.0f;
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
        const uint32_t sbv = __shfl_sync(kFullMask, g < kWarp ? r.sb0 : r.sb1, g % kWarp);
        const uint32_t w = r.w[g];
        const float q0 = __uint_as_float(0x4B000000u | (w & 0xFFu)) - 8388608.0f;      // exact for 0...255
        const float q1 = __uint_as_float(0x4B000000u | (w >> 8)) - 8388608.0f;
        const float2 xv = *reinterpret_cast<const float2*>(xl + g * kGroup);
        const float s = __uint_as_float(sbv << 16);
        const float b = __uint_as_float(sbv & 0xFFFF0000u);
        const float p = __fmaf_rn(q1, xv.y, __fmul_rn(q0, xv.x));
        acc = __fmaf_rn(s, p, acc);
        acc = __fmaf_rn(b, __fadd_rn(xv.x, xv.y), acc);
    }
    return warp_sum(acc);
}

// One warp per token: candidates from the approximate logits and their bounds, canonical logits of the candidates,
// top-k and softmax as in every other router kernel.
template <bool X_BF16, int GROUPS>          // GROUPS: d / 64 when known at compile time, 0 for any width
__global__ void __launch_bounds__(kRecheckWarps * kWarp, 2)
router_recheck_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ S, const uint16_t* __restrict__ B,
                      const uint16_t* __restrict__ hidden, uint32_t hidden_stride, const uint16_t* __restrict__ eff,
                      const uint16_t* __restrict__ per_expert_scale, const float* __restrict__ logit_bias,
                      const float2* __restrict__ approx, uint32_t* __restrict__ out_idx, uint16_t* __restrict__ out_w,
                      uint32_t rows, uint32_t num_experts, uint32_t d, uint32_t top_k) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    float* xf = reinterpret_cast<float*>(smem) + (size_t)warp * d;
    float* scores = reinterpret_cast<float*>(smem) + (size_t)kRecheckWarps * d + (size_t)warp * num_experts;
    const uint32_t row = blockIdx.x * kRecheckWarps + warp;
    const uint32_t groups = d / kGroup;
    pdl_launch_dependents();
    pdl_wait();
    if (row >= rows) return;                     // warps are independent: no block barrier below
    const uint16_t* hrow = hidden + (size_t)row * hidden_stride;
    for (uint32_t c0 = lane * 2; c0 < d; c0 += 8 * 2 * kWarp) {          // eight independent pairs of loads at a time
        uint32_t hv[8], ev[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t c = c0 + u * 2 * kWarp;
            hv[u] = c < d ? *reinterpret_cast<const uint32_t*>(hrow + c) : 0u;
            ev[u] = c < d ? *reinterpret_cast<const uint32_t*>(eff + c) : 0u;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t c = c0 + u * 2 * kWarp;
            const uint16_t h0 = (uint16_t)(hv[u] & 0xFFFFu), h1 = (uint16_t)(hv[u] >> 16);
            const float x0 = __fmul_rn(X_BF16 ? bf16_bits_to_float(h0) : f16_bits_to_float(h0), bf16_bits_to_float((uint16_t)(ev[u] & 0xFFFFu)));
            const float x1 = __fmul_rn(X_BF16 ? bf16_bits_to_float(h1) : f16_bits_to_float(h1), bf16_bits_to_float((uint16_t)(ev[u] >> 16)));
            if (c < d) *reinterpret_cast<float2*>(xf + c) = make_float2(x0, x1);
        }
    }
    constexpr int kPerLane = TF_MAX_ROUTER_EXPERTS / kWarp;
    float upper[kPerLane];
    uint32_t key[kPerLane];
    bool bad = false;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
        const uint32_t e = lane + j * kWarp;
        upper[j] = -INFINITY;
        key[j] = 0u;
        if (e < num_experts) {
            const float2 am = approx[(size_t)row * num_experts + e];
            float v = am.x;
            if (!isfinite(am.x) || !isfinite(am.y)) bad = true;
            if (logit_bias) v = __fadd_rn(v, logit_bias[e]);
            if (v == -INFINITY) {
                key[j] = topk_score_key(-INFINITY);             // a -inf bias: the canonical logit is -inf as well
            } else if (!isfinite(v)) {
                bad = true;
            } else {
                const float eps = fmaf(kApxRelError, am.y, fabsf(v) * 2.384185791015625e-07f);    // + 2^-22 |v|: the bias add
                upper[j] = v + eps;
                key[j] = topk_score_key(v - eps);
            }
        }
    }
    // the top_k-th largest lower bound
    uint32_t lb_key = 0u;
    for (uint32_t r = 0; r < top_k; ++r) {
        uint32_t best = 0u;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) best = max(best, key[j]);
        lb_key = __reduce_max_sync(kFullMask, best);
        const uint32_t who = __reduce_min_sync(kFullMask, (best == lb_key && lb_key != 0u) ? (uint32_t)lane : 32u);
        if ((uint32_t)lane == who) {
            bool done = false;
#pragma unroll
            for (int j = 0; j < kPerLane; ++j)
                if (!done && key[j] == lb_key) { key[j] = 0u; done = true; }
        }
    }
    if (lb_key == 0u) bad = true;                 // fewer than top_k comparable experts
    bad = __any_sync(kFullMask, bad);
    const float lb = bad ? -INFINITY : topk_key_score(lb_key);
    uint32_t masks[kPerLane];
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
        const uint32_t e = lane + j * kWarp;
        const bool cand = e < num_experts && (bad || upper[j] >= lb);
        masks[j] = __ballot_sync(kFullMask, cand);
        if (e < num_experts) scores[e] = -INFINITY;
    }
    __syncwarp();
    // (expert, chunk) pairs in one software pipeline: the next pair's loads are issued before the current pair is multiplied
    uint32_t ld_e = pop_candidate(masks), ld_g = 0u;
    if constexpr (GROUPS > 0) {
        // two operand sets used in turns: the next candidate's loads are in flight while the current one is multiplied
        LogitOperands<GROUPS> ra, rb;
        auto finish = [&](uint32_t e, float l) {
            if (logit_bias) l = __fadd_rn(l, logit_bias[e]);
            if (lane == 0) scores[e] = l;
        };
        uint32_t ea = ld_e;
        if (ea != 0xFFFFFFFFu) router_logit_load_all<GROUPS>(W + (size_t)ea * d, S + (size_t)ea * GROUPS, B + (size_t)ea * GROUPS, lane, ra);
        while (ea != 0xFFFFFFFFu) {
            const uint32_t eb = pop_candidate(masks);
            if (eb != 0xFFFFFFFFu) router_logit_load_all<GROUPS>(W + (size_t)eb * d, S + (size_t)eb * GROUPS, B + (size_t)eb * GROUPS, lane, rb);
            finish(ea, router_logit_all<GROUPS>(ra, xf, lane));
            if (eb == 0xFFFFFFFFu) break;
            ea = pop_candidate(masks);
            if (ea != 0xFFFFFFFFu) router_logit_load_all<GROUPS>(W + (size_t)ea * d, S + (size_t)ea * GROUPS, B + (size_t)ea * GROUPS, lane, ra);
            finish(eb, router_logit_all<GROUPS>(rb, xf, lane));
        }
    } else if (ld_e != 0xFFFFFFFFu) {
        uint32_t wa[kLogitChunk], wb[kLogitChunk], sba, sbb = 0u;          // two chunk buffers, used in turns
        uint32_t cur_e = ld_e, cur_g = 0u;
        float acc = 0.0f;
        auto advance = [&]() {
            ld_g += kLogitChunk;
            if (ld_g >= groups) { ld_e = pop_candidate(masks); ld_g = 0u; }
        };
        // multiplies the chunk in (wc, sbc) after requesting the next one into (wn, sbn); true when it was the last one
        auto step = [&](const uint32_t (&wc)[kLogitChunk], uint32_t sbc, uint32_t (&wn)[kLogitChunk], uint32_t& sbn) -> bool {
            const uint32_t nxt_e = ld_e, nxt_g = ld_g;
            if (nxt_e != 0xFFFFFFFFu) {
                router_logit_load(W + (size_t)nxt_e * d, S + (size_t)nxt_e * groups, B + (size_t)nxt_e * groups, nxt_g, groups, lane, wn, sbn);
                advance();
            }
            acc = router_logit_chunk(acc, wc, sbc, xf, cur_g, groups, lane);
            if (cur_g + kLogitChunk >= groups) {
                float l = warp_sum(acc);
                if (logit_bias) l = __fadd_rn(l, logit_bias[cur_e]);
                if (lane == 0) scores[cur_e] = l;
                acc = 0.0f;
            }
            cur_e = nxt_e; cur_g = nxt_g;
            return nxt_e == 0xFFFFFFFFu;
        };
        router_logit_load(W + (size_t)ld_e * d, S + (size_t)ld_e * groups, B + (size_t)ld_e * groups, 0u, groups, lane, wa, sba);
        advance();
        while (true) {
            if (step(wa, sba, wb, sbb)) break;
            if (step(wb, sbb, wa, sba)) break;
        }
    }
    __syncwarp();
    warp_select_topk(scores, num_experts, top_k, per_expert_scale, out_idx + (size_t)row * top_k, out_w + (size_t)row * top_k, lane);
}

}  // namespace tf
