// Warp-cooperative dot products of one affine-quantised row with an activation
// vector staged in shared memory. All variants use the group factoring of the
// reference kernels (Metal/Quant/dequant_int4.metal:14-19):
//     sum_k (q_k * s + b) * x_k = s * sum_k q_k x_k + b * sum_k x_k
// with fp32 accumulation. The per-16-element sums of x are precomputed once per
// block (xsum16) so no lane re-adds x.
#pragma once

#include "tf_common.cuh"

namespace tf {

// Stage n fp16 (or bf16) activations into shared memory as fp16-or-bf16 bits
// widened lazily, plus fp32 sums of every 16 consecutive elements.
// xs: n floats are NOT stored; we keep 16-bit storage to halve shared traffic.
template <bool X_BF16>
__device__ __forceinline__ float x_to_float(uint16_t b) {
    if constexpr (X_BF16) return bf16_bits_to_float(b);
    else return f16_bits_to_float(b);
}

template <bool X_BF16>
__device__ __forceinline__ void stage_x(const uint16_t* __restrict__ x, uint16_t* xs, float* xsum16, int n) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) xs[i] = x[i];
    __syncthreads();
    for (int c = threadIdx.x; c < (n >> 4); c += blockDim.x) {
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) s += x_to_float<X_BF16>(xs[c * 16 + j]);
        xsum16[c] = s;
    }
    __syncthreads();
}

__host__ __device__ inline size_t stage_x_bytes(int n) {
    // 16-bit x padded to 16 bytes, then one float per 16 elements.
    return ((size_t)n * 2 + 15) / 16 * 16 + (size_t)(n / 16) * 4;
}
__device__ __forceinline__ float* xsum_ptr(uint16_t* xs, int n) {
    return reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xs) + ((size_t)n * 2 + 15) / 16 * 16);
}

// 8 nibbles of one 32-bit word against 8 consecutive activations (4 x 32-bit
// words holding 2 x 16-bit each).
template <bool X_BF16>
__device__ __forceinline__ float dot8_nibbles(uint32_t w, uint32_t x01, uint32_t x23, uint32_t x45, uint32_t x67, float dot) {
    dot = fmaf((float)(w & 0xFu), x_to_float<X_BF16>((uint16_t)(x01 & 0xFFFFu)), dot);
    dot = fmaf((float)((w >> 4) & 0xFu), x_to_float<X_BF16>((uint16_t)(x01 >> 16)), dot);
    dot = fmaf((float)((w >> 8) & 0xFu), x_to_float<X_BF16>((uint16_t)(x23 & 0xFFFFu)), dot);
    dot = fmaf((float)((w >> 12) & 0xFu), x_to_float<X_BF16>((uint16_t)(x23 >> 16)), dot);
    dot = fmaf((float)((w >> 16) & 0xFu), x_to_float<X_BF16>((uint16_t)(x45 & 0xFFFFu)), dot);
    dot = fmaf((float)((w >> 20) & 0xFu), x_to_float<X_BF16>((uint16_t)(x45 >> 16)), dot);
    dot = fmaf((float)((w >> 24) & 0xFu), x_to_float<X_BF16>((uint16_t)(x67 & 0xFFFFu)), dot);
    dot = fmaf((float)(w >> 28), x_to_float<X_BF16>((uint16_t)(x67 >> 16)), dot);
    return dot;
}

// int4 row, weights 16-byte aligned, n % 64 == 0. Lane c handles the 16-byte
// chunk c, c+32, ... (32 elements = half a group). Returns the lane partial.
template <bool SB_FP16, bool X_BF16>
__device__ __forceinline__ float int4_row_partial_a16(const uint8_t* __restrict__ Wrow,
                                                      const uint16_t* __restrict__ s_row,
                                                      const uint16_t* __restrict__ b_row,
                                                      const uint16_t* xs, const float* xsum16, int n, int lane) {
    float acc = 0.0f;
    const int chunks = n >> 5;
#pragma unroll 2
    for (int c = lane; c < chunks; c += kWarp) {
        const uint4 w = ldg_nc_u4(Wrow + (size_t)c * 16);
        const float s = sb_to_float<SB_FP16>(s_row[c >> 1]);
        const float b = sb_to_float<SB_FP16>(b_row[c >> 1]);
        const uint4* xp = reinterpret_cast<const uint4*>(xs + c * 32);
        const uint4 xa = xp[0], xb = xp[1], xc = xp[2], xd = xp[3];
        float dot = 0.0f;
        dot = dot8_nibbles<X_BF16>(w.x, xa.x, xa.y, xa.z, xa.w, dot);
        dot = dot8_nibbles<X_BF16>(w.y, xb.x, xb.y, xb.z, xb.w, dot);
        dot = dot8_nibbles<X_BF16>(w.z, xc.x, xc.y, xc.z, xc.w, dot);
        dot = dot8_nibbles<X_BF16>(w.w, xd.x, xd.y, xd.z, xd.w, dot);
        acc = fmaf(s, dot, acc);
        acc = fmaf(b, xsum16[2 * c] + xsum16[2 * c + 1], acc);
    }
    return acc;
}

// Two int4 rows (gate and up) that share the activation loads.
template <bool X_BF16>
__device__ __forceinline__ float2 int4_row2_partial_a16(const uint8_t* __restrict__ Wg, const uint16_t* __restrict__ sg,
                                                        const uint16_t* __restrict__ bg,
                                                        const uint8_t* __restrict__ Wu, const uint16_t* __restrict__ su,
                                                        const uint16_t* __restrict__ bu,
                                                        const uint16_t* xs, const float* xsum16, int n, int lane) {
    float ga = 0.0f, ua = 0.0f;
    const int chunks = n >> 5;
#pragma unroll 2
    for (int c = lane; c < chunks; c += kWarp) {
        const uint4 wg = ldg_nc_u4(Wg + (size_t)c * 16);
        const uint4 wu = ldg_nc_u4(Wu + (size_t)c * 16);
        const int g = c >> 1;
        const float gs = bf16_bits_to_float(sg[g]), gb = bf16_bits_to_float(bg[g]);
        const float us = bf16_bits_to_float(su[g]), ub = bf16_bits_to_float(bu[g]);
        const uint4* xp = reinterpret_cast<const uint4*>(xs + c * 32);
        const uint4 xa = xp[0], xb = xp[1], xc = xp[2], xd = xp[3];
        float gd = 0.0f, ud = 0.0f;
        gd = dot8_nibbles<X_BF16>(wg.x, xa.x, xa.y, xa.z, xa.w, gd);
        ud = dot8_nibbles<X_BF16>(wu.x, xa.x, xa.y, xa.z, xa.w, ud);
        gd = dot8_nibbles<X_BF16>(wg.y, xb.x, xb.y, xb.z, xb.w, gd);
        ud = dot8_nibbles<X_BF16>(wu.y, xb.x, xb.y, xb.z, xb.w, ud);
        gd = dot8_nibbles<X_BF16>(wg.z, xc.x, xc.y, xc.z, xc.w, gd);
        ud = dot8_nibbles<X_BF16>(wu.z, xc.x, xc.y, xc.z, xc.w, ud);
        gd = dot8_nibbles<X_BF16>(wg.w, xd.x, xd.y, xd.z, xd.w, gd);
        ud = dot8_nibbles<X_BF16>(wu.w, xd.x, xd.y, xd.z, xd.w, ud);
        const float xsum = xsum16[2 * c] + xsum16[2 * c + 1];
        ga = fmaf(gs, gd, ga);
        ga = fmaf(gb, xsum, ga);
        ua = fmaf(us, ud, ua);
        ua = fmaf(ub, xsum, ua);
    }
    return make_float2(ga, ua);
}

// int4 row whose packed bytes are only 2-byte aligned (the resident-layout case
// the reference tests at a +2 byte offset, Tests/.../DequantInt4GEMVTests.swift:114-121).
// Lane handles 4 bytes (8 elements) per step, read as two 16-bit loads.
template <bool SB_FP16, bool X_BF16>
__device__ __forceinline__ float int4_row_partial_a2(const uint8_t* __restrict__ Wrow,
                                                     const uint16_t* __restrict__ s_row,
                                                     const uint16_t* __restrict__ b_row,
                                                     const uint16_t* xs, int n, int lane) {
    float acc = 0.0f;
    const int steps = n >> 3;
    for (int c = lane; c < steps; c += kWarp) {
        const uint16_t* wp = reinterpret_cast<const uint16_t*>(Wrow + (size_t)c * 4);
        const uint32_t w = (uint32_t)wp[0] | ((uint32_t)wp[1] << 16);
        const int g = c >> 3;
        const float s = sb_to_float<SB_FP16>(s_row[g]);
        const float b = sb_to_float<SB_FP16>(b_row[g]);
        const uint4 xv = *reinterpret_cast<const uint4*>(xs + c * 8);
        const float dot = dot8_nibbles<X_BF16>(w, xv.x, xv.y, xv.z, xv.w, 0.0f);
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += x_to_float<X_BF16>(xs[c * 8 + j]);
        acc = fmaf(s, dot, acc);
        acc = fmaf(b, sum, acc);
    }
    return acc;
}

// int8 row, generic alignment: lane handles 4 bytes per step (byte loads when
// the row is not 4-byte aligned).
template <bool SB_FP16, bool X_BF16>
__device__ __forceinline__ float int8_row_partial(const uint8_t* __restrict__ Wrow,
                                                  const uint16_t* __restrict__ s_row,
                                                  const uint16_t* __restrict__ b_row,
                                                  const uint16_t* xs, int n, int lane, bool a4) {
    float acc = 0.0f;
    const int steps = n >> 2;
    for (int c = lane; c < steps; c += kWarp) {
        uint32_t w;
        if (a4) {
            w = __ldg(reinterpret_cast<const uint32_t*>(Wrow + (size_t)c * 4));
        } else {
            const uint8_t* p = Wrow + (size_t)c * 4;
            w = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
        }
        const int g = c >> 4;
        const float s = sb_to_float<SB_FP16>(s_row[g]);
        const float b = sb_to_float<SB_FP16>(b_row[g]);
        const float x0 = x_to_float<X_BF16>(xs[c * 4 + 0]);
        const float x1 = x_to_float<X_BF16>(xs[c * 4 + 1]);
        const float x2 = x_to_float<X_BF16>(xs[c * 4 + 2]);
        const float x3 = x_to_float<X_BF16>(xs[c * 4 + 3]);
        float dot = (float)(w & 0xFFu) * x0;
        dot = fmaf((float)((w >> 8) & 0xFFu), x1, dot);
        dot = fmaf((float)((w >> 16) & 0xFFu), x2, dot);
        dot = fmaf((float)(w >> 24), x3, dot);
        acc = fmaf(s, dot, acc);
        acc = fmaf(b, (x0 + x1) + (x2 + x3), acc);
    }
    return acc;
}

}  // namespace tf
