// Int4 QMM for the shapes and alignments the tensor-core kernel does not take.
//
// MPPPrefillInt4QMM.encode (Kernels/TensorCore/MPPPrefillInt4QMM.swift:34-55) accepts any M and N, any byte
// offset of the packed plane and any even offset of the scale, bias and activation planes; the tcgen05 kernel
// wants N % 8 == 0 and 16-byte aligned planes (TMA and bulk copies). This kernel closes that gap on the CUDA
// cores so that tf_int4_qmm is total over the reference's domain:
//   Y[t, r] = half( sum_k fma(q[r,k], s[r,k/64], b[r,k/64]) * X[t,k] ),  fp32 accumulation
// (the arithmetic of the reference's scalar QMM, Metal/Prefill/prefill.metal:672-709, with the K loop split over
// the lanes of a warp). One warp owns one weight row and kQgTokens token rows; in step j lane l holds byte
// 32 j + l of the row, i.e. columns 64 j + 2 l and + 1 of group j, so scale and bias are warp-uniform per step.
#include "tf_common.cuh"

namespace tf {

constexpr int kQgWarps = 4;
constexpr int kQgTokens = 4;

template <bool SB_FP16>
__global__ void __launch_bounds__(kQgWarps * kWarp)
qmm_generic_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ S, const uint16_t* __restrict__ B,
                   const uint16_t* __restrict__ X, uint16_t* __restrict__ Y, uint32_t m, uint32_t n, uint32_t k) {
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t r = blockIdx.x * kQgWarps + warp;
    const uint32_t t0 = blockIdx.y * kQgTokens;
    if (r >= n) return;
    const uint32_t groups = k / kGroup;
    const uint8_t* wrow = W + (size_t)r * (k / 2);
    const uint16_t* srow = S + (size_t)r * groups;
    const uint16_t* brow = B + (size_t)r * groups;
    float acc[kQgTokens];
#pragma unroll
    for (int t = 0; t < kQgTokens; ++t) acc[t] = 0.0f;
    for (uint32_t j = 0; j < groups; ++j) {
        const uint32_t byte = wrow[j * 32 + lane];
        const float s = sb_to_float<SB_FP16>(srow[j]), b = sb_to_float<SB_FP16>(brow[j]);
        const float w0 = fmaf((float)(byte & 0xFu), s, b), w1 = fmaf((float)(byte >> 4), s, b);
        const uint32_t c = j * kGroup + 2 * lane;
#pragma unroll
        for (int t = 0; t < kQgTokens; ++t) {
            if (t0 + t < m) {
                const uint16_t* xr = X + (size_t)(t0 + t) * k + c;
                acc[t] = fmaf(w0, f16_bits_to_float(xr[0]), acc[t]);
                acc[t] = fmaf(w1, f16_bits_to_float(xr[1]), acc[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < kQgTokens; ++t) {
        const float v = warp_sum(acc[t]);
        if (lane == 0 && t0 + t < m) Y[(size_t)(t0 + t) * n + r] = __half_as_ushort(__float2half_rn(v));
    }
}

tf_status launch_qmm_generic(tf_context* ctx, void* stream, const uint8_t* W, const uint16_t* S, const uint16_t* B,
                             const uint16_t* X, uint16_t* Y, uint32_t m, uint32_t n, uint32_t k, const char* name) {
    dim3 grid((n + kQgWarps - 1) / kQgWarps, (m + kQgTokens - 1) / kQgTokens);
    TF_REQUIRE(ctx, grid.y <= 65535u, TF_ERR_UNSUPPORTED, "%s: M=%u is too large for the unaligned path", name, m);
    qmm_generic_kernel<false><<<grid, kQgWarps * kWarp, 0, static_cast<cudaStream_t>(stream)>>>(W, S, B, X, Y, m, n, k);
    return check_launch(ctx, name);
}

}  // namespace tf
