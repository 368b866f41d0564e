// RMSNorm and the Gemma-4 layer tail, one block per row.
// Replaces rmsnorm_bf16w / rmsnorm_no_scale (Metal/Primitives/rmsnorm.metal:32-93,153-175),
// their block forms (Metal/Prefill/prefill.metal:54-111), fused_post_attn_setup /
// prefill_post_attn_setup_block (Metal/Fusions/fused.metal:190-269; prefill.metal:178-254) and fused_layer_tail /
// prefill_layer_tail_block (Metal/Fusions/fused.metal:271-375; prefill.metal:255-334).
#include "tf_common.cuh"

namespace tf {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    __syncthreads();                       // red may still be read from a previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < (int)(blockDim.x / kWarp)) ? red[lane] : 0.0f;
    t = warp_sum(t);
    return t;                              // every thread holds the total
}

template <bool BF16>
__device__ __forceinline__ float act_to_float(uint16_t b) {
    if constexpr (BF16) return bf16_bits_to_float(b);
    else return f16_bits_to_float(b);
}
template <bool BF16>
__device__ __forceinline__ uint16_t float_to_act(float v) {
    if constexpr (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    else return __half_as_ushort(__float2half_rn(v));
}

template <bool BF16>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ weight, uint16_t* __restrict__ y,
               uint32_t d, uint32_t stride, float eps) {
    __shared__ float red[kNormThreads / kWarp];
    const uint16_t* xr = x + (size_t)blockIdx.x * stride;
    uint16_t* yr = y + (size_t)blockIdx.x * stride;
    float acc = 0.0f;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = act_to_float<BF16>(xr[i]);
        acc = fmaf(v, v, acc);
    }
    const float total = block_sum(acc, red);
    const float inv = rsqrtf(total / (float)d + eps);
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        float v = act_to_float<BF16>(xr[i]) * inv;
        if (weight) v *= bf16_bits_to_float(weight[i]);
        yr[i] = float_to_act<BF16>(v);
    }
}

// fp16 only, with the reference's rounding points:
//   tmp  = half(h2 * inv(h2) * w2); h12 = half(h1 + tmp)
//   tmp2 = half(h12 * inv(h12) * w); hidden = half(half(hidden + tmp2) * half(layer_scalar))
__global__ void __launch_bounds__(kNormThreads)
layer_tail_kernel(const uint16_t* __restrict__ h2, const uint16_t* __restrict__ h1, uint16_t* __restrict__ hidden,
                  const uint16_t* __restrict__ w2, const uint16_t* __restrict__ w,
                  uint32_t d, uint32_t stride, float eps, float layer_scalar) {
    extern __shared__ __align__(16) uint8_t smem[];
    __half* h12 = reinterpret_cast<__half*>(smem);
    __shared__ float red[kNormThreads / kWarp];
    const uint16_t* h2r = h2 + (size_t)blockIdx.x * stride;
    const uint16_t* h1r = h1 + (size_t)blockIdx.x * stride;
    uint16_t* hr = hidden + (size_t)blockIdx.x * stride;
    float acc = 0.0f;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = f16_bits_to_float(h2r[i]);
        acc = fmaf(v, v, acc);
    }
    const float inv_h2 = rsqrtf(block_sum(acc, red) / (float)d + eps);
    acc = 0.0f;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        const __half tmp = __float2half_rn(f16_bits_to_float(h2r[i]) * inv_h2 * bf16_bits_to_float(w2[i]));
        const __half s = __float2half_rn(f16_bits_to_float(h1r[i]) + __half2float(tmp));
        h12[i] = s;
        const float v = __half2float(s);
        acc = fmaf(v, v, acc);
    }
    const float inv_h12 = rsqrtf(block_sum(acc, red) / (float)d + eps);
    const float hs = __half2float(__float2half_rn(layer_scalar));
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        const __half tmp = __float2half_rn(__half2float(h12[i]) * inv_h12 * bf16_bits_to_float(w[i]));
        const __half hsum = __float2half_rn(f16_bits_to_float(hr[i]) + __half2float(tmp));
        hr[i] = __half_as_ushort(__float2half_rn(__half2float(hsum) * hs));
    }
}

// The three-way norm in front of the feed-forward block, fp16 with the reference's rounding points:
//   a      = half(attn * inv(attn) * w_post_attn);  hidden = half(hidden + a)            (written back)
//   h      = hidden * inv(hidden)
//   dense  = half(h * w_pre_ffn);  routed = half(h * w_pre_ffn2);  router = half(h)
// Sums of squares use the thread striding and reduction tree of rmsnorm_kernel, so the outputs equal the chain
// rmsnorm -> add -> rmsnorm x 3 bit for bit.
__global__ void __launch_bounds__(kNormThreads)
post_attn_setup_kernel(uint16_t* __restrict__ hidden, uint32_t hidden_stride, const uint16_t* __restrict__ attn,
                       uint32_t attn_stride, uint16_t* __restrict__ dense_x, uint32_t dense_stride,
                       uint16_t* __restrict__ routed_x, uint32_t routed_stride, uint16_t* __restrict__ router_x,
                       uint32_t router_stride, const uint16_t* __restrict__ w_post_attn,
                       const uint16_t* __restrict__ w_pre_ffn, const uint16_t* __restrict__ w_pre_ffn2,
                       uint32_t d, float eps) {
    extern __shared__ __align__(16) uint8_t smem[];
    __half* hid = reinterpret_cast<__half*>(smem);
    __shared__ float red[kNormThreads / kWarp];
    uint16_t* hr = hidden + (size_t)blockIdx.x * hidden_stride;
    const uint16_t* ar = attn + (size_t)blockIdx.x * attn_stride;
    float acc = 0.0f;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = f16_bits_to_float(ar[i]);
        acc = fmaf(v, v, acc);
    }
    const float attn_inv = rsqrtf(block_sum(acc, red) / (float)d + eps);
    acc = 0.0f;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        const __half a = __float2half_rn(f16_bits_to_float(ar[i]) * attn_inv * bf16_bits_to_float(w_post_attn[i]));
        const __half h = __float2half_rn(f16_bits_to_float(hr[i]) + __half2float(a));
        hid[i] = h;
        hr[i] = __half_as_ushort(h);
        const float hf = __half2float(h);
        acc = fmaf(hf, hf, acc);
    }
    const float hidden_inv = rsqrtf(block_sum(acc, red) / (float)d + eps);
    uint16_t* dr = dense_x + (size_t)blockIdx.x * dense_stride;
    uint16_t* rr = routed_x + (size_t)blockIdx.x * routed_stride;
    uint16_t* qr = router_x + (size_t)blockIdx.x * router_stride;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        const float h = __half2float(hid[i]) * hidden_inv;
        dr[i] = __half_as_ushort(__float2half_rn(h * bf16_bits_to_float(w_pre_ffn[i])));
        rr[i] = __half_as_ushort(__float2half_rn(h * bf16_bits_to_float(w_pre_ffn2[i])));
        qr[i] = __half_as_ushort(__float2half_rn(h));
    }
}

}  // namespace tf

extern "C" {

tf_status tf_post_attn_setup(tf_context* ctx, void* stream, void* hidden, uint32_t hidden_stride_elements,
                             const void* attn, uint32_t attn_stride_elements, void* dense_x, uint32_t dense_stride_elements,
                             void* routed_x, uint32_t routed_stride_elements, void* router_x, uint32_t router_stride_elements,
                             const void* w_post_attn_bf16, const void* w_pre_ffn_bf16, const void* w_pre_ffn2_bf16,
                             uint32_t rows, uint32_t d, float eps) {
    const char* name = "tf_post_attn_setup";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, hidden && attn && dense_x && routed_x && router_x && w_post_attn_bf16 && w_pre_ffn_bf16 && w_pre_ffn2_bf16,
               TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, d > 0 && hidden_stride_elements >= d && attn_stride_elements >= d && dense_stride_elements >= d &&
                        routed_stride_elements >= d && router_stride_elements >= d,
               TF_ERR_INVALID_ARGUMENT, "%s: a row stride is smaller than D", name);
    // FusedPostAttentionSetup.swift:40 requires d <= 4096 (two fp16 rows in threadgroup memory); one row is kept here
    TF_REQUIRE(ctx, (size_t)d * 2 <= 96 * 1024, TF_ERR_UNSUPPORTED, "%s: D too large", name);
    TF_REQUIRE(ctx, tf::aligned(hidden, 2) && tf::aligned(attn, 2) && tf::aligned(dense_x, 2) && tf::aligned(routed_x, 2) &&
                        tf::aligned(router_x, 2), TF_ERR_ALIGNMENT, "%s: rows must be 2-byte aligned", name);
    if (rows == 0) return TF_OK;
    const size_t smem = (size_t)d * 2;
    if (smem > 48 * 1024)
        TF_CUDA(ctx, cudaFuncSetAttribute(tf::post_attn_setup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    tf::post_attn_setup_kernel<<<rows, tf::kNormThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint16_t*>(hidden), hidden_stride_elements, static_cast<const uint16_t*>(attn), attn_stride_elements,
        static_cast<uint16_t*>(dense_x), dense_stride_elements, static_cast<uint16_t*>(routed_x), routed_stride_elements,
        static_cast<uint16_t*>(router_x), router_stride_elements, static_cast<const uint16_t*>(w_post_attn_bf16),
        static_cast<const uint16_t*>(w_pre_ffn_bf16), static_cast<const uint16_t*>(w_pre_ffn2_bf16), d, eps);
    return tf::check_launch(ctx, name);
}

tf_status tf_rmsnorm(tf_context* ctx, void* stream, const void* x, uint64_t x_off, const void* weight_bf16,
                     uint64_t weight_off, void* y, uint64_t y_off, uint32_t rows, uint32_t d,
                     uint32_t stride_elements, float eps, tf_dtype act_dtype) {
    const char* name = "tf_rmsnorm";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, x && y, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, d > 0 && stride_elements >= d, TF_ERR_INVALID_ARGUMENT, "%s: stride is too small", name);
    if (rows == 0) return TF_OK;
    auto xp = reinterpret_cast<const uint16_t*>(tf::byte_ptr(x, x_off));
    auto yp = reinterpret_cast<uint16_t*>(tf::byte_ptr(y, y_off));
    auto wp = weight_bf16 ? reinterpret_cast<const uint16_t*>(tf::byte_ptr(weight_bf16, weight_off)) : nullptr;
    TF_REQUIRE(ctx, tf::aligned(xp, 2) && tf::aligned(yp, 2) && tf::aligned(wp, 2), TF_ERR_ALIGNMENT,
               "%s: planes must be 2-byte aligned", name);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (act_dtype == TF_BF16)
        tf::rmsnorm_kernel<true><<<rows, tf::kNormThreads, 0, st>>>(xp, wp, yp, d, stride_elements, eps);
    else
        tf::rmsnorm_kernel<false><<<rows, tf::kNormThreads, 0, st>>>(xp, wp, yp, d, stride_elements, eps);
    return tf::check_launch(ctx, name);
}

tf_status tf_layer_tail(tf_context* ctx, void* stream, const void* h2, const void* h1, void* hidden,
                        const void* w_postffn2_bf16, const void* w_postffn_bf16, uint32_t rows, uint32_t d,
                        uint32_t stride_elements, float eps, float layer_scalar) {
    const char* name = "tf_layer_tail";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, h2 && h1 && hidden && w_postffn2_bf16 && w_postffn_bf16, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, d > 0 && stride_elements >= d, TF_ERR_INVALID_ARGUMENT, "%s: stride is too small", name);
    TF_REQUIRE(ctx, (size_t)d * 2 <= 96 * 1024, TF_ERR_UNSUPPORTED, "%s: D too large", name);
    if (rows == 0) return TF_OK;
    const size_t smem = (size_t)d * 2;
    if (smem > 48 * 1024)
        TF_CUDA(ctx, cudaFuncSetAttribute(tf::layer_tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    tf::layer_tail_kernel<<<rows, tf::kNormThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(h2), static_cast<const uint16_t*>(h1), static_cast<uint16_t*>(hidden),
        static_cast<const uint16_t*>(w_postffn2_bf16), static_cast<const uint16_t*>(w_postffn_bf16), d,
        stride_elements, eps, layer_scalar);
    return tf::check_launch(ctx, name);
}

}  // extern "C"
