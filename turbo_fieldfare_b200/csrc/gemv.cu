// Stand-alone affine GEMVs: y[m] = deq(W[m,n]) . x[n], fp16 in/out, fp32 accumulate.
// Replaces dequant_int4_gemv_simd / dequant_int8_gemv_simd
// (Metal/Quant/dequant_int4.metal:93-191, Metal/Quant/dequant_int8.metal:57-97).
//
// One warp per row, rows strided over a grid sized to the SM count; x is staged
// once per block in shared memory; packed weights stream through 128-bit
// non-allocating loads when the plane is 16-byte aligned, 16-bit loads otherwise.
#include "rowdot.cuh"

namespace tf {

// gemv_mma.cu: the tensor-core streaming kernel for large, aligned matrices
bool gemv_mma_eligible(const void* W, const void* S, const void* B, const void* x, uint32_t m, uint32_t n);
tf_status launch_gemv_mma(tf_context* ctx, void* stream, const uint8_t* W, const uint16_t* S, const uint16_t* B,
                          const uint16_t* x, void* y, bool out_f32, uint32_t m, uint32_t n, bool sb_fp16, const char* name);
tf_status launch_gemv_mma_batched(tf_context* ctx, void* stream, const uint8_t* W, const uint16_t* S, const uint16_t* B,
                                  uint64_t plane_stride, const uint16_t* x, uint32_t x_stride, uint16_t* y, uint32_t y_stride,
                                  uint32_t m, uint32_t n, uint32_t count, bool sb_fp16, const char* name);

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / kWarp;

// OUT_F32: the row sums are stored as fp32 (the greedy LM head compares unrounded logits).
template <int BITS, bool SB_FP16, bool A16, bool OUT_F32>
__global__ void __launch_bounds__(kGemvThreads)
affine_gemv_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ S, const uint16_t* __restrict__ B,
                   const uint16_t* __restrict__ x, void* __restrict__ y, uint32_t m, uint32_t n, bool a4) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint16_t* xs = reinterpret_cast<uint16_t*>(smem);
    float* xsum16 = xsum_ptr(xs, (int)n);
    stage_x<false>(x, xs, xsum16, (int)n);

    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t groups = n / kGroup;
    const size_t row_bytes = BITS == 4 ? n / 2 : n;
    for (uint32_t row = blockIdx.x * kGemvWarps + warp; row < m; row += gridDim.x * kGemvWarps) {
        const uint8_t* Wrow = W + (size_t)row * row_bytes;
        const uint16_t* s_row = S + (size_t)row * groups;
        const uint16_t* b_row = B + (size_t)row * groups;
        float acc;
        if constexpr (BITS == 4) {
            if constexpr (A16) acc = int4_row_partial_a16<SB_FP16, false>(Wrow, s_row, b_row, xs, xsum16, (int)n, lane);
            else acc = int4_row_partial_a2<SB_FP16, false>(Wrow, s_row, b_row, xs, (int)n, lane);
        } else {
            acc = int8_row_partial<SB_FP16, false>(Wrow, s_row, b_row, xs, (int)n, lane, a4);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            if constexpr (OUT_F32) static_cast<float*>(y)[row] = acc;
            else static_cast<uint16_t*>(y)[row] = __half_as_ushort(__float2half_rn(acc));
        }
    }
}

// Fused gate/up projection of the 8-bit shared expert: one warp per intermediate row computes both dot products over
// the activations staged once per block and stores act = half(gelu(half(gate)) * half(up))
// (shared_int8_gate_up_act_simd, Metal/Quant/dequant_int8.metal:98-154). grid.y walks token rows.
__global__ void __launch_bounds__(kGemvThreads)
shared_int8_gate_up_act_kernel(const uint8_t* __restrict__ Wg, const uint16_t* __restrict__ Sg, const uint16_t* __restrict__ Bg,
                               const uint8_t* __restrict__ Wu, const uint16_t* __restrict__ Su, const uint16_t* __restrict__ Bu,
                               const uint16_t* __restrict__ x, uint32_t x_stride, uint16_t* __restrict__ act, uint32_t act_stride,
                               uint32_t m, uint32_t n, bool a4) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint16_t* xs = reinterpret_cast<uint16_t*>(smem);
    float* xsum16 = xsum_ptr(xs, (int)n);
    stage_x<false>(x + (size_t)blockIdx.y * x_stride, xs, xsum16, (int)n);
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t groups = n / kGroup;
    for (uint32_t row = blockIdx.x * kGemvWarps + warp; row < m; row += gridDim.x * kGemvWarps) {
        float g = int8_row_partial<false, false>(Wg + (size_t)row * n, Sg + (size_t)row * groups, Bg + (size_t)row * groups, xs, (int)n, lane, a4);
        float u = int8_row_partial<false, false>(Wu + (size_t)row * n, Su + (size_t)row * groups, Bu + (size_t)row * groups, xs, (int)n, lane, a4);
        g = warp_sum(g);
        u = warp_sum(u);
        if (lane == 0) {
            const float gh = __half2float(__float2half_rn(g)), uh = __half2float(__float2half_rn(u));
            act[(size_t)blockIdx.y * act_stride + row] = __half_as_ushort(__float2half_rn(gelu_tanh(gh) * uh));
        }
    }
}

// y[row t] = deq8(W) . x[row t] for a block of token rows (grid.y), the down projection of the 8-bit shared expert.
__global__ void __launch_bounds__(kGemvThreads)
int8_gemv_rows_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ S, const uint16_t* __restrict__ B,
                      const uint16_t* __restrict__ x, uint32_t x_stride, uint16_t* __restrict__ y, uint32_t y_stride,
                      uint32_t m, uint32_t n, bool a4) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint16_t* xs = reinterpret_cast<uint16_t*>(smem);
    float* xsum16 = xsum_ptr(xs, (int)n);
    stage_x<false>(x + (size_t)blockIdx.y * x_stride, xs, xsum16, (int)n);
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t groups = n / kGroup;
    for (uint32_t row = blockIdx.x * kGemvWarps + warp; row < m; row += gridDim.x * kGemvWarps) {
        float acc = int8_row_partial<false, false>(W + (size_t)row * n, S + (size_t)row * groups, B + (size_t)row * groups, xs, (int)n, lane, a4);
        acc = warp_sum(acc);
        if (lane == 0) y[(size_t)blockIdx.y * y_stride + row] = __half_as_ushort(__float2half_rn(acc));
    }
}

template <int BITS, bool OUT_F32 = false>
static tf_status launch_gemv(tf_context* ctx, void* stream, const void* weights, uint64_t weights_off,
                             const void* scales, uint64_t scales_off, const void* biases, uint64_t biases_off,
                             const void* x, uint64_t x_off, void* y, uint64_t y_off, uint32_t m, uint32_t n,
                             tf_dtype sb_dtype, const char* name) {
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, weights && scales && biases && x && y, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, m > 0 && n > 0, TF_ERR_INVALID_ARGUMENT, "%s: m and n must be positive", name);
    TF_REQUIRE(ctx, n % kGroup == 0, TF_ERR_INVALID_ARGUMENT, "%s: N=%u must be a multiple of %d", name, n, kGroup);
    TF_REQUIRE(ctx, sb_dtype == TF_BF16 || sb_dtype == TF_FP16, TF_ERR_INVALID_ARGUMENT, "%s: bad sb_dtype", name);
    const uint8_t* W = byte_ptr(weights, weights_off);
    const uint8_t* S = byte_ptr(scales, scales_off);
    const uint8_t* Bp = byte_ptr(biases, biases_off);
    const uint8_t* xp = byte_ptr(x, x_off);
    uint8_t* yp = byte_ptr(y, y_off);
    if (BITS == 4)
        TF_REQUIRE(ctx, aligned(W, 2), TF_ERR_ALIGNMENT, "%s: weightsOffset must be even", name);
    TF_REQUIRE(ctx, aligned(S, 2) && aligned(Bp, 2) && aligned(xp, 2) && aligned(yp, OUT_F32 ? 4 : 2), TF_ERR_ALIGNMENT,
               "%s: scale/bias/x/y planes must be 2-byte aligned", name);
    if (BITS == 4 && gemv_mma_eligible(W, S, Bp, xp, m, n))
        return launch_gemv_mma(ctx, stream, W, reinterpret_cast<const uint16_t*>(S), reinterpret_cast<const uint16_t*>(Bp),
                               reinterpret_cast<const uint16_t*>(xp), yp, OUT_F32, m, n, sb_dtype == TF_FP16, name);
    const size_t smem = stage_x_bytes((int)n);
    TF_REQUIRE(ctx, smem <= 96 * 1024, TF_ERR_UNSUPPORTED, "%s: N=%u too large for the staged-x kernel", name, n);

    const size_t row_bytes = BITS == 4 ? n / 2 : n;
    const bool a16 = aligned(W, 16) && row_bytes % 16 == 0;
    const bool a4 = aligned(W, 4) && row_bytes % 4 == 0;
    const uint32_t blocks_needed = (m + kGemvWarps - 1) / kGemvWarps;
    const uint32_t grid = blocks_needed < (uint32_t)ctx->sm_count * 8u ? blocks_needed : (uint32_t)ctx->sm_count * 8u;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool fp16 = sb_dtype == TF_FP16;

#define TF_GEMV_LAUNCH(SB, A)                                                                          \
    do {                                                                                               \
        auto k = affine_gemv_kernel<BITS, SB, A, OUT_F32>;                                                    \
        if (smem > 48 * 1024) TF_CUDA(ctx, cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        k<<<grid, kGemvThreads, smem, st>>>(W, reinterpret_cast<const uint16_t*>(S),                   \
                                            reinterpret_cast<const uint16_t*>(Bp),                      \
                                            reinterpret_cast<const uint16_t*>(xp),                      \
                                            static_cast<void*>(yp), m, n, a4);                          \
    } while (0)

    if (BITS == 4 && a16) {
        if (fp16) TF_GEMV_LAUNCH(true, true); else TF_GEMV_LAUNCH(false, true);
    } else {
        if (fp16) TF_GEMV_LAUNCH(true, false); else TF_GEMV_LAUNCH(false, false);
    }
#undef TF_GEMV_LAUNCH
    return check_launch(ctx, name);
}

// ---------------------------------------------------------------------------
// Greedy LM head: argmax over the finite fp32 logits, ties to the lowest row
// ---------------------------------------------------------------------------
// A finite float as an unsigned key that orders like the float (every finite value maps above zero).
__device__ __forceinline__ uint32_t ordered_key(float v) {
    if (v == 0.0f) v = 0.0f;                        // -0 and +0 compare equal in the reference's reduction
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

constexpr int kArgmaxThreads = 256;

// best = max over rows of (ordered logit << 32 | ~row): the larger logit wins, then the lower row.
__global__ void __launch_bounds__(kArgmaxThreads)
lm_head_argmax_kernel(const float* __restrict__ logits, uint32_t vocab, unsigned long long* __restrict__ best) {
    unsigned long long mine = 0ull;                 // 0 = no finite candidate
    for (uint32_t r = blockIdx.x * blockDim.x + threadIdx.x; r < vocab; r += gridDim.x * blockDim.x) {
        const float z = logits[r];
        if (isfinite(z)) {
            const unsigned long long k = ((unsigned long long)ordered_key(z) << 32) | (unsigned long long)(~r);
            mine = k > mine ? k : mine;
        }
    }
#pragma unroll
    for (int o = kWarp / 2; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(kFullMask, mine, o);
        mine = other > mine ? other : mine;
    }
    __shared__ unsigned long long per_warp[kArgmaxThreads / kWarp];
    if (threadIdx.x % kWarp == 0) per_warp[threadIdx.x / kWarp] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kArgmaxThreads / kWarp; ++w) mine = per_warp[w] > mine ? per_warp[w] : mine;
        if (mine) atomicMax(best, mine);
    }
}

// Decodes the winner (0 when no logit was finite, lm_head_greedy_int4_rows_reduce's fallback) and clears the
// scratch word for the next call.
__global__ void lm_head_finish_kernel(unsigned long long* __restrict__ best, uint32_t* __restrict__ out_token) {
    const unsigned long long k = *best;
    *out_token = k ? ~(uint32_t)(k & 0xFFFFFFFFull) : 0u;
    *best = 0ull;
}

}  // namespace tf

extern "C" {

tf_status tf_lm_head_greedy_int4(tf_context* ctx, void* stream, const void* hidden, uint64_t hidden_off,
                                 const void* norm_weight_bf16, uint64_t norm_off,
                                 const void* weights, uint64_t weights_off, const void* scales, uint64_t scales_off,
                                 const void* biases, uint64_t biases_off, uint32_t* out_token,
                                 uint32_t d, uint32_t vocab, float rms_eps) {
    const char* name = "tf_lm_head_greedy_int4";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, hidden && norm_weight_bf16 && weights && scales && biases && out_token, TF_ERR_INVALID_ARGUMENT,
               "%s: NULL buffer", name);
    TF_REQUIRE(ctx, d > 0 && vocab > 0, TF_ERR_INVALID_ARGUMENT, "%s: d and vocab must be positive", name);
    TF_REQUIRE(ctx, d % tf::kGroup == 0, TF_ERR_INVALID_ARGUMENT, "%s: d must be a multiple of %d", name, tf::kGroup);
    TF_REQUIRE(ctx, weights_off % 2 == 0, TF_ERR_ALIGNMENT, "%s: weightsOffset must be even", name);
    TF_REQUIRE(ctx, tf::aligned(out_token, 4), TF_ERR_ALIGNMENT, "%s: outToken must be 4-byte aligned", name);
    // scratch owned by the context; growing it allocates (and so cannot happen inside a stream capture)
    if (ctx->lm_best == nullptr) {
        TF_CUDA(ctx, cudaMalloc(&ctx->lm_best, sizeof(unsigned long long)));
        TF_CUDA(ctx, cudaMemset(ctx->lm_best, 0, sizeof(unsigned long long)));
    }
    if (d > ctx->lm_x_capacity) {
        if (ctx->lm_x) { TF_CUDA(ctx, cudaFree(ctx->lm_x)); ctx->lm_x = nullptr; ctx->lm_x_capacity = 0; }
        TF_CUDA(ctx, cudaMalloc(&ctx->lm_x, (size_t)d * 2));
        ctx->lm_x_capacity = d;
    }
    if (vocab > ctx->lm_logits_capacity) {
        if (ctx->lm_logits) { TF_CUDA(ctx, cudaFree(ctx->lm_logits)); ctx->lm_logits = nullptr; ctx->lm_logits_capacity = 0; }
        TF_CUDA(ctx, cudaMalloc(&ctx->lm_logits, (size_t)vocab * 4));
        ctx->lm_logits_capacity = vocab;
    }
    tf_status st = tf_rmsnorm(ctx, stream, hidden, hidden_off, norm_weight_bf16, norm_off, ctx->lm_x, 0, 1, d, d, rms_eps, TF_FP16);
    if (st != TF_OK) return st;
    st = tf::launch_gemv<4, true>(ctx, stream, weights, weights_off, scales, scales_off, biases, biases_off, ctx->lm_x, 0,
                                  ctx->lm_logits, 0, vocab, d, TF_BF16, name);
    if (st != TF_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint32_t want = (vocab + tf::kArgmaxThreads - 1) / tf::kArgmaxThreads;
    const uint32_t grid = want < (uint32_t)ctx->sm_count ? want : (uint32_t)ctx->sm_count;
    tf::lm_head_argmax_kernel<<<grid, tf::kArgmaxThreads, 0, s>>>(ctx->lm_logits, vocab, ctx->lm_best);
    st = tf::check_launch(ctx, name);
    if (st != TF_OK) return st;
    tf::lm_head_finish_kernel<<<1, 1, 0, s>>>(ctx->lm_best, out_token);
    return tf::check_launch(ctx, name);
}

tf_status tf_int4_gemv(tf_context* ctx, void* stream, const void* weights, uint64_t weights_off,
                       const void* scales, uint64_t scales_off, const void* biases, uint64_t biases_off,
                       const void* x, uint64_t x_off, void* y, uint64_t y_off,
                       uint32_t m, uint32_t n, tf_dtype sb_dtype) {
    return tf::launch_gemv<4>(ctx, stream, weights, weights_off, scales, scales_off, biases, biases_off,
                              x, x_off, y, y_off, m, n, sb_dtype, "tf_int4_gemv");
}

tf_status tf_int4_gemv_batched(tf_context* ctx, void* stream, const void* weights, uint64_t weights_off,
                               const void* scales, uint64_t scales_off, const void* biases, uint64_t biases_off,
                               uint64_t matrix_stride_bytes, const void* x, uint64_t x_off, uint32_t x_stride_elements,
                               void* y, uint64_t y_off, uint32_t y_stride_elements,
                               uint32_t m, uint32_t n, uint32_t count, tf_dtype sb_dtype) {
    const char* name = "tf_int4_gemv_batched";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, weights && scales && biases && x && y, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, m > 0 && n > 0, TF_ERR_INVALID_ARGUMENT, "%s: m and n must be positive", name);
    TF_REQUIRE(ctx, sb_dtype == TF_BF16 || sb_dtype == TF_FP16, TF_ERR_INVALID_ARGUMENT, "%s: bad sb_dtype", name);
    TF_REQUIRE(ctx, y_stride_elements >= m, TF_ERR_INVALID_ARGUMENT, "%s: the y stride must be at least m", name);
    if (count == 0) return TF_OK;
    const uint8_t* W = tf::byte_ptr(weights, weights_off);
    const uint8_t* S = tf::byte_ptr(scales, scales_off);
    const uint8_t* Bp = tf::byte_ptr(biases, biases_off);
    const uint8_t* xp = tf::byte_ptr(x, x_off);
    uint8_t* yp = tf::byte_ptr(y, y_off);
    const bool streaming = n % 256 == 0 && tf::aligned(W, 16) && tf::aligned(S, 16) && tf::aligned(Bp, 16) && tf::aligned(xp, 16) &&
                           matrix_stride_bytes % 16 == 0 && (x_stride_elements * 2) % 16 == 0 && tf::aligned(yp, 2) && n <= 16384;
    if (streaming)
        return tf::launch_gemv_mma_batched(ctx, stream, W, reinterpret_cast<const uint16_t*>(S), reinterpret_cast<const uint16_t*>(Bp),
                                           matrix_stride_bytes, reinterpret_cast<const uint16_t*>(xp), x_stride_elements,
                                           reinterpret_cast<uint16_t*>(yp), y_stride_elements, m, n, count, sb_dtype == TF_FP16, name);
    // shapes or alignments the streaming kernel does not take: one ordinary GEMV per matrix
    for (uint32_t b = 0; b < count; ++b) {
        tf_status s = tf::launch_gemv<4>(ctx, stream, W + (size_t)b * matrix_stride_bytes, 0, S + (size_t)b * matrix_stride_bytes, 0,
                                         Bp + (size_t)b * matrix_stride_bytes, 0, xp + (size_t)b * x_stride_elements * 2, 0,
                                         yp + (size_t)b * y_stride_elements * 2, 0, m, n, sb_dtype, name);
        if (s) return s;
    }
    return TF_OK;
}

tf_status tf_int8_gemv(tf_context* ctx, void* stream, const void* weights, uint64_t weights_off,
                       const void* scales, uint64_t scales_off, const void* biases, uint64_t biases_off,
                       const void* x, uint64_t x_off, void* y, uint64_t y_off,
                       uint32_t m, uint32_t n, tf_dtype sb_dtype) {
    return tf::launch_gemv<8>(ctx, stream, weights, weights_off, scales, scales_off, biases, biases_off,
                              x, x_off, y, y_off, m, n, sb_dtype, "tf_int8_gemv");
}

tf_status tf_shared_expert_int8_block(tf_context* ctx, void* stream, const void* x, uint64_t x_off, uint32_t x_stride_elements,
                                      const tf_projection* gate, const tf_projection* up, const tf_projection* down,
                                      void* y, uint64_t y_off, uint32_t y_stride_elements, void* scratch_act, uint32_t rows) {
    const char* name = "tf_shared_expert_int8_block";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, x && gate && up && down && y && scratch_act, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    // SharedExpertInt8.swift:80-88
    TF_REQUIRE(ctx, gate->rows == up->rows && gate->cols == up->cols, TF_ERR_DIMENSION_MISMATCH,
               "gate/up shapes differ: gate=(%u,%u) up=(%u,%u)", gate->rows, gate->cols, up->rows, up->cols);
    TF_REQUIRE(ctx, down->rows == gate->cols && down->cols == gate->rows, TF_ERR_DIMENSION_MISMATCH,
               "down expected (%u,%u), got (%u,%u)", gate->cols, gate->rows, down->rows, down->cols);
    const uint32_t fs = gate->rows, d = gate->cols;
    TF_REQUIRE(ctx, d % tf::kGroup == 0 && fs % tf::kGroup == 0 && d > 0 && fs > 0, TF_ERR_INVALID_ARGUMENT, "%s: dimensions must be multiples of 64", name);
    TF_REQUIRE(ctx, x_stride_elements >= d && y_stride_elements >= d, TF_ERR_INVALID_ARGUMENT, "%s: stride is too small", name);
    if (rows == 0) return TF_OK;
    TF_REQUIRE(ctx, rows <= 65535u, TF_ERR_UNSUPPORTED, "%s: at most 65535 rows per call", name);
    const tf_projection* ps[3] = {gate, up, down};
    const uint8_t* W[3]; const uint16_t* S[3]; const uint16_t* B[3];
    bool a4 = true;
    for (int i = 0; i < 3; ++i) {
        W[i] = tf::byte_ptr(ps[i]->weights, ps[i]->weights_off);
        S[i] = reinterpret_cast<const uint16_t*>(tf::byte_ptr(ps[i]->scales, ps[i]->scales_off));
        B[i] = reinterpret_cast<const uint16_t*>(tf::byte_ptr(ps[i]->biases, ps[i]->biases_off));
        TF_REQUIRE(ctx, tf::aligned(S[i], 2) && tf::aligned(B[i], 2), TF_ERR_ALIGNMENT, "%s: scale and bias planes must be 2-byte aligned", name);
        a4 = a4 && tf::aligned(W[i], 4);
    }
    const uint16_t* xp = reinterpret_cast<const uint16_t*>(tf::byte_ptr(x, x_off));
    uint16_t* yp = reinterpret_cast<uint16_t*>(tf::byte_ptr(y, y_off));
    TF_REQUIRE(ctx, tf::aligned(xp, 2) && tf::aligned(yp, 2) && tf::aligned(scratch_act, 2), TF_ERR_ALIGNMENT, "%s: x, y and the scratch must be 2-byte aligned", name);
    const size_t smem1 = tf::stage_x_bytes((int)d), smem2 = tf::stage_x_bytes((int)fs);
    TF_REQUIRE(ctx, smem1 <= 96 * 1024 && smem2 <= 96 * 1024, TF_ERR_UNSUPPORTED, "%s: dimensions too large for the staged-x kernels", name);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    static tf::DeviceSmemCache c1, c2;
    if (smem1 > 48 * 1024) if (tf_status s = tf::ensure_dynamic_smem(ctx, tf::shared_int8_gate_up_act_kernel, c1, smem1)) return s;
    if (smem2 > 48 * 1024) if (tf_status s = tf::ensure_dynamic_smem(ctx, tf::int8_gemv_rows_kernel, c2, smem2)) return s;
    TF_REQUIRE(ctx, rows <= 65535u, TF_ERR_UNSUPPORTED, "%s: at most 65535 rows per call", name);
    const uint32_t per_row_blocks = rows >= 64 ? 8u : (uint32_t)ctx->sm_count * 2u;       // a block keeps its token's activations staged
    auto blocks = [&](uint32_t m) { const uint32_t need = (m + tf::kGemvWarps - 1) / tf::kGemvWarps; return need < per_row_blocks ? need : per_row_blocks; };
    uint16_t* act = static_cast<uint16_t*>(scratch_act);
    tf::shared_int8_gate_up_act_kernel<<<dim3(blocks(fs), rows), tf::kGemvThreads, smem1, st>>>(W[0], S[0], B[0], W[1], S[1], B[1], xp,
                                                                                              x_stride_elements, act, fs, fs, d, a4);
    if (tf_status s = tf::check_launch(ctx, "tf_shared_expert_int8_block(gate/up)")) return s;
    tf::int8_gemv_rows_kernel<<<dim3(blocks(d), rows), tf::kGemvThreads, smem2, st>>>(W[2], S[2], B[2], act, fs, yp, y_stride_elements, d, fs, a4);
    return tf::check_launch(ctx, "tf_shared_expert_int8_block(down)");
}

}  // extern "C"
