// HBM-resident expert pool, fused MoE block and layer stack.
//
// Replaces, for a GPU whose memory holds every expert:
//   - the expert buffer manager: PreadExpertStreamer's LFU slot cache and pread path
//     (Infrastructure/Streaming/PreadExpertStreamer.swift:57-414) and
//     Model.planRoutedExperts / fetchRoutedExperts / routedExpertOffsets
//     (Runtime/Inference/ModelExpertIO.swift:21-142): "fetch" becomes
//     base + layer * layer_bytes + expert * stride;
//   - the MoE section of the forward runner (Runtime/Inference/RealForwardRunner.swift:902-1186
//     prefill, :1449-1693 decode), whose two CPU<->GPU round trips per layer exist only to
//     plan SSD reads: here router ids, grouping and expert addressing stay on the device.
#include "block.cuh"
#include "peer.cuh"

namespace tf {

constexpr uint32_t kF32PartialTokens = 64;   // decode-sized batches keep fp32 partials (decode kernel semantics)

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float unit_float(uint64_t r) { return ((float)(r >> 40) + 0.5f) * (1.0f / 16777216.0f); }

// One thread per 64-column group: uniform codes, scale = |N(0,1)| * scale_mul,
// bias = -zero_point * scale + N(0, bias_sigma), both rounded to bf16.
__global__ void fill_affine_kernel(uint8_t* W, uint16_t* S, uint16_t* B, uint64_t groups_total, int bits,
                                   uint64_t seed, float scale_mul, float zero_point, float bias_sigma) {
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= groups_total) return;
    uint64_t st = mix64(seed ^ (gid * 0xD1342543DE82EF95ull));
    const int words = bits == 4 ? 4 : 8;            // 64-bit words of codes per group
    uint64_t* wp = reinterpret_cast<uint64_t*>(W + gid * (bits == 4 ? 32 : 64));
    for (int i = 0; i < words; ++i) { st = mix64(st); wp[i] = st; }
    st = mix64(st);
    const float u1 = unit_float(st);
    st = mix64(st);
    const float u2 = unit_float(st);
    const float r = sqrtf(-2.0f * __logf(u1));
    const float n1 = r * __cosf(6.2831853f * u2), n2 = r * __sinf(6.2831853f * u2);
    const float scale = fabsf(n1) * scale_mul;
    const float bias = -zero_point * scale + n2 * bias_sigma;
    S[gid] = __bfloat16_as_ushort(__float2bfloat16_rn(scale));
    B[gid] = __bfloat16_as_ushort(__float2bfloat16_rn(bias));
}

// h += y (fp16, one rounding), then x = half(rmsnorm(h) * w). One block per row; each thread keeps
// its 8-element slices in registers (128-bit loads and stores), so the row is read once.
constexpr int kRrnThreads = 128;
constexpr int kRrnMaxSlices = 4;          // d <= 128 * 8 * 4 = 4096
__global__ void __launch_bounds__(kRrnThreads)
residual_rmsnorm_kernel(uint16_t* __restrict__ h, const uint16_t* __restrict__ y, const uint16_t* __restrict__ w,
                        uint16_t* __restrict__ x, uint32_t d, float eps) {
    __shared__ float red[kRrnThreads / kWarp];
    pdl_launch_dependents();
    pdl_wait();
    uint16_t* hr = h + (size_t)blockIdx.x * d;
    const uint32_t vecs = d / 8;
    float v[kRrnMaxSlices][8];
    float acc = 0.0f;
#pragma unroll
    for (int s = 0; s < kRrnMaxSlices; ++s) {
        const uint32_t i = threadIdx.x + s * kRrnThreads;
        if (i < vecs) {
            const uint4 hv = *reinterpret_cast<const uint4*>(hr + i * 8);
            const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
            uint32_t yw[4] = {0u, 0u, 0u, 0u};
            if (y) {
                const uint4 yv = __ldg(reinterpret_cast<const uint4*>(y + (size_t)blockIdx.x * d + i * 8));
                yw[0] = yv.x; yw[1] = yv.y; yw[2] = yv.z; yw[3] = yv.w;
            }
            uint32_t ow[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 a = __half22float2(*reinterpret_cast<const __half2*>(&hw[j]));
                if (y) {
                    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&yw[j]));
                    const __half2 r = __floats2half2_rn(a.x + b.x, a.y + b.y);
                    ow[j] = *reinterpret_cast<const uint32_t*>(&r);
                    a = __half22float2(r);
                }
                v[s][2 * j] = a.x; v[s][2 * j + 1] = a.y;
                acc = fmaf(a.x, a.x, acc); acc = fmaf(a.y, a.y, acc);
            }
            if (y) *reinterpret_cast<uint4*>(hr + i * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    float tot = (threadIdx.x & 31) < (kRrnThreads / kWarp) ? red[threadIdx.x & 31] : 0.0f;
    tot = warp_sum(tot);
    if (!x) return;
    const float inv = rsqrtf(tot / (float)d + eps);
#pragma unroll
    for (int s = 0; s < kRrnMaxSlices; ++s) {
        const uint32_t i = threadIdx.x + s * kRrnThreads;
        if (i < vecs) {
            const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w + i * 8));
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
            uint32_t ow[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 r = __floats2half2_rn(v[s][2 * j] * inv * bf16_bits_to_float((uint16_t)(ww[j] & 0xFFFFu)),
                                                    v[s][2 * j + 1] * inv * bf16_bits_to_float((uint16_t)(ww[j] >> 16)));
                ow[j] = *reinterpret_cast<const uint32_t*>(&r);
            }
            *reinterpret_cast<uint4*>(x + (size_t)blockIdx.x * d + i * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
    }
}

// Rows of 16-bit floats from one format into the other (TO_BF16 = false: bf16 -> fp16, exact for every value whose
// magnitude is zero or within fp16's normal range, since bf16 carries 8 significant bits and fp16 11; TO_BF16 = true:
// fp16 -> bf16, round to nearest even). Eight elements per thread.
template <bool TO_BF16>
__global__ void convert_rows_kernel(const uint16_t* __restrict__ src, uint32_t src_stride, uint16_t* __restrict__ dst, uint32_t dst_stride,
                                    uint32_t rows, uint32_t d) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t vecs = d / 8;
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (uint64_t)rows * vecs) return;
    const uint32_t r = (uint32_t)(i / vecs), c = (uint32_t)(i % vecs);
    const uint4 v = *reinterpret_cast<const uint4*>(src + (size_t)r * src_stride + c * 8);
    const uint32_t in[4] = {v.x, v.y, v.z, v.w};
    uint32_t out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if constexpr (TO_BF16) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&in[j]));
            const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
            out[j] = *reinterpret_cast<const uint32_t*>(&b);
        } else {
            const __half2 h = __floats2half2_rn(bf16_bits_to_float((uint16_t)(in[j] & 0xFFFFu)), bf16_bits_to_float((uint16_t)(in[j] >> 16)));
            out[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    *reinterpret_cast<uint4*>(dst + (size_t)r * dst_stride + c * 8) = make_uint4(out[0], out[1], out[2], out[3]);
}

// The weighted sum of a decode-sized block's fp32 route partials, the residual add and the next norm in one launch:
//   y = half(float(shared_y) + sum_r float(w_r) * partial_r)   (rank order; reduce_token_major_kernel<true>, moe.metal:473-480)
//   h = half(h + y);  x = half(rmsnorm(h) * w)                 (residual_rmsnorm_kernel)
// with the bits of those two kernels. One block per token, one thread per eight columns (every thread has 2 K + 2
// 16-byte loads in flight), so the 90 KB of partials of a token do not wait on a 128-thread block. The sum of squares
// keeps the order of residual_rmsnorm_kernel: there thread t adds the squares of its slices t, t + 128, t + 256 in turn;
// here the thread of slice s takes over the running sum of the thread of slice s - 1 through shared memory.
// ROWS: the block's results are fp16 rows reached through a permutation (the expert-parallel combine, and prefill-sized
// blocks): y = half(sum_r fma(float(w_r), float(rows[perm[t, r]]), acc) + float(shared_y)) (ep_combine_kernel), and the rows
// may still be on their way from peers (peer_wait).
constexpr int kCrnMaxThreads = kRrnThreads * kRrnMaxSlices;      // 512: d <= 4096
template <bool ROWS>
__global__ void __launch_bounds__(kCrnMaxThreads)
combine_residual_rmsnorm_kernel(uint16_t* __restrict__ h, const void* __restrict__ results, const uint16_t* __restrict__ route_weights,
                                const uint32_t* __restrict__ inverse_perm, const uint16_t* __restrict__ shared_y,
                                const uint16_t* __restrict__ w, uint16_t* __restrict__ x, uint32_t d, uint32_t top_k, float eps,
                                const PeerWait peer_wait) {
    __shared__ float chain[kRrnThreads];
    __shared__ float red[kRrnThreads / kWarp];
    pdl_launch_dependents();
    pdl_wait();
    if constexpr (ROWS) peer_wait_in_block(peer_wait);
    const uint32_t vecs = d / 8, i = threadIdx.x, token = blockIdx.x;
    const uint32_t vt = i % kRrnThreads, slice = i / kRrnThreads;
    float v[8];
    if (i < vecs) {
        float4 p[TF_MAX_TOP_K][2];          // fp32 partials, or (ROWS) the eight fp16 values of a row in p[r][0]
        float rw[TF_MAX_TOP_K];
#pragma unroll
        for (int r = 0; r < TF_MAX_TOP_K; ++r) {
            if ((uint32_t)r < top_k) {
                if constexpr (ROWS) {
                    const uint32_t slot = __ldg(inverse_perm + (size_t)token * top_k + r);
                    const uint4 rv = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(results) + (size_t)slot * d + i * 8);
                    p[r][0] = make_float4(__uint_as_float(rv.x), __uint_as_float(rv.y), __uint_as_float(rv.z), __uint_as_float(rv.w));
                } else {
                    const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(results) + ((size_t)token * top_k + r) * d + i * 8);
                    p[r][0] = __ldg(src); p[r][1] = __ldg(src + 1);
                }
                rw[r] = f16_bits_to_float(__ldg(route_weights + (size_t)token * top_k + r));
            } else {
                p[r][0] = make_float4(0.0f, 0.0f, 0.0f, 0.0f); p[r][1] = p[r][0]; rw[r] = 0.0f;
            }
        }
        const uint4 hv = *reinterpret_cast<const uint4*>(h + (size_t)token * d + i * 8);
        uint4 sv = make_uint4(0u, 0u, 0u, 0u);
        if (shared_y) sv = __ldg(reinterpret_cast<const uint4*>(shared_y + (size_t)token * d + i * 8));
        const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w}, sw[4] = {sv.x, sv.y, sv.z, sv.w};
        uint32_t ow[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 res = __half22float2(*reinterpret_cast<const __half2*>(&sw[j]));
            float a0, a1;
            if constexpr (ROWS) {
                a0 = 0.0f; a1 = 0.0f;
#pragma unroll
                for (int r = 0; r < TF_MAX_TOP_K; ++r) {
                    if ((uint32_t)r < top_k) {
                        const uint32_t pair = __float_as_uint(reinterpret_cast<const float*>(&p[r][0])[j]);
                        a0 = fmaf(rw[r], f16_bits_to_float((uint16_t)(pair & 0xFFFFu)), a0);
                        a1 = fmaf(rw[r], f16_bits_to_float((uint16_t)(pair >> 16)), a1);
                    }
                }
                if (shared_y) { a0 += res.x; a1 += res.y; }
            } else {
                a0 = res.x; a1 = res.y;
#pragma unroll
                for (int r = 0; r < TF_MAX_TOP_K; ++r) {
                    if ((uint32_t)r < top_k) {
                        const float* pr = reinterpret_cast<const float*>(&p[r][0]);
                        a0 = __fadd_rn(a0, __fmul_rn(rw[r], pr[2 * j]));
                        a1 = __fadd_rn(a1, __fmul_rn(rw[r], pr[2 * j + 1]));
                    }
                }
            }
            const float2 yy = __half22float2(__floats2half2_rn(a0, a1));                       // y, stored as fp16 by the reduce
            const float2 hh = __half22float2(*reinterpret_cast<const __half2*>(&hw[j]));
            const __half2 nh = __floats2half2_rn(hh.x + yy.x, hh.y + yy.y);
            ow[j] = *reinterpret_cast<const uint32_t*>(&nh);
            const float2 nf = __half22float2(nh);
            v[2 * j] = nf.x; v[2 * j + 1] = nf.y;
        }
        *reinterpret_cast<uint4*>(h + (size_t)token * d + i * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    // sum of squares in the order of residual_rmsnorm_kernel
    const uint32_t slices = (vecs + kRrnThreads - 1) / kRrnThreads;
    if (i < kRrnThreads) chain[i] = 0.0f;
    __syncthreads();
    for (uint32_t s = 0; s < slices; ++s) {
        if (slice == s && i < vecs) {
            float acc = chain[vt];
#pragma unroll
            for (int q = 0; q < 8; ++q) acc = fmaf(v[q], v[q], acc);
            chain[vt] = acc;
        }
        __syncthreads();
    }
    if (i < kRrnThreads) {
        const float acc = warp_sum(chain[i]);
        if ((i & 31) == 0) red[i >> 5] = acc;
    }
    __syncthreads();
    if (!x) return;
    float tot = (threadIdx.x & 31) < (kRrnThreads / kWarp) ? red[threadIdx.x & 31] : 0.0f;
    tot = warp_sum(tot);
    const float inv = rsqrtf(tot / (float)d + eps);
    if (i < vecs) {
        const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w + i * 8));
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t ow[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __half2 r = __floats2half2_rn(v[2 * j] * inv * bf16_bits_to_float((uint16_t)(ww[j] & 0xFFFFu)),
                                                v[2 * j + 1] * inv * bf16_bits_to_float((uint16_t)(ww[j] >> 16)));
            ow[j] = *reinterpret_cast<const uint32_t*>(&r);
        }
        *reinterpret_cast<uint4*>(x + (size_t)token * d + i * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

}  // namespace tf

extern "C" {

// ---------------------------------------------------------------------------
// pool
// ---------------------------------------------------------------------------

tf_status tf_expert_pool_create(tf_context* ctx, uint32_t layers, uint32_t experts, uint64_t stride,
                                const tf_expert_offsets* offsets, tf_pool** out) {
    const char* name = "tf_expert_pool_create";
    TF_REQUIRE(ctx, ctx != nullptr && out != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    *out = nullptr;
    TF_REQUIRE(ctx, layers > 0 && experts > 0 && stride > 0 && offsets, TF_ERR_INVALID_ARGUMENT, "%s: bad dimensions", name);
    TF_REQUIRE(ctx, stride % 256 == 0, TF_ERR_ALIGNMENT, "%s: expert stride must be a multiple of 256 bytes", name);
    uint8_t* base = nullptr;
    const uint64_t bytes = (uint64_t)layers * experts * stride;
    cudaError_t e = cudaMalloc(&base, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return tf::fail(ctx, TF_ERR_OUT_OF_MEMORY, "failed to allocate expert pool of %llu bytes: %s",
                        (unsigned long long)bytes, cudaGetErrorString(e));
    }
    tf_pool* p = new tf_pool{ctx, base, layers, experts, stride, *offsets};
    *out = p;
    return TF_OK;
}

void tf_expert_pool_destroy(tf_pool* pool) {
    if (!pool) return;
    cudaFree(pool->base);
    delete pool;
}

const void* tf_expert_pool_ptr(const tf_pool* pool, uint32_t layer, uint32_t expert) {
    if (!pool || layer >= pool->layers || expert >= pool->experts) return nullptr;
    return pool->base + ((uint64_t)layer * pool->experts + expert) * pool->stride;
}

uint64_t tf_expert_pool_bytes(const tf_pool* pool) {
    return pool ? (uint64_t)pool->layers * pool->experts * pool->stride : 0;
}

void tf_expert_pool_dims(const tf_pool* pool, uint32_t* layers_out, uint32_t* experts_out, uint64_t* stride_out) {
    if (layers_out) *layers_out = pool ? pool->layers : 0u;
    if (experts_out) *experts_out = pool ? pool->experts : 0u;
    if (stride_out) *stride_out = pool ? pool->stride : 0u;
}

tf_status tf_expert_pool_upload(tf_pool* pool, void* stream, uint32_t layer, uint32_t expert,
                                const void* host_blob, uint64_t bytes) {
    const char* name = "tf_expert_pool_upload";
    TF_REQUIRE(nullptr, pool != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: pool is NULL", name);
    tf_context* ctx = pool->ctx;
    TF_REQUIRE(ctx, host_blob != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: blob is NULL", name);
    TF_REQUIRE(ctx, layer < pool->layers && expert < pool->experts, TF_ERR_INVALID_ARGUMENT,
               "%s: (layer %u, expert %u) out of range", name, layer, expert);
    TF_REQUIRE(ctx, bytes <= pool->stride, TF_ERR_INVALID_ARGUMENT, "%s: blob of %llu bytes exceeds the stride %llu",
               name, (unsigned long long)bytes, (unsigned long long)pool->stride);
    TF_CUDA(ctx, cudaMemcpyAsync(const_cast<void*>(tf_expert_pool_ptr(pool, layer, expert)), host_blob, bytes,
                                 cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
    return TF_OK;
}

tf_status tf_fill_affine_synthetic(tf_context* ctx, void* stream, void* weights, void* scales, void* biases,
                                   uint32_t rows, uint32_t cols, uint32_t bits, uint64_t seed) {
    const char* name = "tf_fill_affine_synthetic";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, weights && scales && biases, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, (bits == 4 || bits == 8) && cols % tf::kGroup == 0, TF_ERR_INVALID_ARGUMENT, "%s: bits must be 4 or 8, cols a multiple of 64", name);
    TF_REQUIRE(ctx, tf::aligned(weights, 8) && tf::aligned(scales, 2) && tf::aligned(biases, 2), TF_ERR_ALIGNMENT, "%s: alignment", name);
    const uint64_t groups = (uint64_t)rows * (cols / tf::kGroup);
    if (groups == 0) return TF_OK;
    const float scale_mul = bits == 4 ? 0.004f : 0.004f / 16.0f;
    const float zero = bits == 4 ? 8.0f : 128.0f;
    tf::fill_affine_kernel<<<(uint32_t)((groups + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint8_t*>(weights), static_cast<uint16_t*>(scales), static_cast<uint16_t*>(biases), groups,
        (int)bits, seed, scale_mul, zero, 1e-4f);
    return tf::check_launch(ctx, name);
}

static tf_status fill_pool_synthetic(tf_pool* pool, void* stream, uint64_t seed, uint32_t d, uint32_t f,
                                     uint32_t global_experts, uint32_t expert_offset, const uint32_t* original_ids) {
    tf_context* ctx = pool->ctx;
    const tf_expert_offsets& o = pool->offsets;
    for (uint32_t l = 0; l < pool->layers; ++l)
        for (uint32_t e = 0; e < pool->experts; ++e) {
            uint8_t* b = const_cast<uint8_t*>(static_cast<const uint8_t*>(tf_expert_pool_ptr(pool, l, e)));
            // seeded by the GLOBAL expert id, so a shard holds the same bytes as the unsharded pool
            const uint32_t id = original_ids ? original_ids[(size_t)l * pool->experts + e] : expert_offset + e;
            const uint64_t s0 = seed + ((uint64_t)l * global_experts + id) * 3;
            tf_status s = tf_fill_affine_synthetic(ctx, stream, b + o.gate_w_off, b + o.gate_s_off, b + o.gate_b_off, f, d, 4, s0);
            if (!s) s = tf_fill_affine_synthetic(ctx, stream, b + o.up_w_off, b + o.up_s_off, b + o.up_b_off, f, d, 4, s0 + 1);
            if (!s) s = tf_fill_affine_synthetic(ctx, stream, b + o.down_w_off, b + o.down_s_off, b + o.down_b_off, d, f, 4, s0 + 2);
            if (s) return s;
        }
    return TF_OK;
}

tf_status tf_expert_pool_fill_synthetic(tf_pool* pool, void* stream, uint64_t seed, uint32_t d, uint32_t f,
                                        uint32_t global_experts, uint32_t expert_offset) {
    const char* name = "tf_expert_pool_fill_synthetic";
    TF_REQUIRE(nullptr, pool != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: pool is NULL", name);
    tf_context* ctx = pool->ctx;
    if (global_experts == 0) global_experts = pool->experts;
    TF_REQUIRE(ctx, expert_offset + pool->experts <= global_experts, TF_ERR_INVALID_ARGUMENT,
               "%s: shard [%u, %u) exceeds %u experts", name, expert_offset, expert_offset + pool->experts, global_experts);
    return fill_pool_synthetic(pool, stream, seed, d, f, global_experts, expert_offset, nullptr);
}

tf_status tf_expert_pool_fill_synthetic_placed(tf_pool* pool, void* stream, uint64_t seed, uint32_t d, uint32_t f,
                                               uint32_t global_experts, const uint32_t* original_ids) {
    const char* name = "tf_expert_pool_fill_synthetic_placed";
    TF_REQUIRE(nullptr, pool != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: pool is NULL", name);
    tf_context* ctx = pool->ctx;
    TF_REQUIRE(ctx, original_ids != nullptr && global_experts >= pool->experts, TF_ERR_INVALID_ARGUMENT,
               "%s: NULL id table or fewer global experts than slots", name);
    for (size_t i = 0; i < (size_t)pool->layers * pool->experts; ++i)
        TF_REQUIRE(ctx, original_ids[i] < global_experts, TF_ERR_INVALID_ARGUMENT, "%s: id %u of entry %zu is not below %u",
                   name, original_ids[i], i, global_experts);
    return fill_pool_synthetic(pool, stream, seed, d, f, global_experts, 0, original_ids);
}

// ---------------------------------------------------------------------------
// workspace
// ---------------------------------------------------------------------------

tf_status tf_workspace_create(tf_context* ctx, uint32_t max_tokens, uint32_t d, uint32_t f, uint32_t fs,
                              uint32_t top_k, uint32_t num_experts, tf_workspace** out) {
    const char* name = "tf_workspace_create";
    TF_REQUIRE(ctx, ctx != nullptr && out != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    *out = nullptr;
    TF_REQUIRE(ctx, max_tokens > 0 && d > 0 && f > 0 && fs > 0 && top_k > 0 && num_experts > 0, TF_ERR_INVALID_ARGUMENT, "%s: bad dimensions", name);
    const uint64_t T = max_tokens, K = top_k, E = num_experts;
    auto up = [](uint64_t v) { return (v + 255) / 256 * 256; };
    uint64_t off = 0;
    auto take = [&](uint64_t bytes) { uint64_t o = off; off += up(bytes); return o; };
    const uint64_t o_idx = take(T * K * 4), o_w = take(T * K * 2), o_pairs = take(T * K * 16), o_eoff = take(E * 4),
                   o_ecnt = take(E * 4), o_groups = take(E * 12), o_cgroup = take((T * K / 8 + E + 1) * 4),
                   o_cstart = take(E * 4), o_counters = take(16), o_acts = take(T * K * f * 2),
                   o_partials = take(T * K * d * (T <= tf::kF32PartialTokens ? 4 : 2)), o_sact = take(T * fs * 2),
                   o_sy = take(T * d * 2), o_xn = take(T * d * 2), o_yb = take(T * d * 2);
    // workspaces that can hold a tensor-core sized block also carry the expert-sorted activation rows
    const bool tensor_path = T >= ctx->tensorcore_min_tokens && d % 64 == 0 && f % 64 == 0 && fs % 64 == 0;
    const uint64_t o_xs = tensor_path ? take(T * K * d * 2) : 0, o_inv = tensor_path ? take(T * K * 4) : 0,
                   o_pid = tensor_path ? take(T * K * 4) : 0;
    uint8_t* base = nullptr;
    cudaError_t e = cudaMalloc(&base, off);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return tf::fail(ctx, TF_ERR_OUT_OF_MEMORY, "failed to allocate workspace of %llu bytes: %s", (unsigned long long)off, cudaGetErrorString(e));
    }
    cudaMemset(base, 0, off);
    tf_workspace* w = new tf_workspace();
    w->ctx = ctx; w->max_tokens = max_tokens; w->d = d; w->f = f; w->fs = fs; w->top_k = top_k; w->num_experts = num_experts;
    w->base = base; w->bytes = off;
    w->indices = reinterpret_cast<uint32_t*>(base + o_idx);
    w->weights = reinterpret_cast<uint16_t*>(base + o_w);
    w->routes.sorted_pairs = reinterpret_cast<tf_pair*>(base + o_pairs);
    w->routes.per_expert_offsets = reinterpret_cast<uint32_t*>(base + o_eoff);
    w->routes.per_expert_counts = reinterpret_cast<uint32_t*>(base + o_ecnt);
    w->routes.groups = reinterpret_cast<tf_group*>(base + o_groups);
    w->routes.chunk_group = reinterpret_cast<uint32_t*>(base + o_cgroup);
    w->routes.chunk_start = reinterpret_cast<uint32_t*>(base + o_cstart);
    w->routes.counters = reinterpret_cast<uint32_t*>(base + o_counters);
    w->acts = reinterpret_cast<uint16_t*>(base + o_acts);
    w->partials = base + o_partials;
    w->shared_act = reinterpret_cast<uint16_t*>(base + o_sact);
    w->shared_y = reinterpret_cast<uint16_t*>(base + o_sy);
    w->x_norm = reinterpret_cast<uint16_t*>(base + o_xn);
    w->y_block = reinterpret_cast<uint16_t*>(base + o_yb);
    w->x_sorted = tensor_path ? reinterpret_cast<uint16_t*>(base + o_xs) : nullptr;
    w->inverse_perm = tensor_path ? reinterpret_cast<uint32_t*>(base + o_inv) : nullptr;
    w->pack_ids = tensor_path ? reinterpret_cast<uint32_t*>(base + o_pid) : nullptr;
    *out = w;
    return TF_OK;
}

void tf_workspace_destroy(tf_workspace* ws) {
    if (!ws) return;
    cudaFree(ws->base);
    delete ws;
}

uint64_t tf_workspace_bytes(const tf_workspace* ws) { return ws ? ws->bytes : 0; }

// Device addresses of the routing results of the last block forward (for inspection by tests).
const uint32_t* tf_workspace_indices(const tf_workspace* ws) { return ws ? ws->indices : nullptr; }
const void* tf_workspace_weights(const tf_workspace* ws) { return ws ? ws->weights : nullptr; }
const tf_device_routes* tf_workspace_routes(const tf_workspace* ws) { return ws ? &ws->routes : nullptr; }

// ---------------------------------------------------------------------------
// fused block and stack
// ---------------------------------------------------------------------------

}  // extern "C"

namespace tf {

// Router, device grouping and the routed experts of one block, on the caller's stream.
static tf_status block_routed(tf_context* ctx, void* stream, const tf_moe_layer* layer, const void* x, uint32_t x_stride_elements,
                              uint32_t tokens, tf_workspace* ws, bool tensor_path) {
    const uint32_t d = layer->d, f = layer->f, K = layer->top_k, E = layer->num_experts;
    // decode-sized blocks route and group in one launch
    tf_status s = tf_router_gemma4_block_grouped(ctx, stream, layer->router.weights, layer->router.weights_off,
                                                 layer->router.scales, layer->router.scales_off,
                                                 layer->router.biases, layer->router.biases_off,
                                                 x, 0, TF_FP16, layer->effective_scale, 0, layer->per_expert_scale, 0,
                                                 layer->logit_bias, ws->indices, ws->weights, tokens, E, d, K,
                                                 x_stride_elements, &ws->routes);
    if (s) return s;
    if (tensor_path) {
        // Prefill-sized block: gather the rows into expert order and run gate/up/GeGLU/down as tcgen05 GEMMs; the
        // combine folds the sorted rows back per token in rank order.
        s = tf_pack_sorted_rows(ctx, stream, x, x_stride_elements, &ws->routes, tokens, K, E, d, ws->x_sorted, ws->pack_ids,
                                ws->inverse_perm);
        if (s) return s;
        return tf_grouped_moe_tensorcore(ctx, stream, ws->x_sorted, tokens * K, layer->pool_layer_base, layer->expert_stride, E,
                                         &layer->offsets, &ws->routes, ws->acts, ws->partials, d, f);
    }
    // The partial dtype follows the workspace's capacity so that one workspace
    // always runs the same arithmetic whatever the call's token count.
    const int f32 = ws->max_tokens <= kF32PartialTokens ? 1 : 0;
    return tf_grouped_moe_batched(ctx, stream, x, 0, x_stride_elements, layer->pool_layer_base, layer->expert_stride,
                                  &layer->offsets, &ws->routes, ws->acts, ws->partials, f32, tokens, d, f, K);
}

}  // namespace tf

extern "C" {

}  // extern "C"

namespace tf {

// Decode-sized blocks leave fp32 route partials that the next layer's norm can fold in (combine_residual_rmsnorm_kernel).
static bool block_keeps_f32_partials(const tf_context* ctx, const tf_workspace* ws, uint32_t tokens) {
    const bool tensor_path = tokens >= ctx->tensorcore_min_tokens && ws->x_sorted != nullptr;
    return !tensor_path && ws->max_tokens <= kF32PartialTokens;
}

// tf_moe_block_forward; with y == nullptr the last step (weighted sum of the route partials plus the shared expert)
// is left to the caller, which finds the partials, weights and shared output in the workspace.
static tf_status block_forward(tf_context* ctx, void* stream, const tf_moe_layer* layer,
                               const void* x, uint32_t x_stride_elements,
                               void* y, uint32_t y_stride_elements, uint32_t tokens, tf_workspace* ws) {
    const char* name = "tf_moe_block_forward";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, layer && x && ws, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, tokens <= ws->max_tokens, TF_ERR_SCRATCH_TOO_SMALL, "%s: %u tokens exceed the workspace (%u)", name, tokens, ws->max_tokens);
    TF_REQUIRE(ctx, layer->d == ws->d && layer->f == ws->f && layer->fs == ws->fs && layer->top_k == ws->top_k &&
                        layer->num_experts == ws->num_experts,
               TF_ERR_DIMENSION_MISMATCH, "%s: layer dimensions differ from the workspace", name);
    TF_REQUIRE(ctx, layer->router.rows == layer->num_experts && layer->router.cols == layer->d, TF_ERR_DIMENSION_MISMATCH,
               "%s: router is (%u,%u), expected (%u,%u)", name, layer->router.rows, layer->router.cols, layer->num_experts, layer->d);
    if (tokens == 0) return TF_OK;
    const uint32_t d = layer->d, K = layer->top_k;
    // The shared expert needs only x, so it runs on the context's side stream beside the router and the routed
    // experts and joins before the combine (inside a stream capture this becomes a fork and a join of the graph).
    cudaStream_t main_st = static_cast<cudaStream_t>(stream);
    TF_CUDA(ctx, cudaEventRecord(ctx->fork_event, main_st));
    TF_CUDA(ctx, cudaStreamWaitEvent(ctx->side_stream, ctx->fork_event, 0));
    const bool tensor_path = tokens >= ctx->tensorcore_min_tokens && ws->x_sorted != nullptr;
    tf_status s;
    if (layer->shared_bits == 8)
        s = tf_shared_expert_int8_block(ctx, ctx->side_stream, x, 0, x_stride_elements, &layer->shared_gate, &layer->shared_up,
                                        &layer->shared_down, ws->shared_y, 0, d, ws->shared_act, tokens);
    else if (tensor_path || (tokens >= ctx->shared_tensorcore_min_tokens && d % 64 == 0 && layer->fs % 64 == 0))
        s = tf_shared_expert_int4_tensorcore(ctx, ctx->side_stream, x, x_stride_elements, &layer->shared_gate, &layer->shared_up,
                                             &layer->shared_down, ws->shared_y, d, ws->shared_act, tokens);
    else
        s = tf_shared_expert_int4_block(ctx, ctx->side_stream, x, 0, x_stride_elements, &layer->shared_gate, &layer->shared_up,
                                        &layer->shared_down, ws->shared_y, 0, d, ws->shared_act, tokens);
    // the join is recorded even after a failure so that a capture in progress stays well formed
    cudaEventRecord(ctx->join_event, ctx->side_stream);
    if (s) { cudaStreamWaitEvent(main_st, ctx->join_event, 0); return s; }
    s = tf::block_routed(ctx, stream, layer, x, x_stride_elements, tokens, ws, tensor_path);
    TF_CUDA(ctx, cudaStreamWaitEvent(main_st, ctx->join_event, 0));
    if (s) return s;
    if (y == nullptr) return TF_OK;
    if (tensor_path)
        return tf_ep_combine(ctx, stream, ws->partials, ws->weights, ws->inverse_perm, ws->shared_y, d, y, y_stride_elements,
                             tokens, K, d);
    const int f32 = ws->max_tokens <= tf::kF32PartialTokens ? 1 : 0;
    return tf_moe_reduce_token_major(ctx, stream, ws->partials, f32, ws->weights, ws->shared_y, d, y,
                                     y_stride_elements, tokens, K, d);
}

}  // namespace tf

namespace tf {

// h += y, x = rmsnorm(h) * w with y formed from fp16 result rows through a permutation (see combine_residual_rmsnorm_kernel);
// norm_weight_bf16 and x may be NULL (the closing residual add of a stack).
tf_status combine_rows_residual_rmsnorm(tf_context* ctx, void* stream, void* hidden, const void* rows, const void* route_weights,
                                        const uint32_t* inverse_perm, const void* shared_y, const void* norm_weight_bf16, void* x,
                                        uint32_t tokens, uint32_t top_k, uint32_t d, float eps, const PeerWait* peer_wait) {
    const char* name = "combine_rows_residual_rmsnorm";
    TF_REQUIRE(ctx, hidden && rows && route_weights && inverse_perm && (x == nullptr || norm_weight_bf16 != nullptr), TF_ERR_INVALID_ARGUMENT,
               "%s: NULL argument", name);
    TF_REQUIRE(ctx, d % 8 == 0 && d <= 8u * kCrnMaxThreads && top_k > 0 && top_k <= TF_MAX_TOP_K, TF_ERR_UNSUPPORTED,
               "%s: D must be a multiple of 8 up to %d and top_k at most %d", name, 8 * kCrnMaxThreads, TF_MAX_TOP_K);
    TF_REQUIRE(ctx, aligned(hidden, 16) && aligned(rows, 16) && aligned(shared_y, 16) && aligned(norm_weight_bf16, 16) && aligned(x, 16),
               TF_ERR_ALIGNMENT, "%s: buffers must be 16-byte aligned", name);
    if (tokens == 0) return TF_OK;
    uint32_t threads = ((d / 8 + 31) / 32) * 32;
    if (threads < (uint32_t)kRrnThreads) threads = kRrnThreads;
    launch_pdl(combine_residual_rmsnorm_kernel<true>, dim3(tokens), dim3(threads), 0, static_cast<cudaStream_t>(stream),
               static_cast<uint16_t*>(hidden), rows, static_cast<const uint16_t*>(route_weights), inverse_perm,
               static_cast<const uint16_t*>(shared_y), static_cast<const uint16_t*>(norm_weight_bf16), static_cast<uint16_t*>(x), d, top_k, eps,
               peer_wait ? *peer_wait : PeerWait{nullptr, nullptr, nullptr, 0u});
    return check_launch(ctx, name);
}

}  // namespace tf

extern "C" {

tf_status tf_moe_block_forward(tf_context* ctx, void* stream, const tf_moe_layer* layer,
                               const void* x, uint32_t x_stride_elements,
                               void* y, uint32_t y_stride_elements, uint32_t tokens, tf_workspace* ws) {
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "tf_moe_block_forward: ctx is NULL");
    TF_REQUIRE(ctx, y != nullptr, TF_ERR_INVALID_ARGUMENT, "tf_moe_block_forward: NULL argument");
    return tf::block_forward(ctx, stream, layer, x, x_stride_elements, y, y_stride_elements, tokens, ws);
}

tf_status tf_convert_rows(tf_context* ctx, void* stream, const void* src, tf_dtype src_dtype, uint32_t src_stride_elements,
                          void* dst, tf_dtype dst_dtype, uint32_t dst_stride_elements, uint32_t rows, uint32_t d) {
    const char* name = "tf_convert_rows";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, src && dst, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, (src_dtype == TF_BF16 && dst_dtype == TF_FP16) || (src_dtype == TF_FP16 && dst_dtype == TF_BF16), TF_ERR_INVALID_ARGUMENT,
               "%s: one side must be fp16 and the other bf16", name);
    TF_REQUIRE(ctx, d % 8 == 0 && src_stride_elements >= d && dst_stride_elements >= d && src_stride_elements % 8 == 0 &&
                        dst_stride_elements % 8 == 0 && tf::aligned(src, 16) && tf::aligned(dst, 16),
               TF_ERR_ALIGNMENT, "%s: rows must be 16-byte aligned and D a multiple of 8", name);
    if (rows == 0 || d == 0) return TF_OK;
    const uint64_t n = (uint64_t)rows * (d / 8);
    const dim3 grid((uint32_t)((n + 255) / 256));
    if (dst_dtype == TF_BF16)
        tf::launch_pdl(tf::convert_rows_kernel<true>, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(src),
                       src_stride_elements, static_cast<uint16_t*>(dst), dst_stride_elements, rows, d);
    else
        tf::launch_pdl(tf::convert_rows_kernel<false>, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(src),
                       src_stride_elements, static_cast<uint16_t*>(dst), dst_stride_elements, rows, d);
    return tf::check_launch(ctx, name);
}

tf_status tf_moe_block_forward_bf16(tf_context* ctx, void* stream, const tf_moe_layer* layer,
                                    const void* x_bf16, uint32_t x_stride_elements,
                                    void* y_bf16, uint32_t y_stride_elements, uint32_t tokens, tf_workspace* ws) {
    const char* name = "tf_moe_block_forward_bf16";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, layer && x_bf16 && y_bf16 && ws, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, tokens <= ws->max_tokens, TF_ERR_SCRATCH_TOO_SMALL, "%s: %u tokens exceed the workspace (%u)", name, tokens, ws->max_tokens);
    TF_REQUIRE(ctx, layer->d == ws->d, TF_ERR_DIMENSION_MISMATCH, "%s: layer dimensions differ from the workspace", name);
    if (tokens == 0) return TF_OK;
    const uint32_t d = ws->d;
    // bf16 rows are exact in fp16 inside fp16's normal range, so the block computes on the same activation values; its fp16
    // weight tiles carry three more significant bits than bf16 tiles would. The workspace's stack scratch holds both copies.
    if (tf_status s = tf_convert_rows(ctx, stream, x_bf16, TF_BF16, x_stride_elements, ws->x_norm, TF_FP16, d, tokens, d)) return s;
    if (tf_status s = tf::block_forward(ctx, stream, layer, ws->x_norm, d, ws->y_block, d, tokens, ws)) return s;
    return tf_convert_rows(ctx, stream, ws->y_block, TF_FP16, d, y_bf16, TF_BF16, y_stride_elements, tokens, d);
}

tf_status tf_residual_rmsnorm(tf_context* ctx, void* stream, void* hidden, const void* y, const void* weight_bf16,
                              void* x_out, uint32_t rows, uint32_t d, float eps) {
    const char* name = "tf_residual_rmsnorm";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, hidden != nullptr && (x_out == nullptr || weight_bf16 != nullptr), TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, d % 8 == 0 && d <= 8u * tf::kRrnThreads * tf::kRrnMaxSlices, TF_ERR_UNSUPPORTED,
               "%s: D must be a multiple of 8 and at most %d", name, 8 * tf::kRrnThreads * tf::kRrnMaxSlices);
    TF_REQUIRE(ctx, tf::aligned(hidden, 16) && tf::aligned(y, 16) && tf::aligned(weight_bf16, 16) && tf::aligned(x_out, 16),
               TF_ERR_ALIGNMENT, "%s: buffers must be 16-byte aligned", name);
    if (rows == 0) return TF_OK;
    tf::launch_pdl(tf::residual_rmsnorm_kernel, dim3(rows), dim3(tf::kRrnThreads), 0, static_cast<cudaStream_t>(stream),
                   static_cast<uint16_t*>(hidden), static_cast<const uint16_t*>(y), static_cast<const uint16_t*>(weight_bf16),
                   static_cast<uint16_t*>(x_out), d, eps);
    return tf::check_launch(ctx, name);
}

// ---------------------------------------------------------------------------
// expert-parallel layer phases (the collectives between them are the caller's)
// ---------------------------------------------------------------------------

tf_status tf_ep_dispatch(tf_context* ctx, void* stream, const tf_moe_layer* layer, const void* x, uint32_t tokens,
                         tf_workspace* ws, uint32_t experts_per_rank, uint32_t capacity,
                         void* send_rows, uint32_t* send_expert_ids, uint32_t* inverse_perm, uint32_t send_row_stride_elements) {
    const char* name = "tf_ep_dispatch";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, layer && x && ws, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, tokens <= ws->max_tokens, TF_ERR_SCRATCH_TOO_SMALL, "%s: %u tokens exceed the workspace (%u)", name, tokens, ws->max_tokens);
    if (tokens == 0) return TF_OK;
    const uint32_t d = layer->d, K = layer->top_k, E = layer->num_experts;
    // router and grouping over the GLOBAL experts (one launch for decode-sized blocks)
    tf_status s = tf_router_gemma4_block_grouped(ctx, stream, layer->router.weights, layer->router.weights_off,
                                                 layer->router.scales, layer->router.scales_off,
                                                 layer->router.biases, layer->router.biases_off,
                                                 x, 0, TF_FP16, layer->effective_scale, 0, layer->per_expert_scale, 0,
                                                 layer->logit_bias, ws->indices, ws->weights, tokens, E, d, K, d, &ws->routes);
    if (s) return s;
    return tf_ep_pack(ctx, stream, x, 0, d, &ws->routes, tokens, K, E, experts_per_rank, capacity, d, send_rows,
                      send_expert_ids, inverse_perm, send_row_stride_elements);
}

}  // extern "C"

namespace tf {

tf_status ep_experts_waiting(tf_context* ctx, void* stream, const void* pool_layer_base, uint64_t expert_stride,
                             const tf_expert_offsets* offsets, const void* recv_rows, const uint32_t* recv_expert_ids,
                             uint32_t recv_slots, uint32_t local_experts, const tf_device_routes* recv_routes,
                             const void* zero_weights, void* acts_scratch, void* out_rows, uint32_t d, uint32_t f,
                             uint32_t recv_row_stride_elements, const PeerWait* peer_wait) {
    const char* name = "tf_ep_experts";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, pool_layer_base && offsets && recv_rows && recv_expert_ids && recv_routes && zero_weights && acts_scratch && out_rows,
               TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    if (recv_slots == 0) return TF_OK;
    const uint32_t stride = recv_row_stride_elements ? recv_row_stride_elements : d;
    tf_status s;
    // every received row is one (token = slot, rank 0) pair of a local expert; empty slots carry UINT32_MAX
    if (stride > d) {
        // the rows carry their expert id in the tail: the grouping reads it there (no second exchange, no extra launch)
        // and fills recv_expert_ids on the way
        TF_REQUIRE(ctx, d % 2 == 0 && stride % 2 == 0 && tf::aligned(recv_rows, 4), TF_ERR_ALIGNMENT, "%s: rows must be 4-byte aligned", name);
        s = tf::group_routes_strided(ctx, stream, reinterpret_cast<const uint32_t*>(static_cast<const uint16_t*>(recv_rows) + d), stride / 2,
                                     const_cast<uint32_t*>(recv_expert_ids), zero_weights, recv_slots, 1, local_experts, recv_routes, name,
                                     peer_wait);
    } else {
        s = tf::group_routes_strided(ctx, stream, recv_expert_ids, 1, nullptr, zero_weights, recv_slots, 1, local_experts, recv_routes,
                                     name, peer_wait);
    }
    if (s) return s;
    return tf_grouped_moe_batched(ctx, stream, recv_rows, 0, stride, pool_layer_base, expert_stride, offsets, recv_routes,
                                  acts_scratch, out_rows, 0, recv_slots, d, f, 1);
}

}  // namespace tf

extern "C" {

tf_status tf_ep_experts(tf_context* ctx, void* stream, const void* pool_layer_base, uint64_t expert_stride,
                        const tf_expert_offsets* offsets, const void* recv_rows, const uint32_t* recv_expert_ids,
                        uint32_t recv_slots, uint32_t local_experts, const tf_device_routes* recv_routes,
                        const void* zero_weights, void* acts_scratch, void* out_rows, uint32_t d, uint32_t f,
                        uint32_t recv_row_stride_elements) {
    return tf::ep_experts_waiting(ctx, stream, pool_layer_base, expert_stride, offsets, recv_rows, recv_expert_ids, recv_slots,
                                  local_experts, recv_routes, zero_weights, acts_scratch, out_rows, d, f, recv_row_stride_elements, nullptr);
}

}  // extern "C"

namespace tf {

// tf_ep_experts_tensorcore for rows of `recv_row_stride_elements` (> d: the ids sit in the row tails, empty slots carry
// UINT32_MAX and are skipped) whose first kernel may have to wait for the peers that write them.
tf_status ep_experts_tensorcore_waiting(tf_context* ctx, void* stream, const void* pool_layer_base, uint64_t expert_stride,
                                        const tf_expert_offsets* offsets, const void* recv_rows, const uint32_t* recv_expert_ids,
                                        uint32_t recv_slots, uint32_t local_experts, const tf_device_routes* recv_routes,
                                        const void* zero_weights, const void* one_weights, void* x_sorted, uint32_t* row_ids,
                                        uint32_t* inverse_perm, void* acts_scratch, void* out_sorted, void* out_rows,
                                        uint32_t d, uint32_t f, uint32_t recv_row_stride_elements, const PeerWait* peer_wait) {
    const char* name = "tf_ep_experts_tensorcore";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, pool_layer_base && offsets && recv_rows && recv_expert_ids && recv_routes && zero_weights && one_weights &&
                        x_sorted && row_ids && inverse_perm && acts_scratch && out_sorted && out_rows,
               TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    if (recv_slots == 0) return TF_OK;
    // group the received rows by local expert, gather them into expert order, run the tcgen05 GEMMs, and put the
    // results back into slot order (a combine with one rank of weight 1.0 is an exact copy through the permutation)
    const uint32_t stride = recv_row_stride_elements ? recv_row_stride_elements : d;
    tf_status s;
    if (stride > d) {
        TF_REQUIRE(ctx, d % 2 == 0 && stride % 2 == 0 && tf::aligned(recv_rows, 4), TF_ERR_ALIGNMENT, "%s: rows must be 4-byte aligned", name);
        s = tf::group_routes_strided(ctx, stream, reinterpret_cast<const uint32_t*>(static_cast<const uint16_t*>(recv_rows) + d), stride / 2,
                                     const_cast<uint32_t*>(recv_expert_ids), zero_weights, recv_slots, 1, local_experts, recv_routes, name,
                                     peer_wait);
    } else {
        s = tf::group_routes_strided(ctx, stream, recv_expert_ids, 1, nullptr, zero_weights, recv_slots, 1, local_experts, recv_routes,
                                     name, peer_wait);
    }
    if (s) return s;
    // only the grouped pairs are gathered (the gather stops at the count the grouping left on the device); the slots that
    // were empty keep whatever inverse_perm held before, which points inside out_sorted, and nobody reads their results
    s = tf_pack_sorted_rows(ctx, stream, recv_rows, stride, recv_routes, recv_slots, 1, local_experts, d, x_sorted, row_ids, inverse_perm);
    if (s) return s;
    s = tf_grouped_moe_tensorcore(ctx, stream, x_sorted, recv_slots, pool_layer_base, expert_stride, local_experts, offsets,
                                  recv_routes, acts_scratch, out_sorted, d, f);
    if (s) return s;
    // back into slot order; with id tails (a fixed-capacity buffer) the empty slots are left alone
    return tf::ep_combine_waiting(ctx, stream, out_sorted, one_weights, inverse_perm, nullptr, d, out_rows, d, recv_slots, 1, d, nullptr,
                                  stride > d ? recv_expert_ids : nullptr);
}

}  // namespace tf

extern "C" {

tf_status tf_ep_experts_tensorcore(tf_context* ctx, void* stream, const void* pool_layer_base, uint64_t expert_stride,
                                   const tf_expert_offsets* offsets, const void* recv_rows, const uint32_t* recv_expert_ids,
                                   uint32_t recv_slots, uint32_t local_experts, const tf_device_routes* recv_routes,
                                   const void* zero_weights, const void* one_weights, void* x_sorted, uint32_t* row_ids,
                                   uint32_t* inverse_perm, void* acts_scratch, void* out_sorted, void* out_rows,
                                   uint32_t d, uint32_t f) {
    return tf::ep_experts_tensorcore_waiting(ctx, stream, pool_layer_base, expert_stride, offsets, recv_rows, recv_expert_ids, recv_slots,
                                             local_experts, recv_routes, zero_weights, one_weights, x_sorted, row_ids, inverse_perm,
                                             acts_scratch, out_sorted, out_rows, d, f, 0, nullptr);
}

tf_status tf_ep_finish(tf_context* ctx, void* stream, const tf_moe_layer* layer, const void* x, uint32_t tokens,
                       tf_workspace* ws, const void* returned_rows, const uint32_t* inverse_perm, void* y) {
    const char* name = "tf_ep_finish";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, layer && x && ws && returned_rows && inverse_perm && y, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    if (tokens == 0) return TF_OK;
    const uint32_t d = layer->d;
    tf_status s = layer->shared_bits == 8
                      ? tf_shared_expert_int8_block(ctx, stream, x, 0, d, &layer->shared_gate, &layer->shared_up, &layer->shared_down,
                                                    ws->shared_y, 0, d, ws->shared_act, tokens)
                      : tf_shared_expert_int4_block(ctx, stream, x, 0, d, &layer->shared_gate, &layer->shared_up, &layer->shared_down,
                                                    ws->shared_y, 0, d, ws->shared_act, tokens);
    if (s) return s;
    return tf_ep_combine(ctx, stream, returned_rows, ws->weights, inverse_perm, ws->shared_y, d, y, d, tokens, layer->top_k, d);
}

tf_status tf_stack_create(tf_context* ctx, const tf_moe_layer* layers, const void* const* norm_weights_bf16,
                          uint32_t layer_count, float eps, tf_stack** out) {
    const char* name = "tf_stack_create";
    TF_REQUIRE(ctx, ctx != nullptr && out != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    *out = nullptr;
    TF_REQUIRE(ctx, layers && norm_weights_bf16 && layer_count > 0, TF_ERR_INVALID_ARGUMENT, "%s: no layers", name);
    tf_stack* st = new tf_stack();
    st->ctx = ctx;
    st->eps = eps;
    st->layers.assign(layers, layers + layer_count);
    st->norm_weights.assign(norm_weights_bf16, norm_weights_bf16 + layer_count);
    if (tf_status s = tf::decode_step_prepare(ctx, st)) { delete st; return s; }
    *out = st;
    return TF_OK;
}

void tf_stack_destroy(tf_stack* st) {
    if (!st) return;
    if (st->device_layers) cudaFree(st->device_layers);
    delete st;
}

// hidden [tokens, d] fp16, contiguous, updated in place:
//   for each layer: x = rmsnorm(h) * w_l;  h = h + block_l(x)
// (the residual add of layer l is fused into the norm of layer l+1; a final add closes the stack).
tf_status tf_stack_forward(tf_stack* st, void* stream, void* hidden, uint32_t tokens, tf_workspace* ws) {
    const char* name = "tf_stack_forward";
    TF_REQUIRE(nullptr, st != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: stack is NULL", name);
    tf_context* ctx = st->ctx;
    TF_REQUIRE(ctx, hidden && ws, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, tokens <= ws->max_tokens, TF_ERR_SCRATCH_TOO_SMALL, "%s: %u tokens exceed the workspace (%u)", name, tokens, ws->max_tokens);
    if (tokens == 0) return TF_OK;
    const uint32_t d = ws->d;
    const size_t smem = 0;
    TF_REQUIRE(ctx, d % 8 == 0 && d <= 8u * tf::kRrnThreads * tf::kRrnMaxSlices, TF_ERR_UNSUPPORTED,
               "%s: D must be a multiple of 8 and at most %d", name, 8 * tf::kRrnThreads * tf::kRrnMaxSlices);
    TF_REQUIRE(ctx, tf::aligned(hidden, 16), TF_ERR_ALIGNMENT, "%s: hidden must be 16-byte aligned", name);
    // one token: the whole step is one persistent launch (decode_step.cu)
    if (tokens == 1 && ctx->single_launch_step && tf::decode_step_eligible(st, ws)) return tf::launch_decode_step(ctx, stream, st, hidden, ws);
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    uint16_t* h = static_cast<uint16_t*>(hidden);
    // Decode-sized steps: the weighted sum of a layer's route partials, the residual add and the next norm are one
    // launch (combine_residual_rmsnorm_kernel; the values of the separate reduce and norm launches, two launches less).
    const bool fold = !st->layers.empty() && tf::block_keeps_f32_partials(ctx, ws, tokens) && st->layers[0].top_k <= TF_MAX_TOP_K &&
                      tf::aligned(ws->partials, 16) && tf::aligned(ws->shared_y, 16);
    uint32_t fold_threads = ((d / 8 + 31) / 32) * 32;          // one thread per eight columns,
    if (fold_threads < (uint32_t)tf::kRrnThreads) fold_threads = tf::kRrnThreads;      // at least the norm's 128 (its reduction tree)
    const uint16_t* no16 = nullptr;
    const uint32_t* no32u = nullptr;
    uint16_t* no_x = nullptr;
    const tf::PeerWait no_wait{nullptr, nullptr, nullptr, 0u};
    for (size_t l = 0; l < st->layers.size(); ++l) {
        const uint16_t* nw = static_cast<const uint16_t*>(st->norm_weights[l]);
        if (l > 0 && fold)
            tf::launch_pdl(tf::combine_residual_rmsnorm_kernel<false>, dim3(tokens), dim3(fold_threads), smem, cs, h,
                           static_cast<const void*>(ws->partials), static_cast<const uint16_t*>(ws->weights), no32u,
                           static_cast<const uint16_t*>(ws->shared_y), nw, ws->x_norm, d, st->layers[l - 1].top_k, st->eps, no_wait);
        else
            tf::launch_pdl(tf::residual_rmsnorm_kernel, dim3(tokens), dim3(tf::kRrnThreads), smem, cs, h,
                           l == 0 ? no16 : static_cast<const uint16_t*>(ws->y_block), nw, ws->x_norm, d, st->eps);
        if (tf_status s = tf::check_launch(ctx, "residual_rmsnorm")) return s;
        if (tf_status s = tf::block_forward(ctx, stream, &st->layers[l], ws->x_norm, d, fold ? nullptr : ws->y_block, d, tokens, ws)) return s;
    }
    if (fold)
        tf::launch_pdl(tf::combine_residual_rmsnorm_kernel<false>, dim3(tokens), dim3(fold_threads), smem, cs, h,
                       static_cast<const void*>(ws->partials), static_cast<const uint16_t*>(ws->weights), no32u,
                       static_cast<const uint16_t*>(ws->shared_y), no16, no_x, d, st->layers.back().top_k, st->eps, no_wait);
    else
        tf::launch_pdl(tf::residual_rmsnorm_kernel, dim3(tokens), dim3(tf::kRrnThreads), smem, cs, h,
                       static_cast<const uint16_t*>(ws->y_block), no16, no_x, d, st->eps);
    return tf::check_launch(ctx, "residual_add");
}

}  // extern "C"
