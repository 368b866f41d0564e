// Decode (one token) routed and shared expert kernels.
// Replaces moe_phase1_gate_up_act[_subset]_u16load, moe_phase2_down_reduce_k8
// (Metal/MoE/moe.metal:248-482) and gelu_mul_fp16 (Metal/Primitives/utility.metal:7-18).
// Expert blobs are addressed through a DEVICE table of base pointers plus the
// nine shared byte offsets, as the reference's argument buffer does
// (moe.metal:62-76); the table is filled on the device from the router's ids,
// so no id ever crosses to the host.
#include "rowdot.cuh"

namespace tf {

constexpr int kP1Threads = 256;
constexpr int kP1Warps = kP1Threads / kWarp;
constexpr int kP1RowsPerWarp = 2;
constexpr int kP1RowsPerBlock = kP1Warps * kP1RowsPerWarp;

// grid (ceil(F / rows_per_block), slots). slot_map == nullptr: slot = blockIdx.y.
__global__ void __launch_bounds__(kP1Threads)
moe_phase1_kernel(const uint8_t* const* __restrict__ blobs, tf_expert_offsets off,
                  const uint16_t* __restrict__ x, uint16_t* __restrict__ acts,
                  uint32_t d, uint32_t f, uint32_t top_k, const uint32_t* __restrict__ slot_map) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint16_t* xs = reinterpret_cast<uint16_t*>(smem);
    float* xsum16 = xsum_ptr(xs, (int)d);
    uint32_t slot = blockIdx.y;
    if (slot_map) {
        slot = slot_map[blockIdx.y];
        if (slot >= top_k) return;      // moe.metal:399 (uniform per block: safe before the barrier)
    }
    stage_x<false>(x, xs, xsum16, (int)d);

    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint8_t* base = blobs[slot];
    const uint32_t groups = d / kGroup;
    const size_t row_bytes = d / 2;
#pragma unroll
    for (int r = 0; r < kP1RowsPerWarp; ++r) {
        const uint32_t row = blockIdx.x * kP1RowsPerBlock + warp * kP1RowsPerWarp + r;
        if (row >= f) break;
        const float2 gu = int4_row2_partial_a16<false>(
            base + off.gate_w_off + row * row_bytes,
            reinterpret_cast<const uint16_t*>(base + off.gate_s_off) + (size_t)row * groups,
            reinterpret_cast<const uint16_t*>(base + off.gate_b_off) + (size_t)row * groups,
            base + off.up_w_off + row * row_bytes,
            reinterpret_cast<const uint16_t*>(base + off.up_s_off) + (size_t)row * groups,
            reinterpret_cast<const uint16_t*>(base + off.up_b_off) + (size_t)row * groups,
            xs, xsum16, (int)d, lane);
        const float g = warp_sum(gu.x), u = warp_sum(gu.y);
        if (lane == 0) acts[(size_t)slot * f + row] = __half_as_ushort(__float2half_rn(gelu_tanh(g) * u));
    }
}

constexpr int kP2Threads = 256;
constexpr int kP2RowsPerBlock = 8;

// Each block owns kP2RowsPerBlock output rows. Warp w computes slot (w % top_k)
// style work items: item = (row_in_block, slot), items strided over the warps.
// Partials land in shared memory and are summed in slot order 0..top_k-1
// (moe.metal:473-480).
__global__ void __launch_bounds__(kP2Threads)
moe_phase2_kernel(const uint8_t* const* __restrict__ blobs, tf_expert_offsets off,
                  const uint16_t* __restrict__ acts, const uint16_t* __restrict__ routing_w,
                  const uint16_t* __restrict__ residual, uint16_t* __restrict__ y,
                  uint32_t d, uint32_t f, uint32_t top_k) {
    extern __shared__ __align__(16) uint8_t smem[];
    // layout: per slot [acts (f * 2 B padded to 16) | xsum16 (f/16 floats)], then partials
    const size_t slot_bytes = stage_x_bytes((int)f);
    float* partial = reinterpret_cast<float*>(smem + slot_bytes * top_k);   // [rows_per_block][top_k]
    for (uint32_t s = 0; s < top_k; ++s) {
        uint16_t* xs = reinterpret_cast<uint16_t*>(smem + slot_bytes * s);
        for (uint32_t i = threadIdx.x; i < f; i += blockDim.x) xs[i] = acts[(size_t)s * f + i];
    }
    __syncthreads();
    for (uint32_t c = threadIdx.x; c < top_k * (f >> 4); c += blockDim.x) {
        const uint32_t s = c / (f >> 4), cc = c % (f >> 4);
        uint16_t* xs = reinterpret_cast<uint16_t*>(smem + slot_bytes * s);
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) sum += f16_bits_to_float(xs[cc * 16 + j]);
        xsum_ptr(xs, (int)f)[cc] = sum;
    }
    __syncthreads();

    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t groups = f / kGroup;
    const size_t row_bytes = f / 2;
    const uint32_t items = kP2RowsPerBlock * top_k;
    for (uint32_t it = warp; it < items; it += kP2Threads / kWarp) {
        const uint32_t r = it / top_k, s = it % top_k;
        const uint32_t row = blockIdx.x * kP2RowsPerBlock + r;
        if (row >= d) continue;
        const uint8_t* base = blobs[s];
        uint16_t* xs = reinterpret_cast<uint16_t*>(smem + slot_bytes * s);
        float acc = int4_row_partial_a16<false, false>(
            base + off.down_w_off + row * row_bytes,
            reinterpret_cast<const uint16_t*>(base + off.down_s_off) + (size_t)row * groups,
            reinterpret_cast<const uint16_t*>(base + off.down_b_off) + (size_t)row * groups,
            xs, xsum_ptr(xs, (int)f), (int)f, lane);
        acc = warp_sum(acc);
        if (lane == 0) partial[r * top_k + s] = f16_bits_to_float(routing_w[s]) * acc;
    }
    __syncthreads();
    if (threadIdx.x < kP2RowsPerBlock) {
        const uint32_t row = blockIdx.x * kP2RowsPerBlock + threadIdx.x;
        if (row < d) {
            float acc = residual ? f16_bits_to_float(residual[row]) : 0.0f;
            for (uint32_t s = 0; s < top_k; ++s) acc += partial[threadIdx.x * top_k + s];
            y[row] = __half_as_ushort(__float2half_rn(acc));
        }
    }
}

__global__ void expert_table_kernel(const uint8_t* base, uint64_t stride, const uint32_t* __restrict__ indices,
                                    uint32_t count, uint32_t num_experts, const void** out) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    uint32_t e = indices[i];
    if (e >= num_experts) e = num_experts - 1;   // min(id, E-1): Runtime/Inference/RealForwardRunner.swift:955,1486
    out[i] = base + (uint64_t)e * stride;
}

__global__ void gelu_mul_kernel(const uint16_t* __restrict__ gate, const uint16_t* __restrict__ up,
                                uint16_t* __restrict__ out, uint32_t count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float g = f16_bits_to_float(gate[i]), u = f16_bits_to_float(up[i]);
    out[i] = __half_as_ushort(__float2half_rn(gelu_tanh(g) * u));
}

static tf_status check_offsets(tf_context* ctx, const tf_expert_offsets* o, const char* name) {
    TF_REQUIRE(ctx, o != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: offsets is NULL", name);
    const uint32_t w[3] = {o->gate_w_off, o->up_w_off, o->down_w_off};
    for (uint32_t v : w)
        TF_REQUIRE(ctx, v % 16 == 0, TF_ERR_ALIGNMENT,
                   "%s: packed sub-tensor offset %u is not 16-byte aligned (the .gturbo blob layout gives 16-byte multiples)", name, v);
    const uint32_t s[6] = {o->gate_s_off, o->gate_b_off, o->up_s_off, o->up_b_off, o->down_s_off, o->down_b_off};
    for (uint32_t v : s)
        TF_REQUIRE(ctx, v % 2 == 0, TF_ERR_ALIGNMENT, "%s: scale/bias offset %u must be even", name, v);
    return TF_OK;
}

static tf_status launch_phase1(tf_context* ctx, void* stream, const void* const* blobs, const tf_expert_offsets* offsets,
                               const void* x, void* acts, uint32_t d, uint32_t f, uint32_t top_k,
                               const uint32_t* slot_map, uint32_t slots, const char* name) {
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, blobs && x && acts, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    if (tf_status s = check_offsets(ctx, offsets, name)) return s;
    TF_REQUIRE(ctx, d > 0 && d % kGroup == 0 && f > 0, TF_ERR_INVALID_ARGUMENT, "%s: D must be a positive multiple of 64, F positive", name);
    TF_REQUIRE(ctx, top_k > 0 && top_k <= TF_MAX_TOP_K, TF_ERR_INVALID_ARGUMENT, "%s: topK must be in 1...8", name);
    TF_REQUIRE(ctx, (d / 2) % 16 == 0, TF_ERR_UNSUPPORTED, "%s: D/2 must be a multiple of 16 bytes", name);
    TF_REQUIRE(ctx, aligned(x, 2) && aligned(acts, 2), TF_ERR_ALIGNMENT, "%s: x/acts must be 2-byte aligned", name);
    if (slots == 0) return TF_OK;
    const size_t smem = stage_x_bytes((int)d);
    TF_REQUIRE(ctx, smem <= 96 * 1024, TF_ERR_UNSUPPORTED, "%s: D too large", name);
    if (smem > 48 * 1024)
        TF_CUDA(ctx, cudaFuncSetAttribute(moe_phase1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((f + kP1RowsPerBlock - 1) / kP1RowsPerBlock, slots);
    moe_phase1_kernel<<<grid, kP1Threads, smem, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint8_t* const*>(blobs), *offsets, static_cast<const uint16_t*>(x),
        static_cast<uint16_t*>(acts), d, f, top_k, slot_map);
    return check_launch(ctx, name);
}

}  // namespace tf

extern "C" {

tf_status tf_moe_phase1(tf_context* ctx, void* stream, const void* const* blobs, const tf_expert_offsets* offsets,
                        const void* x, void* acts, uint32_t d, uint32_t f, uint32_t top_k) {
    return tf::launch_phase1(ctx, stream, blobs, offsets, x, acts, d, f, top_k, nullptr, top_k, "tf_moe_phase1");
}

tf_status tf_moe_phase1_subset(tf_context* ctx, void* stream, const void* const* blobs, const tf_expert_offsets* offsets,
                               const void* x, void* acts, uint32_t d, uint32_t f, uint32_t top_k,
                               const uint32_t* active_slots, uint32_t active_count) {
    TF_REQUIRE(ctx, active_count == 0 || active_slots != nullptr, TF_ERR_INVALID_ARGUMENT,
               "tf_moe_phase1_subset: active_slots is NULL");
    TF_REQUIRE(ctx, active_count <= top_k, TF_ERR_INVALID_ARGUMENT, "tf_moe_phase1_subset: activeCount > topK");
    return tf::launch_phase1(ctx, stream, blobs, offsets, x, acts, d, f, top_k, active_slots, active_count,
                             "tf_moe_phase1_subset");
}

tf_status tf_moe_phase2_reduce(tf_context* ctx, void* stream, const void* const* blobs, const tf_expert_offsets* offsets,
                               const void* acts, const void* routing_weights, const void* residual, void* y,
                               uint32_t d, uint32_t f, uint32_t top_k) {
    const char* name = "tf_moe_phase2_reduce";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, blobs && acts && routing_weights && y, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    if (tf_status s = tf::check_offsets(ctx, offsets, name)) return s;
    TF_REQUIRE(ctx, d > 0 && f > 0 && f % tf::kGroup == 0, TF_ERR_INVALID_ARGUMENT, "%s: F must be a positive multiple of 64", name);
    // moe.metal:446-482 is the k8 kernel; MoE.swift:297-300 traps on other values.
    TF_REQUIRE(ctx, top_k > 0 && top_k <= TF_MAX_TOP_K, TF_ERR_INVALID_ARGUMENT, "%s: topK must be in 1...8", name);
    TF_REQUIRE(ctx, (f / 2) % 16 == 0, TF_ERR_UNSUPPORTED, "%s: F/2 must be a multiple of 16 bytes", name);
    const size_t smem = tf::stage_x_bytes((int)f) * top_k + sizeof(float) * tf::kP2RowsPerBlock * top_k;
    TF_REQUIRE(ctx, smem <= 160 * 1024, TF_ERR_UNSUPPORTED, "%s: F too large", name);
    if (smem > 48 * 1024)
        TF_CUDA(ctx, cudaFuncSetAttribute(tf::moe_phase2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const uint32_t grid = (d + tf::kP2RowsPerBlock - 1) / tf::kP2RowsPerBlock;
    tf::moe_phase2_kernel<<<grid, tf::kP2Threads, smem, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint8_t* const*>(blobs), *offsets, static_cast<const uint16_t*>(acts),
        static_cast<const uint16_t*>(routing_weights), static_cast<const uint16_t*>(residual),
        static_cast<uint16_t*>(y), d, f, top_k);
    return tf::check_launch(ctx, name);
}

tf_status tf_expert_table_from_indices(tf_context* ctx, void* stream, const void* pool_layer_base, uint64_t expert_stride,
                                       const uint32_t* indices, uint32_t count, uint32_t num_experts,
                                       const void** blobs_out) {
    const char* name = "tf_expert_table_from_indices";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, pool_layer_base && indices && blobs_out, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, num_experts > 0, TF_ERR_INVALID_ARGUMENT, "%s: numExperts must be positive", name);
    TF_REQUIRE(ctx, expert_stride % 16 == 0 && tf::aligned(pool_layer_base, 16), TF_ERR_ALIGNMENT,
               "%s: pool base and stride must be 16-byte aligned", name);
    if (count == 0) return TF_OK;
    tf::expert_table_kernel<<<(count + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(pool_layer_base), expert_stride, indices, count, num_experts, blobs_out);
    return tf::check_launch(ctx, name);
}

tf_status tf_shared_expert_int4(tf_context* ctx, void* stream, const void* x, uint64_t x_off, uint64_t x_bytes,
                                const tf_projection* gate, const tf_projection* up, const tf_projection* down,
                                void* y, uint64_t y_off, uint64_t y_bytes,
                                void* scratch_gate, uint64_t scratch_gate_off, uint64_t scratch_gate_bytes,
                                void* scratch_up, uint64_t scratch_up_off, uint64_t scratch_up_bytes,
                                void* scratch_act, uint64_t scratch_act_off, uint64_t scratch_act_bytes) {
    const char* name = "tf_shared_expert_int4";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, x && gate && up && down && y && scratch_gate && scratch_up && scratch_act,
               TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    // SharedExpertInt4.swift:41-46
    TF_REQUIRE(ctx, gate->rows == up->rows && gate->cols == up->cols && down->rows == gate->cols && down->cols == gate->rows,
               TF_ERR_DIMENSION_MISMATCH, "SharedExpert dimension mismatch: gate=(%u,%u) up=(%u,%u) down=(%u,%u)",
               gate->rows, gate->cols, up->rows, up->cols, down->rows, down->cols);
    const uint64_t intermediate = gate->rows;
    const uint64_t required = intermediate * 2;
    // SharedExpertInt4.swift:47-53
    TF_REQUIRE(ctx, scratch_gate_off + required <= scratch_gate_bytes && scratch_up_off + required <= scratch_up_bytes &&
                        scratch_act_off + required <= scratch_act_bytes,
               TF_ERR_SCRATCH_TOO_SMALL, "SharedExpert scratch too small: need %llu bytes per intermediate buffer",
               (unsigned long long)required);
    // SharedExpertInt4.swift:54-61
    TF_REQUIRE(ctx, x_off + (uint64_t)gate->cols * 2 <= x_bytes, TF_ERR_SCRATCH_TOO_SMALL,
               "SharedExpert scratch too small: input range exceeds x buffer");
    TF_REQUIRE(ctx, y_off + (uint64_t)down->rows * 2 <= y_bytes, TF_ERR_SCRATCH_TOO_SMALL,
               "SharedExpert scratch too small: output range exceeds y buffer");

    tf_status s = tf_int4_gemv(ctx, stream, gate->weights, gate->weights_off, gate->scales, gate->scales_off,
                               gate->biases, gate->biases_off, x, x_off, scratch_gate, scratch_gate_off,
                               gate->rows, gate->cols, TF_BF16);
    if (s) return s;
    s = tf_int4_gemv(ctx, stream, up->weights, up->weights_off, up->scales, up->scales_off, up->biases, up->biases_off,
                     x, x_off, scratch_up, scratch_up_off, up->rows, up->cols, TF_BF16);
    if (s) return s;
    tf::gelu_mul_kernel<<<(uint32_t)((intermediate + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint16_t*>(tf::byte_ptr(scratch_gate, scratch_gate_off)),
        reinterpret_cast<const uint16_t*>(tf::byte_ptr(scratch_up, scratch_up_off)),
        reinterpret_cast<uint16_t*>(tf::byte_ptr(scratch_act, scratch_act_off)), (uint32_t)intermediate);
    s = tf::check_launch(ctx, "gelu_mul");
    if (s) return s;
    return tf_int4_gemv(ctx, stream, down->weights, down->weights_off, down->scales, down->scales_off,
                        down->biases, down->biases_off, scratch_act, scratch_act_off, y, y_off,
                        down->rows, down->cols, TF_BF16);
}

}  // extern "C"
