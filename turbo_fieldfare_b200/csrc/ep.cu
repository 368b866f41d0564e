// Expert-parallel dispatch and combine: the data movement either side of the all-to-all.
//
// The reference has no multi-GPU path (one MTLDevice, one queue:
// Infrastructure/Metal/MetalContext.swift:51-71). With experts sharded 128/N per GPU, a layer is
//   route locally -> pack rows by destination rank (this file) -> all-to-all -> grouped experts on
//   the owner (grouped.cu) -> all-to-all back -> weighted combine in rank order (this file).
// The pack kernel gathers each pair's activation row straight into the send buffer in
// (destination, expert, token, rank) order, which is the order the device grouping already produced,
// and records where each (token, rank) went; the combine kernel gathers the returned rows through
// that record, so no row is copied twice and the summation order is fixed (rank 0..K-1).
#include "block.cuh"
#include "peer.cuh"

namespace tf {

constexpr int kPackThreads = 256;

// One warp per send slot. Fixed-capacity mode: slot = dst * capacity + pos. Exact mode (n_dst == 1):
// slot = sorted pair index. PERMUTE_K8 stores every eight columns in the order (0,4,1,5,2,6,3,7), the
// activation layout of the tensor-core grouped GEMM.
template <bool PERMUTE_K8>
__global__ void __launch_bounds__(kPackThreads)
ep_pack_kernel(const uint16_t* __restrict__ hidden, uint32_t hidden_stride, const tf_pair* __restrict__ sorted_pairs,
               const uint32_t* __restrict__ per_expert_counts, uint32_t n_pairs, uint32_t top_k, uint32_t num_experts,
               uint32_t experts_per_rank, uint32_t n_dst, uint32_t capacity, uint32_t d, uint32_t send_stride,
               uint16_t* __restrict__ send_rows, uint32_t* __restrict__ send_ids, uint32_t* __restrict__ inverse_perm,
               uint32_t* __restrict__ overflow, const uint32_t* __restrict__ grouped_pairs) {
    __shared__ uint32_t dst_base[257], dst_count[256];
    if (n_dst > 1) {
        // pairs are sorted by expert, experts are contiguous per rank: dst_base = prefix of the counts
        if (threadIdx.x == 0) {
            uint32_t run = 0;
            for (uint32_t r = 0; r < n_dst; ++r) {
                dst_base[r] = run;
                uint32_t c = 0;
                for (uint32_t e = r * experts_per_rank; e < (r + 1) * experts_per_rank && e < num_experts; ++e) c += per_expert_counts[e];
                dst_count[r] = c;
                run += c;
                if (c > capacity && blockIdx.x == 0) atomicMax(overflow, c);
            }
        }
        __syncthreads();
    }
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t slot = blockIdx.x * (kPackThreads / kWarp) + warp;
    const uint32_t slots = n_dst > 1 ? n_dst * capacity : n_pairs;
    if (slot >= slots) return;
    uint32_t p;
    if (n_dst > 1) {
        const uint32_t dst = slot / capacity, pos = slot % capacity;
        if (pos >= dst_count[dst]) {
            if (lane == 0) {
                send_ids[slot] = 0xFFFFFFFFu;
                if (send_stride > d) *reinterpret_cast<uint32_t*>(send_rows + (size_t)slot * send_stride + d) = 0xFFFFFFFFu;
            }
            return;
        }
        p = dst_base[dst] + pos;
    } else {
        p = slot;
        if (p >= *grouped_pairs) return;      // routes built from an exchange buffer with empty slots hold fewer pairs
    }
    const tf_pair pr = sorted_pairs[p];
    if (lane == 0) {
        send_ids[slot] = pr.expert % experts_per_rank;
        // rows wider than d carry the local expert id in their tail, so one exchange moves rows and ids
        if (send_stride > d) *reinterpret_cast<uint32_t*>(send_rows + (size_t)slot * send_stride + d) = pr.expert % experts_per_rank;
        inverse_perm[pr.token * top_k + pr.rank] = slot;
    }
    const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)pr.token * hidden_stride);
    uint4* dst_row = reinterpret_cast<uint4*>(send_rows + (size_t)slot * send_stride);
    for (uint32_t i = lane; i < d / 8; i += kWarp) {
        uint4 v = __ldg(src + i);
        if (PERMUTE_K8) {
            uint4 o;
            asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(o.x) : "r"(v.x), "r"(v.z));   // (k0, k4)
            asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(o.y) : "r"(v.x), "r"(v.z));   // (k1, k5)
            asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(o.z) : "r"(v.y), "r"(v.w));   // (k2, k6)
            asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(o.w) : "r"(v.y), "r"(v.w));   // (k3, k7)
            v = o;
        }
        dst_row[i] = v;
    }
}

// ids[slot] = the id a row of `stride` > d elements carries in its tail (see ep_pack_kernel).
__global__ void ep_extract_ids_kernel(const uint16_t* __restrict__ rows, uint32_t stride, uint32_t d, uint32_t slots,
                                      uint32_t* __restrict__ ids) {
    const uint32_t slot = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (slot < slots) ids[slot] = *reinterpret_cast<const uint32_t*>(rows + (size_t)slot * stride + d);
}

// y[t,d] = half(sum_r fma(w[t,r], partial[inverse[t*K+r]][d], acc) + residual[t,d]), rank order.
// VEC: a thread owns eight consecutive columns (16-byte loads and stores; D a multiple of 8, rows 16-byte aligned).
template <bool VEC>
__global__ void ep_combine_kernel(const uint16_t* __restrict__ rows, const uint16_t* __restrict__ weights,
                                  const uint32_t* __restrict__ inverse_perm, const uint16_t* __restrict__ residual,
                                  uint32_t residual_stride, uint16_t* __restrict__ out, uint32_t out_stride,
                                  uint32_t T, uint32_t K, uint32_t D, const PeerWait peer_wait, const uint32_t* __restrict__ skip_ids) {
    peer_wait_in_block(peer_wait);      // the rows may come from peers that are still writing them
    // rows in grid.x (up to 2^31 - 1 blocks), column blocks in grid.y: an expert-parallel rank can hold more than 65535 rows
    const uint32_t t = blockIdx.x;
    if (t >= T) return;
    if (skip_ids && skip_ids[t] == 0xFFFFFFFFu) return;      // an empty slot of a fixed-capacity exchange buffer
    if constexpr (VEC) {
        const uint32_t c = blockIdx.y * blockDim.x + threadIdx.x;          // group of eight columns
        if (c >= D / 8) return;
        float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t r0 = 0; r0 < K; r0 += 4) {
            // up to four ranks' rows are requested before the first one is used
            uint4 v[4];
            float w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t r = r0 + j;
                if (r < K) {
                    const uint32_t slot = inverse_perm[(size_t)t * K + r];
                    w[j] = f16_bits_to_float(weights[(size_t)t * K + r]);
                    v[j] = *reinterpret_cast<const uint4*>(rows + (size_t)slot * D + c * 8);
                } else {
                    w[j] = 0.0f; v[j] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (r0 + j < K) {
                    const uint32_t xw[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        acc[2 * q] = fmaf(w[j], f16_bits_to_float((uint16_t)(xw[q] & 0xFFFFu)), acc[2 * q]);
                        acc[2 * q + 1] = fmaf(w[j], f16_bits_to_float((uint16_t)(xw[q] >> 16)), acc[2 * q + 1]);
                    }
                }
            }
        }
        if (residual) {
            const uint4 rv = *reinterpret_cast<const uint4*>(residual + (size_t)t * residual_stride + c * 8);
            const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                acc[2 * q] += f16_bits_to_float((uint16_t)(rw[q] & 0xFFFFu));
                acc[2 * q + 1] += f16_bits_to_float((uint16_t)(rw[q] >> 16));
            }
        }
        uint32_t ow[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const __half2 h = __floats2half2_rn(acc[2 * q], acc[2 * q + 1]);
            ow[q] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(out + (size_t)t * out_stride + c * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    } else {
        const uint32_t d = blockIdx.y * blockDim.x + threadIdx.x;
        if (d >= D) return;
        float acc = 0.0f;
        for (uint32_t r = 0; r < K; ++r) {
            const uint32_t slot = inverse_perm[(size_t)t * K + r];
            acc = fmaf(f16_bits_to_float(weights[(size_t)t * K + r]), f16_bits_to_float(rows[(size_t)slot * D + d]), acc);
        }
        if (residual) acc += f16_bits_to_float(residual[(size_t)t * residual_stride + d]);
        out[(size_t)t * out_stride + d] = __half_as_ushort(__float2half_rn(acc));
    }
}

}  // namespace tf

extern "C" {

static tf_status pack_rows(tf_context* ctx, void* stream, const void* hidden, uint64_t hidden_off, uint32_t hidden_stride_elements,
                           const tf_device_routes* routes, uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                           uint32_t experts_per_rank, uint32_t capacity, uint32_t d, uint32_t send_stride,
                           void* send_rows, uint32_t* send_expert_ids, uint32_t* inverse_perm, bool permute_k8, const char* name) {
    if (send_stride == 0) send_stride = d;
    TF_REQUIRE(ctx, send_stride == d || (send_stride >= d + 8 && send_stride % 8 == 0), TF_ERR_INVALID_ARGUMENT,
               "%s: the send row stride must be D, or at least D + 8 and a multiple of 8 elements (the id sits in the tail)", name);
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, hidden && routes && routes->counters && send_rows && send_expert_ids && inverse_perm, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, experts_per_rank > 0 && num_experts % experts_per_rank == 0 && num_experts <= TF_MAX_ROUTER_EXPERTS,
               TF_ERR_INVALID_ARGUMENT, "%s: experts (%u) must divide evenly over ranks (%u per rank)", name, num_experts, experts_per_rank);
    TF_REQUIRE(ctx, d % 8 == 0 && hidden_stride_elements >= d, TF_ERR_INVALID_ARGUMENT, "%s: D must be a multiple of 8", name);
    const uint8_t* hp = tf::byte_ptr(hidden, hidden_off);
    TF_REQUIRE(ctx, tf::aligned(hp, 16) && (hidden_stride_elements * 2) % 16 == 0 && tf::aligned(send_rows, 16), TF_ERR_ALIGNMENT,
               "%s: rows must be 16-byte aligned", name);
    const uint32_t n_pairs = query_count * top_k;
    if (n_pairs == 0) return TF_OK;
    const uint32_t n_dst = capacity > 0 ? num_experts / experts_per_rank : 1;
    const uint32_t slots = capacity > 0 ? n_dst * capacity : n_pairs;
    const uint32_t per_block = tf::kPackThreads / tf::kWarp;
    auto kern = permute_k8 ? tf::ep_pack_kernel<true> : tf::ep_pack_kernel<false>;
    kern<<<(slots + per_block - 1) / per_block, tf::kPackThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint16_t*>(hp), hidden_stride_elements, routes->sorted_pairs, routes->per_expert_counts, n_pairs,
        top_k, num_experts, experts_per_rank, n_dst, capacity, d, send_stride, static_cast<uint16_t*>(send_rows), send_expert_ids,
        inverse_perm, ctx->device_error, routes->counters + 3);
    return tf::check_launch(ctx, name);
}

tf_status tf_ep_pack(tf_context* ctx, void* stream, const void* hidden, uint64_t hidden_off, uint32_t hidden_stride_elements,
                     const tf_device_routes* routes, uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                     uint32_t experts_per_rank, uint32_t capacity, uint32_t d,
                     void* send_rows, uint32_t* send_expert_ids, uint32_t* inverse_perm, uint32_t send_row_stride_elements) {
    return pack_rows(ctx, stream, hidden, hidden_off, hidden_stride_elements, routes, query_count, top_k, num_experts,
                     experts_per_rank, capacity, d, send_row_stride_elements, send_rows, send_expert_ids, inverse_perm, false, "tf_ep_pack");
}

tf_status tf_ep_extract_ids(tf_context* ctx, void* stream, const void* rows, uint32_t row_stride_elements, uint32_t d,
                            uint32_t slots, uint32_t* ids) {
    const char* name = "tf_ep_extract_ids";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, rows && ids, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, row_stride_elements >= d + 2 && d % 2 == 0 && row_stride_elements % 2 == 0 && tf::aligned(rows, 4), TF_ERR_INVALID_ARGUMENT,
               "%s: rows must be wider than D and 4-byte aligned", name);
    if (slots == 0) return TF_OK;
    tf::launch_pdl(tf::ep_extract_ids_kernel, dim3((slots + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream),
                   static_cast<const uint16_t*>(rows), row_stride_elements, d, slots, ids);
    return tf::check_launch(ctx, name);
}

tf_status tf_pack_sorted_rows(tf_context* ctx, void* stream, const void* hidden, uint32_t hidden_stride_elements,
                              const tf_device_routes* routes, uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                              uint32_t d, void* x_sorted, uint32_t* row_expert_ids, uint32_t* inverse_perm) {
    return pack_rows(ctx, stream, hidden, 0, hidden_stride_elements, routes, query_count, top_k, num_experts, num_experts, 0, d, d,
                     x_sorted, row_expert_ids, inverse_perm, true, "tf_pack_sorted_rows");
}

}  // extern "C"

namespace tf {

tf_status ep_combine_waiting(tf_context* ctx, void* stream, const void* returned_rows, const void* route_weights,
                             const uint32_t* inverse_perm, const void* residual, uint32_t residual_stride_elements,
                             void* out, uint32_t out_stride_elements, uint32_t query_count, uint32_t top_k, uint32_t d,
                             const PeerWait* peer_wait, const uint32_t* skip_ids) {
    const char* name = "tf_ep_combine";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, returned_rows && route_weights && inverse_perm && out, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, top_k > 0 && d > 0 && out_stride_elements >= d, TF_ERR_INVALID_ARGUMENT, "%s: bad dimensions", name);
    if (query_count == 0) return TF_OK;
    const PeerWait pw = peer_wait ? *peer_wait : PeerWait{nullptr, nullptr, nullptr, 0u};
    const bool vec = d % 8 == 0 && out_stride_elements % 8 == 0 && tf::aligned(returned_rows, 16) && tf::aligned(out, 16) &&
                     (!residual || (residual_stride_elements % 8 == 0 && tf::aligned(residual, 16)));
    if (vec) {
        uint32_t threads = (d / 8 + 31) / 32 * 32;          // one block per row up to 4096 columns
        if (threads > 512) threads = 512;
        dim3 grid(query_count, (d / 8 + threads - 1) / threads);
        tf::ep_combine_kernel<true><<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint16_t*>(returned_rows), static_cast<const uint16_t*>(route_weights), inverse_perm,
            static_cast<const uint16_t*>(residual), residual_stride_elements, static_cast<uint16_t*>(out), out_stride_elements,
            query_count, top_k, d, pw, skip_ids);
    } else {
        dim3 grid(query_count, (d + 255) / 256);
        tf::ep_combine_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint16_t*>(returned_rows), static_cast<const uint16_t*>(route_weights), inverse_perm,
            static_cast<const uint16_t*>(residual), residual_stride_elements, static_cast<uint16_t*>(out), out_stride_elements,
            query_count, top_k, d, pw, skip_ids);
    }
    return tf::check_launch(ctx, name);
}

}  // namespace tf

extern "C" {

tf_status tf_ep_combine(tf_context* ctx, void* stream, const void* returned_rows, const void* route_weights,
                        const uint32_t* inverse_perm, const void* residual, uint32_t residual_stride_elements,
                        void* out, uint32_t out_stride_elements, uint32_t query_count, uint32_t top_k, uint32_t d) {
    return tf::ep_combine_waiting(ctx, stream, returned_rows, route_weights, inverse_perm, residual, residual_stride_elements, out,
                                  out_stride_elements, query_count, top_k, d, nullptr, nullptr);
}

}  // extern "C"
