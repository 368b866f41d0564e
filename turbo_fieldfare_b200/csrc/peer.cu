// Expert-parallel exchange over peer memory (NVLink), for decode steps.
//
// The fixed-capacity exchange of a decode step is small (at most tokens x top_k rows per destination) and bound by
// the latency of a library collective per direction per layer. Here every rank owns one exchange buffer that its
// peers map (CUDA IPC); a rank stores the rows for expert owner r straight into r's receive area, and a flag
// barrier (one release store per peer, one bounded acquire wait per peer) orders the phases. Everything is plain
// kernels with plain peer loads and stores, so a whole decode step, exchange included, replays as one CUDA graph.
//
// Every wait is bounded: after kPeerSpinLimit polls the kernel records kErrPeerTimeout in the context's peer status
// word (its own word: codes of other kernels do not touch it) and returns; once that word is set, later barriers do
// not wait at all, so a missing rank costs one timeout. From that point on the ranks are no longer synchronised and
// every result is invalid until tf_device_status has reported and cleared the code.
// Ranks must run one process per GPU (kernels that wait on one another never share a GPU).
#include "peer.cuh"

#include <cstring>

namespace tf {

constexpr int kPeerPushThreads = 256;

// Flag barrier: thread r tells peer r "rank `me` reached epoch e" and waits until peer r has said the same here.
// The epoch lives on the device and advances by one per barrier, so a replayed graph needs no host value.
// Called by every thread of one block (at least `world` threads).
// WAIT = false publishes the epoch and returns: the wait is then the consumer kernel's (peer_wait_in_block).
template <bool WAIT>
__device__ __forceinline__ void peer_barrier_in_block(uint8_t* const* __restrict__ peers, uint64_t flags_offset_bytes,
                                                      uint32_t* __restrict__ epoch_counter, uint32_t* __restrict__ error,
                                                      uint32_t world, uint32_t me) {
    __shared__ uint32_t epoch;
    if (threadIdx.x == 0) {
        epoch = *epoch_counter + 1u;
        *epoch_counter = epoch;
        // One system-scope fence by the thread that saw every block's ticket: it orders all rows written before the
        // tickets (each block fenced before its own) ahead of the flag stores below, which follow it through the block barrier.
        __threadfence_system();
    }
    __syncthreads();
    const uint32_t r = threadIdx.x;
    if (r >= world) return;
    st_release_sys(reinterpret_cast<uint32_t*>(peers[r] + flags_offset_bytes) + me, epoch);
    if constexpr (WAIT) peer_wait_flag(reinterpret_cast<const uint32_t*>(peers[me] + flags_offset_bytes) + r, epoch, error);
}

// A warp copies nvec 16-byte pieces with eight loads per lane in flight before the first store (a row is a few
// hundred pieces: one load per trip would pay the memory latency a dozen times in a row).
__device__ __forceinline__ void warp_copy_u4(const uint4* __restrict__ in, uint4* __restrict__ out, uint32_t nvec, uint32_t lane) {
    for (uint32_t v0 = lane; v0 < nvec; v0 += kWarp * 8) {
        uint4 t[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const uint32_t v = v0 + q * kWarp;
            if (v < nvec) t[q] = in[v];
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const uint32_t v = v0 + q * kWarp;
            if (v < nvec) out[v] = t[q];
        }
    }
}

// One warp per slot (source rank block s, slot j). A slot is in use when its expert id is not 0xFFFFFFFF: the id is
// read from `ids` when given, else from the row's tail (element `tail_at`, as 32 bits). Used slots are copied
// (`copy_elems` fp16 elements, a multiple of 8) into peer s's buffer at block `me`; with tails, an unused slot gets
// only its tail written so that the receiver sees it as empty.
template <bool WAIT>
__global__ void __launch_bounds__(kPeerPushThreads)
ep_peer_push_kernel(const uint16_t* __restrict__ src, uint32_t src_stride, uint8_t* const* __restrict__ peers,
                    uint64_t dst_offset_bytes, uint32_t dst_stride, uint32_t copy_elems, const uint32_t* __restrict__ ids,
                    uint32_t tail_at, uint32_t world, uint32_t me, uint32_t cap,
                    uint64_t flags_offset_bytes, uint32_t* __restrict__ epoch_and_ticket, uint32_t* __restrict__ error) {
    const uint32_t warps_per_block = kPeerPushThreads / kWarp;
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t total = world * cap;
    for (uint32_t slot = blockIdx.x * warps_per_block + threadIdx.x / kWarp; slot < total; slot += gridDim.x * warps_per_block) {
        const uint32_t s = slot / cap, j = slot % cap;
        const uint16_t* row = src + (size_t)slot * src_stride;
        uint32_t id;
        if (ids) id = ids[slot];
        else id = *reinterpret_cast<const uint32_t*>(row + tail_at);
        uint16_t* dst = reinterpret_cast<uint16_t*>(peers[s] + dst_offset_bytes) + ((size_t)me * cap + j) * dst_stride;
        if (id != 0xFFFFFFFFu) {
            warp_copy_u4(reinterpret_cast<const uint4*>(row), reinterpret_cast<uint4*>(dst), copy_elems / 8, lane);
        } else if (!ids && lane == 0) {
            *reinterpret_cast<uint4*>(dst + tail_at) = *reinterpret_cast<const uint4*>(row + tail_at);
        }
    }
    // The block's rows are ordered before its ticket by ONE system-scope fence: the block barrier makes the fencing
    // thread the successor of every thread's stores, and a fence is cumulative over what its thread has synchronised with.
    __shared__ bool last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        if (epoch_and_ticket != nullptr) {
            // the block that finishes last runs the flag barrier (word 0: epoch, word 1: self-resetting ticket)
            const uint32_t tk = atomicAdd(&epoch_and_ticket[1], 1u);
            last = tk == gridDim.x - 1;
            if (last) epoch_and_ticket[1] = 0u;
        } else {
            last = false;
        }
    }
    __syncthreads();
    if (!last) return;
    peer_barrier_in_block<WAIT>(peers, flags_offset_bytes, epoch_and_ticket, error, world, me);
}

// Dispatch of a decode step in one launch: the rows of this rank's (token, rank) pairs go straight from the activation
// rows into the owners' receive areas (no local send buffer), in the slot order of ep_pack_kernel: destination r holds
// this rank's pairs for r's experts in (expert, token, rank) order from slot 0, unused slots get an empty id tail. The
// row's 16-byte tail carries the local expert id. inverse_perm[token * top_k + rank] = dst * capacity + position, the
// slot the result comes back in. The block that finishes last runs the flag barrier.
template <bool WAIT>
__global__ void __launch_bounds__(kPeerPushThreads)
ep_pack_push_kernel(const uint16_t* __restrict__ hidden, uint32_t hidden_stride, const tf_pair* __restrict__ sorted_pairs,
                    const uint32_t* __restrict__ per_expert_counts, uint32_t top_k, uint32_t num_experts, uint32_t experts_per_rank,
                    uint32_t d, uint32_t dst_stride, uint8_t* const* __restrict__ peers, uint64_t dst_offset_bytes,
                    uint32_t* __restrict__ inverse_perm, uint32_t world, uint32_t me, uint32_t cap,
                    uint64_t flags_offset_bytes, uint32_t* __restrict__ epoch_and_ticket, uint32_t* __restrict__ error,
                    uint32_t* __restrict__ overflow) {
    __shared__ uint32_t dst_base[33], dst_count[32];
    const uint32_t warps_per_block = kPeerPushThreads / kWarp;
    const uint32_t lane = threadIdx.x % kWarp;
    // pairs are sorted by expert and experts are contiguous per rank: a destination's pairs are one run. A warp sums a
    // destination's expert counts (independent loads), then one thread prefixes the at most 32 totals.
    for (uint32_t r = threadIdx.x / kWarp; r < world; r += warps_per_block) {
        uint32_t c = 0;
        for (uint32_t e = r * experts_per_rank + lane; e < (r + 1) * experts_per_rank && e < num_experts; e += kWarp) c += per_expert_counts[e];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) c += __shfl_xor_sync(kFullMask, c, off);
        if (lane == 0) dst_count[r] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (uint32_t r = 0; r < world; ++r) {
            dst_base[r] = run;
            run += dst_count[r];
            if (dst_count[r] > cap && blockIdx.x == 0) atomicMax(overflow, dst_count[r]);
        }
    }
    __syncthreads();
    const uint32_t total = world * cap;
    for (uint32_t slot = blockIdx.x * warps_per_block + threadIdx.x / kWarp; slot < total; slot += gridDim.x * warps_per_block) {
        const uint32_t dst = slot / cap, pos = slot % cap;
        uint16_t* out_row = reinterpret_cast<uint16_t*>(peers[dst] + dst_offset_bytes) + ((size_t)me * cap + pos) * dst_stride;
        if (pos >= dst_count[dst]) {
            if (lane == 0) *reinterpret_cast<uint4*>(out_row + d) = make_uint4(0xFFFFFFFFu, 0u, 0u, 0u);
            continue;
        }
        const tf_pair pr = sorted_pairs[dst_base[dst] + pos];
        uint4* out = reinterpret_cast<uint4*>(out_row);
        warp_copy_u4(reinterpret_cast<const uint4*>(hidden + (size_t)pr.token * hidden_stride), out, d / 8, lane);
        if (lane == 0) {
            out[d / 8] = make_uint4(pr.expert % experts_per_rank, 0u, 0u, 0u);
            inverse_perm[pr.token * top_k + pr.rank] = slot;
        }
    }
    __shared__ bool last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();          // this block's rows before its ticket (see ep_peer_push_kernel)
        const uint32_t tk = atomicAdd(&epoch_and_ticket[1], 1u);
        last = tk == gridDim.x - 1;
        if (last) epoch_and_ticket[1] = 0u;
    }
    __syncthreads();
    if (!last) return;
    peer_barrier_in_block<WAIT>(peers, flags_offset_bytes, epoch_and_ticket, error, world, me);
}

__global__ void ep_peer_barrier_kernel(uint8_t* const* __restrict__ peers, uint64_t flags_offset_bytes,
                                       uint32_t* __restrict__ epoch_counter, uint32_t* __restrict__ error,
                                       uint32_t world, uint32_t me) {
    peer_barrier_in_block<true>(peers, flags_offset_bytes, epoch_counter, error, world, me);
}

}  // namespace tf

struct tf_peer_buffer {
    tf_context* ctx = nullptr;
    void* base = nullptr;
    uint64_t bytes = 0;
    cudaIpcMemHandle_t handle;
};

extern "C" {

tf_status tf_peer_buffer_create(tf_context* ctx, uint64_t bytes, tf_peer_buffer** out) {
    const char* name = "tf_peer_buffer_create";
    TF_REQUIRE(ctx, ctx != nullptr && out != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    *out = nullptr;
    TF_REQUIRE(ctx, bytes > 0, TF_ERR_INVALID_ARGUMENT, "%s: size must be positive", name);
    void* base = nullptr;
    cudaError_t e = cudaMalloc(&base, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return tf::fail(ctx, TF_ERR_OUT_OF_MEMORY, "%s: %llu bytes: %s", name, (unsigned long long)bytes, cudaGetErrorString(e));
    }
    e = cudaMemset(base, 0, bytes);
    tf_peer_buffer* b = new tf_peer_buffer();
    b->ctx = ctx; b->base = base; b->bytes = bytes;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&b->handle, base);
    if (e != cudaSuccess) {
        cudaGetLastError();
        cudaFree(base);
        delete b;
        return tf::fail(ctx, TF_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e));
    }
    *out = b;
    return TF_OK;
}

void tf_peer_buffer_destroy(tf_peer_buffer* buffer) {
    if (!buffer) return;
    if (buffer->base) cudaFree(buffer->base);
    delete buffer;
}

void* tf_peer_buffer_ptr(const tf_peer_buffer* buffer) { return buffer ? buffer->base : nullptr; }

tf_status tf_peer_buffer_export(const tf_peer_buffer* buffer, void* handle_out_64_bytes) {
    if (!buffer || !handle_out_64_bytes) return tf::fail(nullptr, TF_ERR_INVALID_ARGUMENT, "tf_peer_buffer_export: NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == TF_PEER_HANDLE_BYTES, "handle size");
    memcpy(handle_out_64_bytes, &buffer->handle, sizeof(cudaIpcMemHandle_t));
    return TF_OK;
}

tf_status tf_peer_buffer_import(tf_context* ctx, const void* handle_64_bytes, void** ptr_out) {
    const char* name = "tf_peer_buffer_import";
    TF_REQUIRE(ctx, ctx != nullptr && handle_64_bytes && ptr_out, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle_64_bytes, sizeof h);
    *ptr_out = nullptr;
    TF_CUDA(ctx, cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
    return TF_OK;
}

tf_status tf_peer_buffer_release(tf_context* ctx, void* imported_ptr) {
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "tf_peer_buffer_release: ctx is NULL");
    if (imported_ptr) TF_CUDA(ctx, cudaIpcCloseMemHandle(imported_ptr));
    return TF_OK;
}

}  // extern "C"

namespace tf {

// tf_ep_peer_push; wait = false: the launch publishes this rank's flags and ends, the consumer kernel waits.
tf_status peer_push(tf_context* ctx, void* stream, const void* src_rows, uint32_t src_stride_elements,
                    const void* const* peer_bases_device, uint64_t dst_offset_bytes, uint32_t dst_stride_elements,
                    uint32_t copy_elements, const uint32_t* slot_ids, uint32_t tail_at_element,
                    uint32_t world, uint32_t rank, uint32_t capacity,
                    uint64_t flags_offset_bytes, uint32_t* epoch_and_ticket_device, bool wait) {
    const char* name = "tf_ep_peer_push";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, src_rows && peer_bases_device, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, world > 0 && world <= 32 && rank < world && capacity > 0, TF_ERR_INVALID_ARGUMENT,
               "%s: bad rank, world (1...32) or capacity", name);
    TF_REQUIRE(ctx, flags_offset_bytes % 4 == 0, TF_ERR_ALIGNMENT, "%s: flags must be 4-byte aligned", name);
    TF_REQUIRE(ctx, copy_elements % 8 == 0 && copy_elements <= src_stride_elements && copy_elements <= dst_stride_elements,
               TF_ERR_INVALID_ARGUMENT, "%s: rows are copied in 16-byte pieces within both strides", name);
    TF_REQUIRE(ctx, src_stride_elements % 8 == 0 && dst_stride_elements % 8 == 0 && dst_offset_bytes % 16 == 0 &&
                        tf::aligned(src_rows, 16),
               TF_ERR_ALIGNMENT, "%s: rows must be 16-byte aligned", name);
    TF_REQUIRE(ctx, slot_ids != nullptr || (tail_at_element % 8 == 0 && tail_at_element + 8 <= src_stride_elements &&
                                             tail_at_element + 8 <= dst_stride_elements),
               TF_ERR_INVALID_ARGUMENT, "%s: the id tail must lie inside the row", name);
    const uint32_t slots = world * capacity;
    const uint32_t per_block = tf::kPeerPushThreads / tf::kWarp;
    uint32_t grid = (slots + per_block - 1) / per_block;
    const uint32_t limit = (uint32_t)ctx->sm_count * 4u;
    if (grid > limit) grid = limit;
    auto kern = wait ? tf::ep_peer_push_kernel<true> : tf::ep_peer_push_kernel<false>;
    kern<<<grid, tf::kPeerPushThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(src_rows), src_stride_elements, (uint8_t* const*)peer_bases_device,
        dst_offset_bytes, dst_stride_elements, copy_elements, slot_ids, tail_at_element, world, rank, capacity,
        flags_offset_bytes, epoch_and_ticket_device, ctx->peer_error);
    return tf::check_launch(ctx, name);
}

// tf_ep_pack_push with the same choice.
tf_status pack_push(tf_context* ctx, void* stream, const void* hidden, uint32_t hidden_stride_elements,
                    const tf_device_routes* routes, uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                    uint32_t experts_per_rank, uint32_t d, const void* const* peer_bases_device, uint64_t dst_offset_bytes,
                    uint32_t dst_stride_elements, uint32_t* inverse_perm, uint32_t world, uint32_t rank, uint32_t capacity,
                    uint64_t flags_offset_bytes, uint32_t* epoch_and_ticket_device, bool wait) {
    const char* name = "tf_ep_pack_push";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, hidden && routes && routes->sorted_pairs && routes->per_expert_counts && peer_bases_device && inverse_perm &&
                        epoch_and_ticket_device,
               TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, world > 0 && world <= 32 && rank < world && capacity > 0, TF_ERR_INVALID_ARGUMENT,
               "%s: bad rank, world (1...32) or capacity", name);
    TF_REQUIRE(ctx, experts_per_rank > 0 && experts_per_rank * world == num_experts, TF_ERR_INVALID_ARGUMENT,
               "%s: %u experts do not divide over %u ranks of %u", name, num_experts, world, experts_per_rank);
    TF_REQUIRE(ctx, d % 8 == 0 && hidden_stride_elements >= d && dst_stride_elements >= d + 8 && dst_stride_elements % 8 == 0,
               TF_ERR_INVALID_ARGUMENT, "%s: D must be a multiple of 8 and the destination rows at least D + 8 wide", name);
    TF_REQUIRE(ctx, tf::aligned(hidden, 16) && (hidden_stride_elements * 2) % 16 == 0 && dst_offset_bytes % 16 == 0 && flags_offset_bytes % 4 == 0,
               TF_ERR_ALIGNMENT, "%s: rows must be 16-byte aligned", name);
    if (query_count == 0) return TF_OK;
    const uint32_t slots = world * capacity;
    const uint32_t per_block = tf::kPeerPushThreads / tf::kWarp;
    uint32_t grid = (slots + per_block - 1) / per_block;
    const uint32_t limit = (uint32_t)ctx->sm_count * 4u;
    if (grid > limit) grid = limit;
    auto kern = wait ? tf::ep_pack_push_kernel<true> : tf::ep_pack_push_kernel<false>;
    kern<<<grid, tf::kPeerPushThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(hidden), hidden_stride_elements, routes->sorted_pairs, routes->per_expert_counts, top_k, num_experts,
        experts_per_rank, d, dst_stride_elements, (uint8_t* const*)peer_bases_device, dst_offset_bytes, inverse_perm, world, rank,
        capacity, flags_offset_bytes, epoch_and_ticket_device, ctx->peer_error, ctx->device_error);
    return tf::check_launch(ctx, name);
}

}  // namespace tf

extern "C" {

tf_status tf_ep_peer_push(tf_context* ctx, void* stream, const void* src_rows, uint32_t src_stride_elements,
                          const void* const* peer_bases_device, uint64_t dst_offset_bytes, uint32_t dst_stride_elements,
                          uint32_t copy_elements, const uint32_t* slot_ids, uint32_t tail_at_element,
                          uint32_t world, uint32_t rank, uint32_t capacity,
                          uint64_t flags_offset_bytes, uint32_t* epoch_and_ticket_device) {
    return tf::peer_push(ctx, stream, src_rows, src_stride_elements, peer_bases_device, dst_offset_bytes, dst_stride_elements,
                         copy_elements, slot_ids, tail_at_element, world, rank, capacity, flags_offset_bytes, epoch_and_ticket_device, true);
}

tf_status tf_ep_pack_push(tf_context* ctx, void* stream, const void* hidden, uint32_t hidden_stride_elements,
                          const tf_device_routes* routes, uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                          uint32_t experts_per_rank, uint32_t d, const void* const* peer_bases_device, uint64_t dst_offset_bytes,
                          uint32_t dst_stride_elements, uint32_t* inverse_perm, uint32_t world, uint32_t rank, uint32_t capacity,
                          uint64_t flags_offset_bytes, uint32_t* epoch_and_ticket_device) {
    return tf::pack_push(ctx, stream, hidden, hidden_stride_elements, routes, query_count, top_k, num_experts, experts_per_rank, d,
                         peer_bases_device, dst_offset_bytes, dst_stride_elements, inverse_perm, world, rank, capacity,
                         flags_offset_bytes, epoch_and_ticket_device, true);
}

tf_status tf_ep_peer_barrier(tf_context* ctx, void* stream, const void* const* peer_bases_device, uint64_t flags_offset_bytes,
                             uint32_t* epoch_counter_device, uint32_t world, uint32_t rank) {
    const char* name = "tf_ep_peer_barrier";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, peer_bases_device && epoch_counter_device, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, world > 0 && world <= 32 && rank < world, TF_ERR_INVALID_ARGUMENT, "%s: world must be 1...32", name);
    TF_REQUIRE(ctx, flags_offset_bytes % 4 == 0, TF_ERR_ALIGNMENT, "%s: flags must be 4-byte aligned", name);
    tf::ep_peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        (uint8_t* const*)peer_bases_device, flags_offset_bytes, epoch_counter_device, ctx->peer_error, world, rank);
    return tf::check_launch(ctx, name);
}

}  // extern "C"
