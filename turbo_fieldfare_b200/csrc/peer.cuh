// Flag barrier between the ranks of an expert-parallel group, split in two halves so that the wait can sit at the start
// of the kernel that consumes the exchanged rows instead of at the end of the kernel that sent them: the producer's
// last block publishes "rank `me` reached epoch e" in every peer's flag row and ends; the consumer reads the epoch
// (advanced by the producer earlier on the same stream) and waits, bounded, until every peer has published it here.
// Every wait is bounded: after kPeerSpinLimit polls the kernel records kErrPeerTimeout in the context's peer status
// word and goes on; once that word is set, later waits return at once.
#pragma once

#include "tf_common.cuh"

namespace tf {

constexpr uint32_t kPeerSpinLimit = 1u << 23;           // x ~0.2 us per poll: about 2 s
constexpr uint32_t kErrPeerTimeout = 0x7F000011u;

// What a consumer kernel needs to wait for its peers; flags == nullptr: nothing to wait for.
struct PeerWait {
    const uint32_t* flags;              // this rank's flag row: word r is written by rank r
    const uint32_t* epoch_counter;      // this rank's epoch word (device), already advanced by the producer
    uint32_t* error;                    // the context's peer status word
    uint32_t world;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Thread r < world waits for peer r's flag. Polls back to back at first (the flag is usually there within a few
// microseconds), then with short sleeps.
__device__ __forceinline__ void peer_wait_flag(const uint32_t* flag, uint32_t epoch, uint32_t* error) {
    if (*reinterpret_cast<volatile uint32_t*>(error) != 0u) return;      // a wait already gave up: do not wait again
    for (uint32_t spin = 0; spin < kPeerSpinLimit; ++spin) {
        if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return;
        if (spin > 64) __nanosleep(100);
    }
    atomicCAS(error, 0u, kErrPeerTimeout);
}

// Called by every thread of a block (at least `world` threads) before it touches rows a peer has written.
__device__ __forceinline__ void peer_wait_in_block(const PeerWait& w) {
    if (w.flags == nullptr) return;
    if (threadIdx.x < w.world) {
        const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(w.epoch_counter);
        peer_wait_flag(w.flags + threadIdx.x, epoch, w.error);
    }
    __syncthreads();
}

// peer.cu: the C ABI's tf_ep_peer_push / tf_ep_pack_push with the choice of who waits (wait = false: the consumer).
tf_status peer_push(tf_context* ctx, void* stream, const void* src_rows, uint32_t src_stride_elements,
                    const void* const* peer_bases_device, uint64_t dst_offset_bytes, uint32_t dst_stride_elements,
                    uint32_t copy_elements, const uint32_t* slot_ids, uint32_t tail_at_element,
                    uint32_t world, uint32_t rank, uint32_t capacity,
                    uint64_t flags_offset_bytes, uint32_t* epoch_and_ticket_device, bool wait);
tf_status pack_push(tf_context* ctx, void* stream, const void* hidden, uint32_t hidden_stride_elements,
                    const tf_device_routes* routes, uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                    uint32_t experts_per_rank, uint32_t d, const void* const* peer_bases_device, uint64_t dst_offset_bytes,
                    uint32_t dst_stride_elements, uint32_t* inverse_perm, uint32_t world, uint32_t rank, uint32_t capacity,
                    uint64_t flags_offset_bytes, uint32_t* epoch_and_ticket_device, bool wait);

}  // namespace tf
