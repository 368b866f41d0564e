// Shared device/host helpers for the sm_100a routed-expert kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <string>

#include "turbofieldfare_cuda.h"

namespace tf {

constexpr int kGroup = TF_GROUP_SIZE;
constexpr int kWarp = 32;
constexpr unsigned kFullMask = 0xFFFFFFFFu;
constexpr int kRouterSplitRows = 64;   // rows served by the multi-block decode router
constexpr int kChunkTokens = 8;        // tokens per work chunk of the grouped kernels (the n of m16n8k16)

// ---------------------------------------------------------------------------
// host side: context and error plumbing
// ---------------------------------------------------------------------------

std::string& global_error();
void set_global_error(const char* fmt, ...);

}  // namespace tf

struct tf_context {
    int device = 0;
    int sm_count = 0;
    uint64_t launches = 0;
    std::string last_error;
    // Router scratch owned by the context, like the 1 KiB logits buffer the
    // reference's MoE wrapper owns (Kernels/MoE/MoE.swift:92-106).
    float* router_logits = nullptr;        // [kRouterSplitRows, 256]
    unsigned int* router_tickets = nullptr;  // [kRouterSplitRows], self-resetting
    // Prefill-sized router: (approximate logit, magnitude) per (row, expert) between its two launches; grown on demand.
    void* router_approx = nullptr;
    size_t router_approx_bytes = 0;
    // Batches of at least this many rows take the two-launch router (tensor-core logits + canonical re-check).
    uint32_t router_tensorcore_min_rows = 256;
    // One device word that kernels with bounded waits set when a wait gives up (0 = healthy).
    uint32_t* device_error = nullptr;
    // The same for the flag barriers of the peer exchange (peer.cu), kept apart so that a code from another kernel
    // cannot switch the cross-GPU waits off.
    uint32_t* peer_error = nullptr;
    // Group and chunk tables of tf_grouped_moe_streamed (built on the device per call).
    void* streamed_scratch = nullptr;
    // Arrival counter of the grid barriers of the single-launch decode step (zeroed on the stream before each launch).
    uint32_t* grid_barrier = nullptr;
    // tf_stack_forward runs a one-token step as one persistent launch when set (tf_context_set_single_launch_step).
    bool single_launch_step = false;
    // Optional caller-owned device buffer that the single-launch decode step fills with global-timer stamps.
    unsigned long long* step_trace = nullptr;
    uint32_t step_trace_capacity = 0;
    // Per-slice expert histograms and start positions of the grouping of many pairs (grouped.cu): 2 x 256 slices x 256 experts.
    uint32_t* group_scratch = nullptr;
    // Group tables and tile totals of the tensor-core grouped GEMM (filled on the device per launch): one set for
    // routed launches and one for dense launches, which may run on two streams at once.
    void* qmm_groups = nullptr;
    uint32_t* qmm_totals = nullptr;
    // Side stream and fork/join events: the shared expert of a block runs beside its router and routed experts.
    cudaStream_t side_stream = nullptr;
    cudaEvent_t fork_event = nullptr, join_event = nullptr;
    // Block forwards of at least this many tokens run their expert GEMMs on the tcgen05 tensor cores.
    uint32_t tensorcore_min_tokens = 256;
    // The same for the shared expert alone (a dense GEMM over all tokens of the block).
    uint32_t shared_tensorcore_min_tokens = 256;
    // Fixed-capacity expert-parallel exchanges whose expected rows per local expert (ranks x tokens x top_k / experts of
    // a rank) reach this number run the owner's expert phase on the tensor cores. Off by default (measured slower at eight
    // ranks x 64 tokens, 32 rows per expert: 6.62 ms against 5.98 ms per step).
    uint32_t ep_tensorcore_min_rows_per_expert = 0xFFFFFFFFu;
    // Scratch of the greedy LM head, like the normed-row and row-summary buffers the reference's wrapper owns
    // (Kernels/Fusions/LMHeadChainInt4.swift:26-51); grown on demand by tf_lm_head_greedy_int4.
    uint16_t* lm_x = nullptr;               // fp16 [lm_x_capacity]
    uint32_t lm_x_capacity = 0;
    float* lm_logits = nullptr;             // fp32 [lm_logits_capacity]
    uint32_t lm_logits_capacity = 0;
    unsigned long long* lm_best = nullptr;  // packed (ordered logit, ~row); zero between calls
};

namespace tf {

tf_status fail(tf_context* ctx, tf_status code, const char* fmt, ...);
tf_status check_launch(tf_context* ctx, const char* what);

#define TF_REQUIRE(ctx, cond, code, ...)                      \
    do {                                                      \
        if (!(cond)) return ::tf::fail((ctx), (code), __VA_ARGS__); \
    } while (0)

#define TF_CUDA(ctx, expr)                                                          \
    do {                                                                            \
        cudaError_t _e = (expr);                                                    \
        if (_e != cudaSuccess)                                                      \
            return ::tf::fail((ctx), TF_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

// Launch with the programmatic-stream-serialisation attribute (see pdl_wait in the device helpers).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Function attributes and occupancy are properties of (kernel, device): caches of them are keyed by the device ordinal
// and guarded, so a second GPU in the same process (or a second thread) configures its own copy of a kernel.
constexpr int kMaxDevices = 64;
struct DeviceSmemCache {
    std::mutex mu;
    uint32_t bytes[kMaxDevices] = {};
};
// Raises the kernel's dynamic shared-memory limit on ctx's device to at least `bytes` (once per device and size).
template <typename Kernel>
inline tf_status ensure_dynamic_smem(tf_context* ctx, Kernel kernel, DeviceSmemCache& cache, size_t bytes) {
    const int dev = ctx->device >= 0 && ctx->device < kMaxDevices ? ctx->device : -1;
    std::lock_guard<std::mutex> lock(cache.mu);
    if (dev >= 0 && bytes <= cache.bytes[dev]) return TF_OK;
    TF_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (dev >= 0) cache.bytes[dev] = (uint32_t)bytes;
    return TF_OK;
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline const uint8_t* byte_ptr(const void* p, uint64_t off) { return static_cast<const uint8_t*>(p) + off; }
inline uint8_t* byte_ptr(void* p, uint64_t off) { return static_cast<uint8_t*>(p) + off; }

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
__device__ __forceinline__ float f16_bits_to_float(uint16_t b) { return __half2float(__ushort_as_half(b)); }

template <bool SB_FP16>
__device__ __forceinline__ float sb_to_float(uint16_t b) {
    if constexpr (SB_FP16) return f16_bits_to_float(b);
    else return bf16_bits_to_float(b);
}

// Fixed xor-butterfly: every lane ends with the same bits, and the order is the
// one the CPU oracle emulates for the router logits.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(kFullMask, v, off));
    return v;
}

// tanh GELU with the inner argument clamped to +-20 (Metal/MoE/moe.metal:53-60).
// tanh(u) = 1 - 2 / (exp(2u) + 1) with the hardware exp2: relative error about 1e-6, far below
// the fp16 rounding of the activation, at a fraction of tanhf's instruction count.
__device__ __forceinline__ float gelu_tanh(float x) {
    const float x3 = x * x * x;
    float inner = 0.7978845608028654f * (x + 0.044715f * x3);
    inner = fminf(fmaxf(inner, -20.0f), 20.0f);
    const float e = __expf(2.0f * inner);
    const float th = 1.0f - __fdividef(2.0f, e + 1.0f);
    return 0.5f * x * (1.0f + th);
}

// Programmatic dependent launch: a kernel launched with launch_pdl may start (block scheduling, shared-memory set-up)
// while its predecessor on the stream is still draining; pdl_wait() returns once the predecessor has completed and its
// writes are visible, so it comes before the first access to anything another kernel produces (and before any
// write). Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint4 ldg_nc_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

}  // namespace tf
