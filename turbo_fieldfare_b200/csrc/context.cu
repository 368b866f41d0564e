// Context and error reporting. Replaces the device/queue/pipeline-cache role of
// MetalContext (Infrastructure/Metal/MetalContext.swift:51-214): CUDA kernels
// are compiled ahead of time, so the context only pins a device, owns the small
// router scratch and records errors.
#include "tf_common.cuh"

namespace tf {

size_t streamed_scratch_bytes();      // grouped.cu

std::string& global_error() {
    static std::string s;
    return s;
}

static std::mutex& err_mutex() {
    static std::mutex m;
    return m;
}

void set_global_error(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    std::lock_guard<std::mutex> lock(err_mutex());
    global_error() = buf;
}

tf_status fail(tf_context* ctx, tf_status code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    std::lock_guard<std::mutex> lock(err_mutex());
    if (ctx) ctx->last_error = buf;
    global_error() = buf;
    return code;
}

tf_status check_launch(tf_context* ctx, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ctx, TF_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
    if (ctx) ctx->launches += 1;
    return TF_OK;
}

}  // namespace tf

extern "C" {

int tf_abi_version(void) { return TF_ABI_VERSION; }

tf_status tf_context_create(int device, tf_context** out) {
    if (!out) return tf::fail(nullptr, TF_ERR_INVALID_ARGUMENT, "tf_context_create: out is NULL");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return tf::fail(nullptr, TF_ERR_NO_DEVICE, "no CUDA device: %s (this library has no CPU fallback)",
                        e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    if (device < 0 || device >= count)
        return tf::fail(nullptr, TF_ERR_INVALID_ARGUMENT, "device %d out of range (0..%d)", device, count - 1);
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return tf::fail(nullptr, TF_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10)
        return tf::fail(nullptr, TF_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only",
                        device, prop.major, prop.minor);
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return tf::fail(nullptr, TF_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
    tf_context* ctx = new tf_context();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    e = cudaMalloc(&ctx->router_logits, sizeof(float) * tf::kRouterSplitRows * TF_MAX_ROUTER_EXPERTS);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->router_tickets, sizeof(unsigned int) * (tf::kRouterSplitRows + 1));   // rows + one for the whole block
    if (e == cudaSuccess) e = cudaMemset(ctx->router_tickets, 0, sizeof(unsigned int) * (tf::kRouterSplitRows + 1));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->device_error, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ctx->device_error, 0, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->peer_error, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ctx->peer_error, 0, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->streamed_scratch, tf::streamed_scratch_bytes());
    if (e == cudaSuccess) e = cudaMalloc(&ctx->group_scratch, sizeof(uint32_t) * 2 * 256 * TF_MAX_ROUTER_EXPERTS);     // counts, then start positions
    if (e == cudaSuccess) e = cudaMalloc(&ctx->grid_barrier, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ctx->grid_barrier, 0, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->qmm_groups, 2 * 64 * (TF_MAX_ROUTER_EXPERTS + 1));   // routed and dense tables
    if (e == cudaSuccess) e = cudaMalloc(&ctx->qmm_totals, 4 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->fork_event, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->join_event, cudaEventDisableTiming);
    if (e != cudaSuccess) {
        tf_status s = tf::fail(nullptr, TF_ERR_OUT_OF_MEMORY, "context scratch: %s", cudaGetErrorString(e));
        tf_context_destroy(ctx);
        return s;
    }
    *out = ctx;
    return TF_OK;
}

void tf_context_destroy(tf_context* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->router_logits) cudaFree(ctx->router_logits);
    if (ctx->router_tickets) cudaFree(ctx->router_tickets);
    if (ctx->router_approx) cudaFree(ctx->router_approx);
    if (ctx->device_error) cudaFree(ctx->device_error);
    if (ctx->peer_error) cudaFree(ctx->peer_error);
    if (ctx->streamed_scratch) cudaFree(ctx->streamed_scratch);
    if (ctx->group_scratch) cudaFree(ctx->group_scratch);
    if (ctx->grid_barrier) cudaFree(ctx->grid_barrier);
    if (ctx->qmm_groups) cudaFree(ctx->qmm_groups);
    if (ctx->qmm_totals) cudaFree(ctx->qmm_totals);
    if (ctx->lm_x) cudaFree(ctx->lm_x);
    if (ctx->lm_logits) cudaFree(ctx->lm_logits);
    if (ctx->lm_best) cudaFree(ctx->lm_best);
    if (ctx->side_stream) cudaStreamDestroy(ctx->side_stream);
    if (ctx->fork_event) cudaEventDestroy(ctx->fork_event);
    if (ctx->join_event) cudaEventDestroy(ctx->join_event);
    delete ctx;
}

const char* tf_last_error(tf_context* ctx) {
    if (ctx) return ctx->last_error.c_str();
    return tf::global_error().c_str();
}

uint64_t tf_launch_count(tf_context* ctx) { return ctx ? ctx->launches : 0; }

tf_status tf_context_set_tensorcore_min_tokens(tf_context* ctx, uint32_t tokens) {
    TF_REQUIRE(ctx, ctx != nullptr && tokens > 0, TF_ERR_INVALID_ARGUMENT, "tf_context_set_tensorcore_min_tokens: ctx is NULL or tokens is 0");
    ctx->tensorcore_min_tokens = tokens;
    return TF_OK;
}

tf_status tf_context_set_shared_tensorcore_min_tokens(tf_context* ctx, uint32_t tokens) {
    TF_REQUIRE(ctx, ctx != nullptr && tokens > 0, TF_ERR_INVALID_ARGUMENT, "tf_context_set_shared_tensorcore_min_tokens: ctx is NULL or tokens is 0");
    ctx->shared_tensorcore_min_tokens = tokens;
    return TF_OK;
}

tf_status tf_context_set_router_tensorcore_min_rows(tf_context* ctx, uint32_t rows) {
    TF_REQUIRE(ctx, ctx != nullptr && rows > 0, TF_ERR_INVALID_ARGUMENT, "tf_context_set_router_tensorcore_min_rows: ctx is NULL or rows is 0");
    ctx->router_tensorcore_min_rows = rows;
    return TF_OK;
}

tf_status tf_context_set_ep_tensorcore_min_rows_per_expert(tf_context* ctx, uint32_t rows) {
    TF_REQUIRE(ctx, ctx != nullptr && rows > 0, TF_ERR_INVALID_ARGUMENT, "tf_context_set_ep_tensorcore_min_rows_per_expert: ctx is NULL or rows is 0");
    ctx->ep_tensorcore_min_rows_per_expert = rows;
    return TF_OK;
}

tf_status tf_context_set_single_launch_step(tf_context* ctx, int enabled) {
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "tf_context_set_single_launch_step: ctx is NULL");
    ctx->single_launch_step = enabled != 0;
    return TF_OK;
}

tf_status tf_context_set_step_trace(tf_context* ctx, void* device_u64, uint32_t capacity) {
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "tf_context_set_step_trace: ctx is NULL");
    TF_REQUIRE(ctx, device_u64 == nullptr || tf::aligned(device_u64, 8), TF_ERR_ALIGNMENT, "tf_context_set_step_trace: the buffer must be 8-byte aligned");
    ctx->step_trace = static_cast<unsigned long long*>(device_u64);
    ctx->step_trace_capacity = device_u64 ? capacity : 0;
    return TF_OK;
}

tf_status tf_device_status(tf_context* ctx, uint32_t* code_out) {
    TF_REQUIRE(ctx, ctx != nullptr && code_out != nullptr, TF_ERR_INVALID_ARGUMENT, "tf_device_status: NULL argument");
    TF_CUDA(ctx, cudaDeviceSynchronize());
    uint32_t kernel_code = 0, peer_code = 0;
    TF_CUDA(ctx, cudaMemcpy(&kernel_code, ctx->device_error, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    TF_CUDA(ctx, cudaMemcpy(&peer_code, ctx->peer_error, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    *code_out = kernel_code ? kernel_code : peer_code;
    if (*code_out != 0) {
        const uint32_t code = *code_out;
        TF_CUDA(ctx, cudaMemset(ctx->device_error, 0, sizeof(uint32_t)));
        TF_CUDA(ctx, cudaMemset(ctx->peer_error, 0, sizeof(uint32_t)));
        return tf::fail(ctx, TF_ERR_CUDA, "a kernel gave up a bounded wait (device code 0x%08x); results since the last check are invalid", code);
    }
    return TF_OK;
}

}  // extern "C"
