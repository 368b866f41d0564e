// Expert parallelism behind the C ABI: communicator, exchange buffers, the per-layer loop and every collective.
//
// The reference is single-GPU (Infrastructure/Metal/MetalContext.swift:51-71); its MoE section of the forward runner
// (Runtime/Inference/RealForwardRunner.swift:902-1186 prefill, :1449-1693 decode) is what a host calls per layer.
// With the experts sharded E/N per GPU the same call becomes tf_moe_block_forward_ep / tf_stack_forward_ep:
//
//   tf_ep_dispatch   router, top-8, device grouping over the global experts, rows packed by owner rank
//   exchange         rows (and expert ids) to the owners
//   experts          owners group the received rows by local expert and run gate/up/GeGLU/down
//   exchange         result rows back to the tokens' home ranks
//   combine          shared expert (replicated; on the side stream, beside the exchanges) + weighted sum in rank order
//
// Three exchange modes:
//   TF_EP_EXACT        exact row counts over NCCL send/recv in one group per direction. The per-expert histograms of
//                      all ranks are all-gathered on the device and read back once per layer (the one host
//                      synchronisation of the layer); used for prefill-sized blocks, whose expert phase runs on the
//                      tensor cores.
//   TF_EP_FIXED_NCCL   a fixed capacity per destination (static shapes, no host synchronisation), rows carry their
//                      expert id in an 8-element tail, NCCL send/recv.
//   TF_EP_FIXED_PEER   the same layout, but rows are pushed straight into the owners' buffers by a kernel over peer
//                      memory with flag barriers (peer.cu): plain kernels only, so a whole decode step can be captured
//                      in a CUDA graph. Falls back to TF_EP_FIXED_NCCL on every rank together when a mapping fails.
//
// NCCL is bound at run time (dlopen of libnccl.so.2), so the library has no link-time dependency on it and a host
// process that already loaded NCCL (e.g. through another framework) shares that copy.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstring>
#include <vector>

#include "block.cuh"
#include "peer.cuh"

namespace tf {

struct NcclApi {
    bool ready = false;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

static NcclApi& nccl_api() {
    static NcclApi api;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (api.ready) return api;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return api;
    auto sym = [&](const char* n) { return dlsym(h, n); };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
    api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
    api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.ready = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.GroupStart && api.GroupEnd && api.Send && api.Recv &&
                api.AllGather && api.AllReduce && api.GetErrorString;
    return api;
}

#define TF_NCCL(ctx, expr)                                                                                   \
    do {                                                                                                     \
        ncclResult_t _r = (expr);                                                                            \
        if (_r != ncclSuccess)                                                                               \
            return ::tf::fail((ctx), TF_ERR_CUDA, "%s: %s", #expr, ::tf::nccl_api().GetErrorString(_r));    \
    } while (0)

}  // namespace tf

struct tf_ep {
    tf_context* ctx = nullptr;
    ncclComm_t comm = nullptr;
    bool owns_comm = false;
    int rank = 0, world = 1;
};

struct tf_ep_buffers {
    tf_ep* ep = nullptr;
    tf_workspace* ws = nullptr;
    tf_ep_mode mode = TF_EP_EXACT;
    uint32_t max_tokens = 0, d = 0, f = 0, fs = 0, top_k = 0, num_experts = 0, local_experts = 0;
    uint32_t n_pairs = 0, capacity = 0, row_stride = 0, send_slots = 0;
    // send side
    uint16_t* send_rows = nullptr; uint32_t* send_ids = nullptr; uint32_t* inverse = nullptr; uint16_t* back_rows = nullptr;
    uint16_t* x_norm = nullptr; uint16_t* y_block = nullptr;
    // receive side (grown on demand in exact mode)
    uint32_t recv_cap = 0;
    uint16_t* recv_rows = nullptr; uint32_t* recv_ids = nullptr; uint16_t* out_rows = nullptr; uint16_t* acts = nullptr;
    uint16_t* zero_weights = nullptr; uint16_t* one_weights = nullptr;
    uint16_t* x_sorted = nullptr; uint16_t* out_sorted = nullptr; uint32_t* row_ids = nullptr; uint32_t* inverse_sorted = nullptr;
    uint8_t* routes_mem = nullptr; tf_device_routes routes{};
    // exact mode: histograms of all ranks
    uint32_t* all_hist_dev = nullptr; uint32_t* all_hist_host = nullptr;
    std::vector<uint64_t> send_counts, recv_counts;
    // peer mode
    tf_peer_buffer* peer = nullptr;
    std::vector<void*> imported;
    void** peer_bases_dev = nullptr; uint32_t* epoch = nullptr;
    uint64_t back_offset = 0, flags_offset = 0;
    bool owns_recv_rows = true, owns_back_rows = true;
    uint32_t tensorcore_min_rows = 2048;       // exact exchanges of at least this many rows run the experts on the tensor cores
    bool fixed_tensor = false;                 // fixed-capacity exchanges: the expert phase runs on the tensor cores
};

namespace tf {

static void free_recv(tf_ep_buffers* b) {
    if (b->owns_recv_rows && b->recv_rows) cudaFree(b->recv_rows);
    void* ptrs[] = {b->recv_ids, b->out_rows, b->acts, b->zero_weights, b->one_weights, b->x_sorted, b->out_sorted, b->row_ids,
                    b->inverse_sorted, b->routes_mem};
    for (void* p : ptrs) if (p) cudaFree(p);
    b->recv_rows = nullptr; b->recv_ids = nullptr; b->out_rows = nullptr; b->acts = nullptr; b->zero_weights = nullptr;
    b->one_weights = nullptr; b->x_sorted = nullptr; b->out_sorted = nullptr; b->row_ids = nullptr; b->inverse_sorted = nullptr;
    b->routes_mem = nullptr; b->recv_cap = 0;
}

__global__ void fill_u16_kernel(uint16_t* p, size_t n, uint16_t v) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}

// Receive-side buffers for `slots` rows (exact mode grows them; never called inside a stream capture).
static tf_status ensure_recv(tf_ep_buffers* b, uint32_t slots, bool sorted_scratch) {
    tf_context* ctx = b->ep->ctx;
    if (slots <= b->recv_cap && (!sorted_scratch || b->x_sorted)) return TF_OK;
    uint32_t cap = slots > b->recv_cap ? slots : b->recv_cap;
    if (b->recv_cap && cap < b->recv_cap + b->recv_cap / 2 && slots > b->recv_cap) cap = b->recv_cap + b->recv_cap / 2;
    TF_CUDA(ctx, cudaDeviceSynchronize());
    uint16_t* keep_recv = b->owns_recv_rows ? nullptr : b->recv_rows;
    free_recv(b);
    const size_t d = b->d, f = b->f, le = b->local_experts;
    if (keep_recv) b->recv_rows = keep_recv;
    else TF_CUDA(ctx, cudaMalloc(&b->recv_rows, (size_t)cap * b->row_stride * 2));
    TF_CUDA(ctx, cudaMalloc(&b->recv_ids, (size_t)cap * 4));
    TF_CUDA(ctx, cudaMalloc(&b->out_rows, (size_t)cap * d * 2));
    TF_CUDA(ctx, cudaMalloc(&b->acts, (size_t)cap * f * 2));
    TF_CUDA(ctx, cudaMalloc(&b->zero_weights, (size_t)cap * 2));
    TF_CUDA(ctx, cudaMemset(b->zero_weights, 0, (size_t)cap * 2));
    if (sorted_scratch) {
        TF_CUDA(ctx, cudaMalloc(&b->one_weights, (size_t)cap * 2));
        fill_u16_kernel<<<64, 256>>>(b->one_weights, cap, (uint16_t)0x3C00);      // fp16 1.0
        TF_CUDA(ctx, cudaMalloc(&b->x_sorted, (size_t)cap * d * 2));
        TF_CUDA(ctx, cudaMalloc(&b->out_sorted, (size_t)cap * d * 2));
        TF_CUDA(ctx, cudaMalloc(&b->row_ids, (size_t)cap * 4));
        TF_CUDA(ctx, cudaMalloc(&b->inverse_sorted, (size_t)cap * 4));
        TF_CUDA(ctx, cudaMemset(b->inverse_sorted, 0, (size_t)cap * 4));      // entries of empty slots must point inside out_sorted
    }
    // routing tables of the received rows: every row is one (token = slot, rank 0) pair of a local expert
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    const size_t o_pairs = 0, o_off = o_pairs + up((size_t)cap * 16), o_cnt = o_off + up(le * 4), o_grp = o_cnt + up(le * 4),
                 o_cg = o_grp + up(le * 12), o_cs = o_cg + up(((size_t)cap / 8 + le + 1) * 4), o_ctr = o_cs + up(le * 4),
                 total = o_ctr + 256;
    TF_CUDA(ctx, cudaMalloc(&b->routes_mem, total));
    TF_CUDA(ctx, cudaMemset(b->routes_mem, 0, total));
    b->routes.sorted_pairs = reinterpret_cast<tf_pair*>(b->routes_mem + o_pairs);
    b->routes.per_expert_offsets = reinterpret_cast<uint32_t*>(b->routes_mem + o_off);
    b->routes.per_expert_counts = reinterpret_cast<uint32_t*>(b->routes_mem + o_cnt);
    b->routes.groups = reinterpret_cast<tf_group*>(b->routes_mem + o_grp);
    b->routes.chunk_group = reinterpret_cast<uint32_t*>(b->routes_mem + o_cg);
    b->routes.chunk_start = reinterpret_cast<uint32_t*>(b->routes_mem + o_cs);
    b->routes.counters = reinterpret_cast<uint32_t*>(b->routes_mem + o_ctr);
    TF_CUDA(ctx, cudaDeviceSynchronize());
    b->recv_cap = cap;
    return TF_OK;
}

// All ranks meet on the host: a one-word all-reduce, waited for.
static tf_status ep_host_barrier(tf_ep* ep, int* min_flag) {
    tf_context* ctx = ep->ctx;
    if (ep->world == 1) return TF_OK;
    int32_t* dev = nullptr;
    TF_CUDA(ctx, cudaMalloc(&dev, 4));
    const int32_t v = min_flag ? *min_flag : 1;
    TF_CUDA(ctx, cudaMemcpy(dev, &v, 4, cudaMemcpyHostToDevice));
    TF_NCCL(ctx, nccl_api().AllReduce(dev, dev, 1, ncclInt32, ncclMin, ep->comm, nullptr));
    TF_CUDA(ctx, cudaStreamSynchronize(nullptr));
    int32_t r = 0;
    TF_CUDA(ctx, cudaMemcpy(&r, dev, 4, cudaMemcpyDeviceToHost));
    cudaFree(dev);
    if (min_flag) *min_flag = r;
    return TF_OK;
}

// Collective tear-down of the peer mappings in the order CUDA IPC asks for: every rank closes its imports, all ranks
// meet, and only then does each rank free the buffer it exported.
static void drop_peer(tf_ep_buffers* b) {
    tf_ep* ep = b->ep;
    for (void* p : b->imported) if (p) tf_peer_buffer_release(ep->ctx, p);
    b->imported.clear();
    ep_host_barrier(ep, nullptr);
    if (b->peer) { tf_peer_buffer_destroy(b->peer); b->peer = nullptr; }
    if (b->peer_bases_dev) { cudaFree(b->peer_bases_dev); b->peer_bases_dev = nullptr; }
    if (b->epoch) { cudaFree(b->epoch); b->epoch = nullptr; }
}

// One exchange buffer per rank: [receive area | return area | flags], mapped by every other rank (CUDA IPC); the
// receive and return areas replace recv_rows and back_rows. Collective; returns false (on every rank) when any rank
// could not allocate, export or map.
static tf_status map_peer_buffers(tf_ep_buffers* b, bool* ok_out) {
    tf_ep* ep = b->ep;
    tf_context* ctx = ep->ctx;
    const uint64_t recv_bytes = (uint64_t)b->send_slots * b->row_stride * 2, back_bytes = (uint64_t)b->send_slots * b->d * 2;
    b->back_offset = (recv_bytes + 255) / 256 * 256;
    b->flags_offset = (b->back_offset + back_bytes + 255) / 256 * 256;
    const uint64_t total = b->flags_offset + 256;
    int ok = 1;
    uint8_t handle[TF_PEER_HANDLE_BYTES] = {0};
    if (tf_peer_buffer_create(ctx, total, &b->peer) != TF_OK || tf_peer_buffer_export(b->peer, handle) != TF_OK) ok = 0;
    std::vector<uint8_t> all((size_t)ep->world * TF_PEER_HANDLE_BYTES, 0);
    if (ep->world > 1) {
        uint8_t* dev = nullptr;
        TF_CUDA(ctx, cudaMalloc(&dev, all.size() + TF_PEER_HANDLE_BYTES));
        TF_CUDA(ctx, cudaMemcpy(dev + all.size(), handle, TF_PEER_HANDLE_BYTES, cudaMemcpyHostToDevice));
        TF_NCCL(ctx, nccl_api().AllGather(dev + all.size(), dev, TF_PEER_HANDLE_BYTES, ncclUint8, ep->comm, nullptr));
        TF_CUDA(ctx, cudaStreamSynchronize(nullptr));
        TF_CUDA(ctx, cudaMemcpy(all.data(), dev, all.size(), cudaMemcpyDeviceToHost));
        cudaFree(dev);
        if (tf_status s = ep_host_barrier(ep, &ok)) return s;          // did every rank allocate and export?
    } else {
        memcpy(all.data(), handle, TF_PEER_HANDLE_BYTES);
    }
    std::vector<void*> bases(ep->world, nullptr);
    if (ok) {
        for (int r = 0; r < ep->world; ++r) {
            if (r == ep->rank) { bases[r] = tf_peer_buffer_ptr(b->peer); continue; }
            void* p = nullptr;
            if (tf_peer_buffer_import(ctx, all.data() + (size_t)r * TF_PEER_HANDLE_BYTES, &p) != TF_OK) { ok = 0; break; }
            b->imported.push_back(p);
            bases[r] = p;
        }
        if (tf_status s = ep_host_barrier(ep, &ok)) return s;          // did every rank map every peer?
    }
    if (!ok) {
        drop_peer(b);
        *ok_out = false;
        return TF_OK;
    }
    TF_CUDA(ctx, cudaMalloc(&b->peer_bases_dev, sizeof(void*) * ep->world));
    TF_CUDA(ctx, cudaMemcpy(b->peer_bases_dev, bases.data(), sizeof(void*) * ep->world, cudaMemcpyHostToDevice));
    TF_CUDA(ctx, cudaMalloc(&b->epoch, 8));
    TF_CUDA(ctx, cudaMemset(b->epoch, 0, 8));
    uint8_t* own = static_cast<uint8_t*>(tf_peer_buffer_ptr(b->peer));
    b->recv_rows = reinterpret_cast<uint16_t*>(own); b->owns_recv_rows = false;
    b->back_rows = reinterpret_cast<uint16_t*>(own + b->back_offset); b->owns_back_rows = false;
    *ok_out = true;
    return TF_OK;
}

}  // namespace tf

extern "C" {

tf_status tf_ep_unique_id(void* out_128_bytes) {
    if (!out_128_bytes) return tf::fail(nullptr, TF_ERR_INVALID_ARGUMENT, "tf_ep_unique_id: NULL argument");
    tf::NcclApi& api = tf::nccl_api();
    if (!api.ready) return tf::fail(nullptr, TF_ERR_UNSUPPORTED, "tf_ep_unique_id: libnccl.so.2 could not be loaded");
    static_assert(sizeof(ncclUniqueId) == TF_EP_UNIQUE_ID_BYTES, "unique id size");
    ncclUniqueId id;
    ncclResult_t r = api.GetUniqueId(&id);
    if (r != ncclSuccess) return tf::fail(nullptr, TF_ERR_CUDA, "ncclGetUniqueId: %s", api.GetErrorString(r));
    memcpy(out_128_bytes, &id, sizeof id);
    return TF_OK;
}

tf_status tf_ep_balanced_placement(const uint64_t* counts, uint32_t layers, uint32_t num_experts, uint32_t world,
                                   uint32_t* placement) {
    const char* name = "tf_ep_balanced_placement";
    if (!counts || !placement) return tf::fail(nullptr, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    if (layers == 0 || num_experts == 0 || world == 0 || num_experts % world != 0)
        return tf::fail(nullptr, TF_ERR_INVALID_ARGUMENT, "%s: %u experts do not divide over %u ranks", name, num_experts, world);
    const uint32_t per_rank = num_experts / world;
    std::vector<uint32_t> order(num_experts), used(world);
    std::vector<uint64_t> load(world);
    for (uint32_t l = 0; l < layers; ++l) {
        const uint64_t* c = counts + (size_t)l * num_experts;
        for (uint32_t e = 0; e < num_experts; ++e) order[e] = e;
        std::stable_sort(order.begin(), order.end(), [c](uint32_t a, uint32_t b) { return c[a] > c[b]; });
        std::fill(used.begin(), used.end(), 0u);
        std::fill(load.begin(), load.end(), (uint64_t)0);
        for (uint32_t e : order) {
            uint32_t best = world;
            for (uint32_t r = 0; r < world; ++r)
                if (used[r] < per_rank && (best == world || load[r] < load[best])) best = r;
            placement[(size_t)l * num_experts + best * per_rank + used[best]] = e;
            used[best] += 1;
            load[best] += c[e];
        }
    }
    return TF_OK;
}

static tf_status ep_new(tf_context* ctx, int rank, int world, tf_ep** out, const char* name) {
    TF_REQUIRE(ctx, ctx != nullptr && out != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    *out = nullptr;
    TF_REQUIRE(ctx, world >= 1 && world <= 32 && rank >= 0 && rank < world, TF_ERR_INVALID_ARGUMENT, "%s: bad rank %d of %d (1...32 ranks)", name, rank, world);
    tf_ep* ep = new tf_ep();
    ep->ctx = ctx; ep->rank = rank; ep->world = world;
    *out = ep;
    return TF_OK;
}

tf_status tf_ep_create(tf_context* ctx, const void* unique_id_128_bytes, int rank, int world, tf_ep** out) {
    const char* name = "tf_ep_create";
    if (tf_status s = ep_new(ctx, rank, world, out, name)) return s;
    if (world == 1) return TF_OK;                       // one rank: no communicator needed
    tf_ep* ep = *out;
    *out = nullptr;
    tf::NcclApi& api = tf::nccl_api();
    if (!api.ready || !unique_id_128_bytes) {
        delete ep;
        return tf::fail(ctx, api.ready ? TF_ERR_INVALID_ARGUMENT : TF_ERR_UNSUPPORTED,
                        api.ready ? "%s: the unique id is NULL" : "%s: libnccl.so.2 could not be loaded", name);
    }
    ncclUniqueId id;
    memcpy(&id, unique_id_128_bytes, sizeof id);
    cudaSetDevice(ctx->device);
    ncclResult_t r = api.CommInitRank(&ep->comm, world, id, rank);
    if (r != ncclSuccess) {
        delete ep;
        return tf::fail(ctx, TF_ERR_CUDA, "ncclCommInitRank: %s", api.GetErrorString(r));
    }
    ep->owns_comm = true;
    *out = ep;
    return TF_OK;
}

tf_status tf_ep_create_from_comm(tf_context* ctx, void* nccl_comm, int rank, int world, tf_ep** out) {
    const char* name = "tf_ep_create_from_comm";
    if (tf_status s = ep_new(ctx, rank, world, out, name)) return s;
    if (world > 1 && (!nccl_comm || !tf::nccl_api().ready)) {
        delete *out; *out = nullptr;
        return tf::fail(ctx, TF_ERR_INVALID_ARGUMENT, "%s: a communicator is needed for more than one rank", name);
    }
    (*out)->comm = static_cast<ncclComm_t>(nccl_comm);
    return TF_OK;
}

void tf_ep_destroy(tf_ep* ep) {
    if (!ep) return;
    if (ep->owns_comm && ep->comm) tf::nccl_api().CommDestroy(ep->comm);
    delete ep;
}

int tf_ep_rank(const tf_ep* ep) { return ep ? ep->rank : -1; }
int tf_ep_world(const tf_ep* ep) { return ep ? ep->world : 0; }

void tf_ep_buffers_destroy(tf_ep_buffers* b) {
    if (!b) return;
    cudaDeviceSynchronize();
    if (b->peer) {
        tf::ep_host_barrier(b->ep, nullptr);          // nobody is still writing into a buffer that is about to go
        tf::drop_peer(b);
    }
    tf::free_recv(b);
    if (b->owns_back_rows && b->back_rows) cudaFree(b->back_rows);
    void* ptrs[] = {b->send_rows, b->send_ids, b->inverse, b->x_norm, b->y_block, b->all_hist_dev};
    for (void* p : ptrs) if (p) cudaFree(p);
    if (b->all_hist_host) cudaFreeHost(b->all_hist_host);
    if (b->ws) tf_workspace_destroy(b->ws);
    delete b;
}

tf_status tf_ep_buffers_create(tf_ep* ep, uint32_t max_tokens, uint32_t d, uint32_t f, uint32_t fs, uint32_t top_k,
                               uint32_t num_experts, tf_ep_mode mode, tf_ep_buffers** out) {
    const char* name = "tf_ep_buffers_create";
    TF_REQUIRE(nullptr, ep != nullptr && out != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    tf_context* ctx = ep->ctx;
    *out = nullptr;
    TF_REQUIRE(ctx, max_tokens > 0 && d > 0 && f > 0 && fs > 0 && top_k > 0 && num_experts > 0, TF_ERR_INVALID_ARGUMENT, "%s: bad dimensions", name);
    TF_REQUIRE(ctx, num_experts % (uint32_t)ep->world == 0, TF_ERR_INVALID_ARGUMENT, "%s: %u experts do not divide over %d ranks", name, num_experts, ep->world);
    TF_REQUIRE(ctx, mode == TF_EP_EXACT || mode == TF_EP_FIXED_NCCL || mode == TF_EP_FIXED_PEER, TF_ERR_INVALID_ARGUMENT, "%s: bad mode", name);
    tf_ep_buffers* b = new tf_ep_buffers();
    b->ep = ep; b->mode = mode; b->max_tokens = max_tokens; b->d = d; b->f = f; b->fs = fs; b->top_k = top_k; b->num_experts = num_experts;
    b->local_experts = num_experts / (uint32_t)ep->world;
    b->n_pairs = max_tokens * top_k;
    const bool fixed = mode != TF_EP_EXACT;
    b->capacity = fixed ? b->n_pairs : 0;           // a destination can receive every pair of this rank
    b->send_slots = fixed ? (uint32_t)ep->world * b->capacity : b->n_pairs;
    b->row_stride = fixed ? d + 8 : d;              // fixed-capacity rows carry their expert id in the tail
    b->send_counts.assign(ep->world, 0); b->recv_counts.assign(ep->world, 0);
    tf_status s = tf_workspace_create(ctx, max_tokens, d, f, fs, top_k, num_experts, &b->ws);
    auto dev = [&](void* pp, size_t bytes) {
        if (s) return;
        void** p = static_cast<void**>(pp);
        cudaError_t e = cudaMalloc(p, bytes);
        if (e == cudaSuccess) e = cudaMemset(*p, 0, bytes);
        if (e != cudaSuccess) s = tf::fail(ctx, TF_ERR_OUT_OF_MEMORY, "%s: %zu bytes: %s", name, bytes, cudaGetErrorString(e));
    };
    dev(&b->send_rows, (size_t)b->send_slots * b->row_stride * 2);
    dev(&b->send_ids, (size_t)b->send_slots * 4);
    dev(&b->inverse, (size_t)b->n_pairs * 4);
    dev(&b->x_norm, (size_t)max_tokens * d * 2);
    dev(&b->y_block, (size_t)max_tokens * d * 2);
    if (!fixed) {
        dev(&b->all_hist_dev, (size_t)ep->world * num_experts * 4);
        if (!s && cudaMallocHost(&b->all_hist_host, (size_t)ep->world * num_experts * 4) != cudaSuccess)
            s = tf::fail(ctx, TF_ERR_OUT_OF_MEMORY, "%s: pinned host memory for the histograms", name);
    }
    if (s) { tf_ep_buffers_destroy(b); return s; }
    if (mode == TF_EP_FIXED_PEER) {
        bool ok = false;
        s = tf::map_peer_buffers(b, &ok);
        if (s) { tf_ep_buffers_destroy(b); return s; }
        if (!ok) b->mode = TF_EP_FIXED_NCCL;        // every rank takes this branch together
    }
    if (b->owns_back_rows) dev(&b->back_rows, (size_t)b->send_slots * d * 2);
    // fixed capacity: the choice of the expert kernels cannot wait for a row count (no host synchronisation), so it is
    // made here from the expected rows per local expert
    b->fixed_tensor = fixed && d % 64 == 0 && f % 64 == 0 &&
                      (uint64_t)ep->world * max_tokens * top_k >= (uint64_t)b->local_experts * ctx->ep_tensorcore_min_rows_per_expert;
    if (!s) s = tf::ensure_recv(b, fixed ? b->send_slots : (b->n_pairs ? b->n_pairs : 1), b->fixed_tensor);
    if (s) { tf_ep_buffers_destroy(b); return s; }
    *out = b;
    return TF_OK;
}

tf_ep_mode tf_ep_buffers_mode(const tf_ep_buffers* b) { return b ? b->mode : TF_EP_EXACT; }
tf_workspace* tf_ep_buffers_workspace(const tf_ep_buffers* b) { return b ? b->ws : nullptr; }

}  // extern "C"

namespace tf {

// What the combine of a layer needs, for a caller that folds it into its next launch.
struct EpPendingCombine {
    const uint16_t* back = nullptr;      // returned result rows
    PeerWait wait{nullptr, nullptr, nullptr, 0u};
    bool has_wait = false;
};

// tf_moe_block_forward_ep; with y == nullptr the weighted combine is left to the caller (`pending` says from what).
static tf_status block_forward_ep(tf_ep* ep, void* stream, const tf_moe_layer* layer, const void* x, void* y, uint32_t tokens,
                                  tf_ep_buffers* b, EpPendingCombine* pending) {
    const char* name = "tf_moe_block_forward_ep";
    TF_REQUIRE(nullptr, ep != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ep is NULL", name);
    tf_context* ctx = ep->ctx;
    TF_REQUIRE(ctx, layer && x && (y || pending) && b && b->ep == ep, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument or buffers of another communicator", name);
    TF_REQUIRE(ctx, tokens <= b->max_tokens, TF_ERR_SCRATCH_TOO_SMALL, "%s: %u tokens exceed the buffers (%u)", name, tokens, b->max_tokens);
    TF_REQUIRE(ctx, layer->d == b->d && layer->f == b->f && layer->fs == b->fs && layer->top_k == b->top_k && layer->num_experts == b->num_experts,
               TF_ERR_DIMENSION_MISMATCH, "%s: layer dimensions differ from the buffers", name);
    if (tokens == 0) return TF_OK;
    tf::NcclApi& api = tf::nccl_api();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t d = b->d, f = b->f, K = b->top_k, world = (uint32_t)ep->world, le = b->local_experts;
    const uint32_t n_pairs = tokens * K, cap = b->capacity, stride = b->row_stride;
    const bool fixed = b->mode != TF_EP_EXACT, peer = b->mode == TF_EP_FIXED_PEER;
    tf_workspace* ws = b->ws;
    // peer mode: a push publishes this rank's flag and ends; the kernel that consumes the exchanged rows waits for the peers
    tf::PeerWait peer_wait{nullptr, nullptr, nullptr, 0u};
    if (peer)
        peer_wait = tf::PeerWait{reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(tf_peer_buffer_ptr(b->peer)) + b->flags_offset), b->epoch,
                                 ctx->peer_error, world};

    // the shared expert needs only x: it runs on the side stream beside the dispatch, the exchanges and the experts
    TF_CUDA(ctx, cudaEventRecord(ctx->fork_event, st));
    TF_CUDA(ctx, cudaStreamWaitEvent(ctx->side_stream, ctx->fork_event, 0));
    tf_status s;
    const bool shared_tensor = tokens >= ctx->tensorcore_min_tokens && d % 64 == 0 && b->fs % 64 == 0;
    if (layer->shared_bits == 8)
        s = tf_shared_expert_int8_block(ctx, ctx->side_stream, x, 0, d, &layer->shared_gate, &layer->shared_up, &layer->shared_down,
                                        ws->shared_y, 0, d, ws->shared_act, tokens);
    else if (shared_tensor)
        s = tf_shared_expert_int4_tensorcore(ctx, ctx->side_stream, x, d, &layer->shared_gate, &layer->shared_up, &layer->shared_down,
                                             ws->shared_y, d, ws->shared_act, tokens);
    else
        s = tf_shared_expert_int4_block(ctx, ctx->side_stream, x, 0, d, &layer->shared_gate, &layer->shared_up, &layer->shared_down,
                                        ws->shared_y, 0, d, ws->shared_act, tokens);
    cudaEventRecord(ctx->join_event, ctx->side_stream);          // recorded even after a failure: a capture stays well formed
    auto bail = [&](tf_status code) { cudaStreamWaitEvent(st, ctx->join_event, 0); return code; };
    if (s) return bail(s);

    uint32_t recv_slots = 0;
    const uint16_t* recv_rows = nullptr; const uint32_t* recv_ids = b->recv_ids; const uint16_t* back = nullptr;
    if (peer) {
        // router + grouping over the global experts, then one launch that takes every pair's row from x straight into
        // its owner's receive area (id in the row tail) and ends with the flag barrier
        s = tf_router_gemma4_block_grouped(ctx, stream, layer->router.weights, layer->router.weights_off, layer->router.scales,
                                           layer->router.scales_off, layer->router.biases, layer->router.biases_off, x, 0, TF_FP16,
                                           layer->effective_scale, 0, layer->per_expert_scale, 0, layer->logit_bias, ws->indices,
                                           ws->weights, tokens, b->num_experts, d, K, d, tf_workspace_routes(ws));
        if (s) return bail(s);
        recv_slots = world * cap;
        s = tf::pack_push(ctx, stream, x, d, tf_workspace_routes(ws), tokens, K, b->num_experts, le, d,
                          (const void* const*)b->peer_bases_dev, 0, stride, b->inverse, world, (uint32_t)ep->rank, cap,
                          b->flags_offset, b->epoch, false);      // the grouping of the received rows waits for the peers
        if (s) return bail(s);
        recv_rows = b->recv_rows;
    } else if ((s = tf_ep_dispatch(ctx, stream, layer, x, tokens, ws, le, cap, b->send_rows, b->send_ids, b->inverse, stride)) != TF_OK) {
        return bail(s);
    } else if (fixed) {
        recv_slots = world * cap;
        if (world > 1) {
            const size_t bytes = (size_t)cap * stride * 2;
            TF_NCCL(ctx, api.GroupStart());
            for (uint32_t r = 0; r < world; ++r) {
                api.Send(reinterpret_cast<const uint8_t*>(b->send_rows) + r * bytes, bytes, ncclUint8, (int)r, ep->comm, st);
                api.Recv(reinterpret_cast<uint8_t*>(b->recv_rows) + r * bytes, bytes, ncclUint8, (int)r, ep->comm, st);
            }
            TF_NCCL(ctx, api.GroupEnd());
            recv_rows = b->recv_rows;
        } else {
            recv_rows = b->send_rows;
        }
    } else {
        // exact counts: all ranks' per-expert histograms, one read-back per layer
        const uint32_t E = b->num_experts;
        if (world > 1) {
            TF_NCCL(ctx, api.AllGather(ws->routes.per_expert_counts, b->all_hist_dev, E, ncclUint32, ep->comm, st));
            TF_CUDA(ctx, cudaMemcpyAsync(b->all_hist_host, b->all_hist_dev, (size_t)world * E * 4, cudaMemcpyDeviceToHost, st));
        } else {
            TF_CUDA(ctx, cudaMemcpyAsync(b->all_hist_host, ws->routes.per_expert_counts, (size_t)E * 4, cudaMemcpyDeviceToHost, st));
        }
        TF_CUDA(ctx, cudaStreamSynchronize(st));
        uint64_t total_recv = 0;
        for (uint32_t r = 0; r < world; ++r) {
            uint64_t sc = 0, rc = 0;
            for (uint32_t e = 0; e < le; ++e) {
                sc += b->all_hist_host[(size_t)ep->rank * E + r * le + e];           // my pairs for rank r's experts
                rc += b->all_hist_host[(size_t)r * E + (uint32_t)ep->rank * le + e];  // rank r's pairs for my experts
            }
            b->send_counts[r] = sc; b->recv_counts[r] = rc;
            total_recv += rc;
        }
        recv_slots = (uint32_t)total_recv;
        const bool tensor = recv_slots >= b->tensorcore_min_rows && d % 64 == 0 && f % 64 == 0;
        if (tf_status e2 = tf::ensure_recv(b, recv_slots ? recv_slots : 1, tensor)) return bail(e2);
        recv_ids = b->recv_ids;
        if (world > 1) {
            TF_NCCL(ctx, api.GroupStart());
            uint64_t so = 0, ro = 0;
            for (uint32_t r = 0; r < world; ++r) {
                if (b->send_counts[r]) {
                    api.Send(b->send_ids + so, b->send_counts[r], ncclUint32, (int)r, ep->comm, st);
                    api.Send(b->send_rows + so * d, b->send_counts[r] * d, ncclFloat16, (int)r, ep->comm, st);
                }
                if (b->recv_counts[r]) {
                    api.Recv(b->recv_ids + ro, b->recv_counts[r], ncclUint32, (int)r, ep->comm, st);
                    api.Recv(b->recv_rows + ro * d, b->recv_counts[r] * d, ncclFloat16, (int)r, ep->comm, st);
                }
                so += b->send_counts[r]; ro += b->recv_counts[r];
            }
            TF_NCCL(ctx, api.GroupEnd());
            recv_rows = b->recv_rows;
        } else {
            recv_rows = b->send_rows; recv_ids = b->send_ids;
        }
    }

    // the owner's expert phase
    const bool tensor = (fixed ? b->fixed_tensor : (recv_slots >= b->tensorcore_min_rows && d % 64 == 0 && f % 64 == 0)) && b->x_sorted;
    if (recv_slots) {
        if (tensor)
            s = tf::ep_experts_tensorcore_waiting(ctx, stream, layer->pool_layer_base, layer->expert_stride, &layer->offsets, recv_rows,
                                                  recv_ids, recv_slots, le, &b->routes, b->zero_weights, b->one_weights, b->x_sorted,
                                                  b->row_ids, b->inverse_sorted, b->acts, b->out_sorted, b->out_rows, d, f,
                                                  fixed ? stride : 0, peer ? &peer_wait : nullptr);
        else
            s = tf::ep_experts_waiting(ctx, stream, layer->pool_layer_base, layer->expert_stride, &layer->offsets, recv_rows, recv_ids,
                                       recv_slots, le, &b->routes, b->zero_weights, b->acts, b->out_rows, d, f, stride,
                                       peer ? &peer_wait : nullptr);
        if (s) return bail(s);
    }

    // results back to the home ranks
    if (peer) {
        s = tf::peer_push(ctx, stream, b->out_rows, d, (const void* const*)b->peer_bases_dev, b->back_offset, d, d, b->recv_ids, 0,
                          world, (uint32_t)ep->rank, cap, b->flags_offset, b->epoch, false);      // the combine waits for the peers
        if (s) return bail(s);
        back = b->back_rows;
    } else if (world > 1) {
        TF_NCCL(ctx, api.GroupStart());
        if (fixed) {
            const size_t bytes = (size_t)cap * d * 2;
            for (uint32_t r = 0; r < world; ++r) {
                api.Send(reinterpret_cast<const uint8_t*>(b->out_rows) + r * bytes, bytes, ncclUint8, (int)r, ep->comm, st);
                api.Recv(reinterpret_cast<uint8_t*>(b->back_rows) + r * bytes, bytes, ncclUint8, (int)r, ep->comm, st);
            }
        } else {
            uint64_t so = 0, ro = 0;
            for (uint32_t r = 0; r < world; ++r) {
                if (b->recv_counts[r]) api.Send(b->out_rows + ro * d, b->recv_counts[r] * d, ncclFloat16, (int)r, ep->comm, st);
                if (b->send_counts[r]) api.Recv(b->back_rows + so * d, b->send_counts[r] * d, ncclFloat16, (int)r, ep->comm, st);
                so += b->send_counts[r]; ro += b->recv_counts[r];
            }
        }
        TF_NCCL(ctx, api.GroupEnd());
        back = b->back_rows;
    } else {
        back = b->out_rows;
    }
    TF_CUDA(ctx, cudaStreamWaitEvent(st, ctx->join_event, 0));
    (void)n_pairs;
    if (y == nullptr) {
        pending->back = back; pending->wait = peer_wait; pending->has_wait = peer;
        return TF_OK;
    }
    return tf::ep_combine_waiting(ctx, stream, back, ws->weights, b->inverse, ws->shared_y, d, y, d, tokens, K, d,
                                  peer ? &peer_wait : nullptr);
}

}  // namespace tf

extern "C" {

tf_status tf_moe_block_forward_ep(tf_ep* ep, void* stream, const tf_moe_layer* layer, const void* x, void* y, uint32_t tokens,
                                  tf_ep_buffers* b) {
    TF_REQUIRE(ep ? ep->ctx : nullptr, y != nullptr, TF_ERR_INVALID_ARGUMENT, "tf_moe_block_forward_ep: NULL argument");
    return tf::block_forward_ep(ep, stream, layer, x, y, tokens, b, nullptr);
}

tf_status tf_stack_forward_ep(tf_ep* ep, void* stream, const tf_moe_layer* layers, const void* const* norm_weights_bf16,
                              uint32_t layer_count, float eps, void* hidden, uint32_t tokens, tf_ep_buffers* b) {
    const char* name = "tf_stack_forward_ep";
    TF_REQUIRE(nullptr, ep != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ep is NULL", name);
    tf_context* ctx = ep->ctx;
    TF_REQUIRE(ctx, layers && norm_weights_bf16 && hidden && b, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, tokens <= b->max_tokens, TF_ERR_SCRATCH_TOO_SMALL, "%s: %u tokens exceed the buffers (%u)", name, tokens, b->max_tokens);
    if (tokens == 0 || layer_count == 0) return TF_OK;
    // The weighted combine of layer l - 1, its residual add and the norm of layer l are one launch when the layout
    // allows (16-byte rows, top_k <= 8, D <= 4096); otherwise combine, then tf_residual_rmsnorm.
    const uint32_t d = b->d;
    const bool fold = d % 8 == 0 && d <= 4096 && b->top_k <= TF_MAX_TOP_K && tf::aligned(hidden, 16);
    const void* y_prev = nullptr;
    tf::EpPendingCombine pending;
    bool have_pending = false;
    tf_workspace* ws = b->ws;
    for (uint32_t l = 0; l < layer_count; ++l) {
        tf_status s;
        if (have_pending)
            s = tf::combine_rows_residual_rmsnorm(ctx, stream, hidden, pending.back, tf_workspace_weights(ws), b->inverse, ws->shared_y,
                                                  norm_weights_bf16[l], b->x_norm, tokens, b->top_k, d, eps,
                                                  pending.has_wait ? &pending.wait : nullptr);
        else
            s = tf_residual_rmsnorm(ctx, stream, hidden, y_prev, norm_weights_bf16[l], b->x_norm, tokens, d, eps);
        if (s) return s;
        if (fold) {
            if ((s = tf::block_forward_ep(ep, stream, &layers[l], b->x_norm, nullptr, tokens, b, &pending)) != TF_OK) return s;
            have_pending = true;
        } else {
            if ((s = tf::block_forward_ep(ep, stream, &layers[l], b->x_norm, b->y_block, tokens, b, nullptr)) != TF_OK) return s;
            y_prev = b->y_block;
        }
    }
    if (have_pending)
        return tf::combine_rows_residual_rmsnorm(ctx, stream, hidden, pending.back, tf_workspace_weights(ws), b->inverse, ws->shared_y,
                                                 nullptr, nullptr, tokens, b->top_k, d, eps, pending.has_wait ? &pending.wait : nullptr);
    return tf_residual_rmsnorm(ctx, stream, hidden, y_prev, nullptr, nullptr, tokens, d, eps);
}

}  // extern "C"
