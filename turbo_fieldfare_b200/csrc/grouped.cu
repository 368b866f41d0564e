// Device-side route grouping and the grouped small-batch expert kernels
// (decode at batch 1..64 and the first-correct path for larger batches).
//
// Replaces, for HBM-resident experts:
//   - PrefillMoEGrouping.groupTokenExpertPairs (Kernels/Prefill/MoE/PrefillMoEGrouping.swift:91-193)
//     as a device kernel: order (expert, token, rank), offsets, counts, groups;
//   - prefill_grouped_routed_moe_batched_phase1 / _down (Metal/Prefill/prefill.metal:598-670)
//     and, at batch 1, moe_phase1_gate_up_act / the per-slot part of moe_phase2
//     (Metal/MoE/moe.metal:248-482);
//   - the per-row shared-expert loop (Kernels/Prefill/MoE/PrefillSharedExpert.swift:11-59).
//
// Kernel design (memory-bound; HBM roofline): weights are the A operand of
// mma.sync.m16n8k16 (16 weight rows per tile), up to 8 tokens are the B operand
// (decode-sized batches put few tokens on an expert, so the tokens take the narrow side).
// A 4-bit code q placed in the low mantissa bits of an fp16 IS the subnormal
// q * 2^-24, so "dequantisation" is one AND per two codes and the tensor core
// multiplies exact integers by fp16 activations with fp32 accumulation. Scale
// and bias are applied per 64-column group after the MMAs:
//     y += (s * 2^24) * acc + b * sum_k x_k
// i.e. the reference's group factoring (Metal/Quant/dequant_int4.metal:14-19).
//
// A CTA is K-split: compute warp w owns columns [256 w, 256 w + 256) and keeps the
// activations of the current chunk (<= 8 tokens of one expert) for those columns in
// registers, already in MMA fragment order. A loader warp streams whole 16-row tiles
// (packed codes of every matrix plus their scale/bias rows) into a shared ring with
// bulk asynchronous copies (cp.async.bulk, one full row or one contiguous tile per
// copy, mbarrier completion; rows are padded so that the fragment loads are free of
// bank conflicts). After each tile a compute warp stores its partial sums and
// arrives on an mbarrier; two reducer warps add the partials in warp order
// (deterministic), apply the epilogue and store. No warp ever meets another at a
// block-wide barrier in the steady state. Every mbarrier wait is bounded: on expiry
// the kernel records an error code and returns.
#include "async_copy.cuh"
#include "peer.cuh"

namespace tf {

// ---------------------------------------------------------------------------
// route grouping on the device
// ---------------------------------------------------------------------------

constexpr int kGroupThreads = 256;
constexpr int kGroupPerThread = 4;

// counters: [0] group count, [1] total chunks (sum over groups of ceil(count/8)), [2] pair count
__global__ void __launch_bounds__(kGroupThreads)
group_routes_kernel(const uint32_t* __restrict__ indices, uint32_t idx_stride, uint32_t* __restrict__ ids_out,
                    const uint16_t* __restrict__ weights, uint32_t T, uint32_t K, uint32_t E,
                    tf_pair* __restrict__ sorted_pairs, uint32_t* __restrict__ per_expert_offsets,
                    uint32_t* __restrict__ per_expert_counts, tf_group* __restrict__ groups,
                    uint32_t* __restrict__ chunk_group, uint32_t* __restrict__ chunk_start,
                    uint32_t* __restrict__ counters, const PeerWait peer_wait) {
    __shared__ uint32_t hist[TF_MAX_ROUTER_EXPERTS];
    __shared__ uint32_t warp_tot[kGroupThreads / kWarp];
    __shared__ uint32_t s_offset;
    const uint32_t e = blockIdx.x;
    const uint32_t n = T * K;
    pdl_launch_dependents();
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) hist[i] = 0;
    pdl_wait();
    peer_wait_in_block(peer_wait);      // the ids may sit in rows that peers are still writing (ends with a block barrier)
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        // idx_stride > 1: the ids sit in the tails of exchanged rows; the first block also writes them out densely
        uint32_t ex = indices[(size_t)i * idx_stride];
        if (ids_out && e == 0) ids_out[i] = ex;
        if (ex == 0xFFFFFFFFu) continue;    // empty slot of a fixed-capacity exchange buffer
        if (ex >= E) ex = E - 1;            // min(id, E-1): Runtime/Inference/RealForwardRunner.swift:955
        atomicAdd(&hist[ex], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t off = 0, gi = 0, ch = 0;
        for (uint32_t i = 0; i < e; ++i) {
            off += hist[i];
            gi += hist[i] ? 1u : 0u;
            ch += (hist[i] + kChunkTokens - 1) / kChunkTokens;
        }
        s_offset = off;
        const uint32_t cnt = hist[e];
        per_expert_counts[e] = cnt;
        per_expert_offsets[e] = cnt ? off : 0xFFFFFFFFu;
        if (cnt) {
            groups[gi] = tf_group{e, off, cnt};
            chunk_start[gi] = ch;
            const uint32_t nch = (cnt + kChunkTokens - 1) / kChunkTokens;
            for (uint32_t j = 0; j < nch; ++j) chunk_group[ch + j] = gi;
        }
        if (e == E - 1) {
            counters[0] = gi + (cnt ? 1u : 0u);
            counters[1] = ch + (cnt + kChunkTokens - 1) / kChunkTokens;
            counters[2] = n;
            counters[3] = off + cnt;            // pairs that were grouped (empty slots of an exchange buffer are not)
        }
    }
    __syncthreads();
    if (hist[e] == 0) return;
    // stable scatter of this expert's pairs in token-major order
    uint32_t running = s_offset;
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    for (uint32_t base = 0; base < n; base += kGroupThreads * kGroupPerThread) {
        const uint32_t first = base + threadIdx.x * kGroupPerThread;
        uint32_t flags = 0, cnt = 0;
#pragma unroll
        for (int j = 0; j < kGroupPerThread; ++j) {
            const uint32_t i = first + j;
            if (i < n) {
                uint32_t ex = indices[(size_t)i * idx_stride];
                if (ex != 0xFFFFFFFFu && ex >= E) ex = E - 1;
                if (ex == e) { flags |= 1u << j; ++cnt; }
            }
        }
        uint32_t incl = cnt;
#pragma unroll
        for (int off = 1; off < kWarp; off <<= 1) {
            const uint32_t v = __shfl_up_sync(kFullMask, incl, off);
            if (lane >= off) incl += v;
        }
        if (lane == kWarp - 1) warp_tot[warp] = incl;
        __syncthreads();
        uint32_t wbase = 0, total = 0;
        for (int w2 = 0; w2 < kGroupThreads / kWarp; ++w2) {
            if (w2 < warp) wbase += warp_tot[w2];
            total += warp_tot[w2];
        }
        uint32_t pos = running + wbase + incl - cnt;
#pragma unroll
        for (int j = 0; j < kGroupPerThread; ++j) {
            if (flags & (1u << j)) {
                const uint32_t i = first + j;
                sorted_pairs[pos++] = tf_pair{i / K, e, i % K, (uint32_t)weights[i]};
            }
        }
        running += total;
        __syncthreads();
    }
}

// Many pairs (prefill, large exchanges): the one-block-per-expert kernel above reads all n ids in every expert's block
// (E x n reads). Here the pairs are split into contiguous slices, one per block: (1) per-slice expert histograms,
// (2) one block turns them into per-expert offsets, groups, chunks and per-(slice, expert) start positions, (3) every
// slice places its pairs: a warp takes 32 consecutive pairs, lanes with the same expert find their rank among
// themselves with match.any, the warps' counts are prefixed per expert in shared memory. The result is the same stable
// (expert, token, rank) order.
constexpr int kGrpSliceThreads = 1024;
constexpr int kGrpMaxSlices = 256;
constexpr uint32_t kGrpLargePairs = 4096;       // from this many pairs on

__host__ __device__ inline uint32_t grp_slice_len(uint32_t n, uint32_t slices) {
    const uint32_t per = (n + slices - 1) / slices;
    return (per + kGrpSliceThreads - 1) / kGrpSliceThreads * kGrpSliceThreads;      // whole rounds of the block
}

__global__ void __launch_bounds__(kGrpSliceThreads)
group_count_kernel(const uint32_t* __restrict__ indices, uint32_t idx_stride, uint32_t* __restrict__ ids_out, uint32_t n, uint32_t E,
                   uint32_t slice_len, uint32_t* __restrict__ slice_hist, const PeerWait peer_wait) {
    __shared__ uint32_t hist[TF_MAX_ROUTER_EXPERTS];
    pdl_launch_dependents();
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) hist[i] = 0;
    pdl_wait();
    peer_wait_in_block(peer_wait);
    __syncthreads();
    const uint32_t lo = blockIdx.x * slice_len, hi = lo + slice_len < n ? lo + slice_len : n;
    for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        uint32_t ex = indices[(size_t)i * idx_stride];
        if (ids_out) ids_out[i] = ex;
        if (ex == 0xFFFFFFFFu) continue;
        if (ex >= E) ex = E - 1;
        atomicAdd(&hist[ex], 1u);
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) slice_hist[(size_t)blockIdx.x * E + i] = hist[i];
}

__global__ void __launch_bounds__(TF_MAX_ROUTER_EXPERTS)
group_scan_kernel(const uint32_t* __restrict__ slice_hist, uint32_t* __restrict__ slice_start, uint32_t slices, uint32_t n, uint32_t E,
                  uint32_t* __restrict__ per_expert_offsets, uint32_t* __restrict__ per_expert_counts, tf_group* __restrict__ groups,
                  uint32_t* __restrict__ chunk_group, uint32_t* __restrict__ chunk_start, uint32_t* __restrict__ counters) {
    __shared__ uint32_t wtot[3][TF_MAX_ROUTER_EXPERTS / kWarp];
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t e = threadIdx.x, lane = threadIdx.x % kWarp, warp = threadIdx.x / kWarp, nwarps = blockDim.x / kWarp;
    // per expert: total count over the slices (independent loads, no stores in between)
    uint32_t cnt = 0;
    if (e < E) {
#pragma unroll 8
        for (uint32_t b = 0; b < slices; ++b) cnt += slice_hist[(size_t)b * E + e];
    }
    const uint32_t nch = (cnt + (uint32_t)kChunkTokens - 1) / (uint32_t)kChunkTokens;
    uint32_t i_off = cnt, i_g = cnt ? 1u : 0u, i_ch = nch;
#pragma unroll
    for (int o = 1; o < kWarp; o <<= 1) {
        const uint32_t a = __shfl_up_sync(kFullMask, i_off, o), b2 = __shfl_up_sync(kFullMask, i_g, o), c = __shfl_up_sync(kFullMask, i_ch, o);
        if ((int)lane >= o) { i_off += a; i_g += b2; i_ch += c; }
    }
    if (lane == kWarp - 1) { wtot[0][warp] = i_off; wtot[1][warp] = i_g; wtot[2][warp] = i_ch; }
    __syncthreads();
    uint32_t p_off = 0, p_g = 0, p_ch = 0, t_off = 0, t_g = 0, t_ch = 0;
    for (uint32_t v = 0; v < nwarps; ++v) {
        if (v < warp) { p_off += wtot[0][v]; p_g += wtot[1][v]; p_ch += wtot[2][v]; }
        t_off += wtot[0][v]; t_g += wtot[1][v]; t_ch += wtot[2][v];
    }
    const uint32_t my_off = p_off + i_off - cnt, my_g = p_g + i_g - (cnt ? 1u : 0u), my_ch = p_ch + i_ch - nch;
    if (e < E) {
        per_expert_counts[e] = cnt;
        per_expert_offsets[e] = cnt ? my_off : 0xFFFFFFFFu;
        if (cnt) {
            groups[my_g] = tf_group{e, my_off, cnt};
            chunk_start[my_g] = my_ch;
            for (uint32_t j = 0; j < nch; ++j) chunk_group[my_ch + j] = my_g;
        }
        // where each slice's pairs of this expert start
        uint32_t running = my_off;
#pragma unroll 8
        for (uint32_t b = 0; b < slices; ++b) {
            slice_start[(size_t)b * E + e] = running;
            running += slice_hist[(size_t)b * E + e];
        }
    }
    if (threadIdx.x == 0) { counters[0] = t_g; counters[1] = t_ch; counters[2] = n; counters[3] = t_off; }
}

__global__ void __launch_bounds__(kGrpSliceThreads)
group_place_kernel(const uint32_t* __restrict__ indices, uint32_t idx_stride, const uint16_t* __restrict__ weights, uint32_t n, uint32_t K,
                   uint32_t E, uint32_t slice_len, const uint32_t* __restrict__ slice_start, tf_pair* __restrict__ sorted_pairs) {
    __shared__ uint32_t wcnt[kGrpSliceThreads / kWarp][TF_MAX_ROUTER_EXPERTS];     // per warp and expert: count, then start
    __shared__ uint32_t run[TF_MAX_ROUTER_EXPERTS];                                // next free position per expert
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t lane = threadIdx.x % kWarp, warp = threadIdx.x / kWarp;
    constexpr uint32_t kWarps = kGrpSliceThreads / kWarp;
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) run[i] = slice_start[(size_t)blockIdx.x * E + i];
    const uint32_t lo = blockIdx.x * slice_len, hi = lo + slice_len < n ? lo + slice_len : n;
    for (uint32_t base = lo; base < hi; base += kGrpSliceThreads) {        // uniform trip count: slice_len is whole rounds
        for (uint32_t i = threadIdx.x; i < kWarps * E; i += blockDim.x) (&wcnt[0][0])[(i / E) * TF_MAX_ROUTER_EXPERTS + i % E] = 0;
        __syncthreads();
        const uint32_t i = base + threadIdx.x;
        uint32_t ex = 0xFFFFFFFFu;
        if (i < hi) {
            ex = indices[(size_t)i * idx_stride];
            if (ex != 0xFFFFFFFFu && ex >= E) ex = E - 1;
        }
        const bool valid = ex != 0xFFFFFFFFu;
        const uint32_t peers = __match_any_sync(kFullMask, ex);            // invalid lanes match one another and are ignored
        const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
        if (valid && rank == 0) wcnt[warp][ex] = __popc(peers);
        __syncthreads();
        for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) {
            uint32_t acc = run[e];
            for (uint32_t w2 = 0; w2 < kWarps; ++w2) {
                const uint32_t c = wcnt[w2][e];
                wcnt[w2][e] = acc;
                acc += c;
            }
            run[e] = acc;
        }
        __syncthreads();
        if (valid) sorted_pairs[wcnt[warp][ex] + rank] = tf_pair{i / K, ex, i % K, (uint32_t)weights[i]};
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// grouped small-batch expert kernels
// ---------------------------------------------------------------------------

constexpr int kGPW = 4;                 // 64-column groups per compute warp
constexpr int kWStages = 3;             // ring depth (items) of the tile ring (codes + scales)
// Narrow single-matrix tiles (the routed down projection: 16 rows x 352 bytes) are a few KB each, so three of them in
// flight per CTA leave the memory system idle; their ring is deeper.
template <int NMAT, int KC>
__host__ __device__ constexpr uint32_t ring_stages() { return (NMAT == 1 && KC > 0 && KC <= 1024) ? 8u : (uint32_t)kWStages; }
constexpr int kReducers = 2;            // reducer warps; reducer q owns the items and the partial buffer of parity q
constexpr int kRedStages = kReducers;   // partial-sum buffers
constexpr int kTileRows = 16;           // weight rows per MMA tile (the m of m16n8k16)
constexpr int kRowsPerCopy = 4;         // rows per bulk copy when the rows need padding against bank conflicts
// Row m of the MMA tile (m = g for the a0/a2 registers, g + 8 for a1/a3) is weight row tile_row(m) of the 16-row tile:
// the four rows that one half warp reads in one shared-memory pass (m = 4j ... 4j + 3) then lie in the four different
// 4-row blocks of the ring stage, whose paddings put them 32 bytes apart in the banks. No conflicts, four rows per copy.
__host__ __device__ constexpr uint32_t tile_row(uint32_t m) { return 4u * (m & 3u) + (m >> 2); }
constexpr int kMaxComputeWarps = 12;    // K <= 12 * 256 = 3072 columns
constexpr uint32_t kErrTimeoutCodes = 0x7F000001u;   // device error words
constexpr uint32_t kErrTimeoutPartials = 0x7F000003u;
constexpr uint32_t kErrTimeoutRedFree = 0x7F000004u;
constexpr uint32_t kErrTimeoutStageFree = 0x7F000005u;
constexpr int kExtraWarps = kReducers + 1;   // reducers + loader

struct MatPlanes {
    const uint8_t* W;
    const uint16_t* S;
    const uint16_t* B;
};

// Arguments shared by the gate/up (NMAT = 2) and down (NMAT = 1) kernels.
struct GroupedArgs {
    // routed mode: blobs at pool_base + expert * stride with these plane offsets
    const uint8_t* pool_base;
    uint64_t expert_stride;
    uint32_t w_off[2], s_off[2], b_off[2];
    // dense mode (one matrix set for all tokens)
    MatPlanes dense[2];
    // routing metadata (routed mode)
    const tf_pair* sorted_pairs;
    const tf_group* groups;
    const uint32_t* chunk_group;
    const uint32_t* chunk_start;
    const uint32_t* counters;
    // activations in: row r of the chunk's tokens at x + row_index * x_stride (elements)
    const uint16_t* x;
    uint32_t x_stride;
    // out
    void* out;
    uint32_t out_stride;       // elements between consecutive output rows
    uint32_t rows;             // weight rows (F for gate/up, D for down)
    uint32_t k;                // columns (D for gate/up, F for down)
    uint32_t top_k;
    uint32_t dense_tokens;     // dense mode: number of tokens
    uint32_t* error;           // device word: 0, or the code of the wait that gave up
};

// D = A * B + C with C either the constant zero (first MMA of a group) or D itself.
// A = codes of weight rows g (a0, a2) and g + 8 (a1, a3); B = activations of token g.
__device__ __forceinline__ void mma16816_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, const uint2& b,
                                               const float (&z)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y), "f"(z[0]), "f"(z[1]), "f"(z[2]), "f"(z[3]));
}
__device__ __forceinline__ void mma16816_acc(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, const uint2& b) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t hmul2_sixteenth(uint32_t v) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&v), __half2half2(__float2half_rn(0.0625f)));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 lds_f32x4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts_f32x2(uint32_t addr, float a, float b) {
    asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}


enum OutMode { kOutActs = 0, kOutPartialF16 = 1, kOutPartialF32 = 2, kOutDenseF16 = 3 };

// Ring row stride: rows of a tile must start on different banks for the 8-rows-by-8-bytes fragment
// loads. A stride of 8 (mod 32) words does that for each half warp; strides that already satisfy it
// (or 24 mod 32) are kept, so the whole tile is one contiguous copy.
__host__ __device__ inline uint32_t ring_row_stride(uint32_t row_bytes) {
    const uint32_t words = (row_bytes / 4) % 32;
    if (words == 8 || words == 24) return row_bytes;
    return row_bytes + ((8 + 32 - words) % 32) * 4;
}

// Shared-memory layout of a CTA with `cw` compute warps.
template <int NMAT>
struct KSplitSmem {
    uint32_t cw, ng, row_bytes, stages;
    // Rows whose natural stride would put a half warp's four rows on the same banks get 32 bytes of padding per
    // kRowsPerCopy rows: the loader moves kRowsPerCopy rows per bulk copy (a copy has a fixed cost of some tens of cycles
    // in the copy engine, and sixteen single-row copies per matrix kept the compute warps waiting for a third of an
    // item's time); the row permutation tile_row keeps the fragment loads free of bank conflicts all the same.
    __host__ __device__ uint32_t row_pad() const { return ring_row_stride(row_bytes) - row_bytes; }
    // weight row of the tile behind MMA row m: permuted when the rows are padded per block of kRowsPerCopy (see tile_row),
    // the identity when the natural row stride already spreads a half warp's rows over the banks
    __host__ __device__ uint32_t mma_row(uint32_t m) const { return row_pad() ? tile_row(m) : m; }
    __host__ __device__ uint32_t rows_per_copy() const { return row_pad() ? (uint32_t)kRowsPerCopy : (uint32_t)kTileRows; }
    __host__ __device__ uint32_t row_off(uint32_t r) const { return r * row_bytes + (r / rows_per_copy()) * row_pad(); }
    __host__ __device__ uint32_t mat_bytes() const { return kTileRows * row_bytes + (kTileRows / rows_per_copy()) * row_pad(); }
    __host__ __device__ uint32_t sb_plane_bytes() const { return kTileRows * ng * 2; }                            // multiple of 16
    __host__ __device__ uint32_t stage_bytes() const { return NMAT * mat_bytes() + NMAT * 2 * sb_plane_bytes(); } // codes, then scales
    __host__ __device__ uint32_t off_sb_in_stage() const { return NMAT * mat_bytes(); }
    __host__ __device__ uint32_t ring_bytes() const { return stages * stage_bytes(); }
    __host__ __device__ uint32_t red_stage_bytes() const { return cw * NMAT * 128 * 4; }
    __host__ __device__ uint32_t red_bytes() const { return kRedStages * red_stage_bytes(); }
    __host__ __device__ uint32_t bar_count() const { return 2 * stages + 2 * kRedStages; }
    __host__ __device__ uint32_t off_red() const { return ring_bytes(); }
    __host__ __device__ uint32_t off_bar() const { return off_red() + red_bytes(); }
    __host__ __device__ size_t total() const { return (size_t)off_bar() + (size_t)bar_count() * 8; }
};

// Where a warp is in its CTA's item sequence and what the chunk resolves to.
template <int NMAT>
struct ItemCursor {
    uint32_t chunk, tile;
    MatPlanes pl[NMAT];
    uint32_t ntok, row_base;
};

template <int NMAT, bool DENSE>
__device__ __forceinline__ void resolve_chunk(const GroupedArgs& args, ItemCursor<NMAT>& c) {
    if constexpr (DENSE) {
#pragma unroll
        for (int m = 0; m < NMAT; ++m) c.pl[m] = args.dense[m];
        c.row_base = c.chunk * kChunkTokens;
        const uint32_t left = args.dense_tokens - c.row_base;
        c.ntok = left < (uint32_t)kChunkTokens ? left : (uint32_t)kChunkTokens;
    } else {
        const uint32_t gi = args.chunk_group[c.chunk];
        const tf_group grp = args.groups[gi];
        const uint32_t cin = c.chunk - args.chunk_start[gi];
        const uint8_t* blob = args.pool_base + (uint64_t)grp.expert * args.expert_stride;
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
            c.pl[m].W = blob + args.w_off[m];
            c.pl[m].S = reinterpret_cast<const uint16_t*>(blob + args.s_off[m]);
            c.pl[m].B = reinterpret_cast<const uint16_t*>(blob + args.b_off[m]);
        }
        c.row_base = grp.pair_start + cin * kChunkTokens;
        const uint32_t left = grp.pair_count - cin * kChunkTokens;
        c.ntok = left < (uint32_t)kChunkTokens ? left : (uint32_t)kChunkTokens;
    }
}

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
// KC > 0 fixes the column count at compile time (the production shapes), so that the shared-memory layout, the
// warp count and every loop bound fold into constants; KC = 0 reads them from the arguments.
template <int NMAT, bool DENSE, int OUT_MODE, int KC>
__global__ void __launch_bounds__((KC ? (KC / kGroup + kGPW - 1) / kGPW : kMaxComputeWarps) * kWarp + kExtraWarps * kWarp)
grouped_ksplit_kernel(const GroupedArgs args) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t ng = KC ? (uint32_t)(KC / kGroup) : args.k / kGroup;
    const uint32_t cw = KC ? (ng + kGPW - 1) / kGPW : blockDim.x / kWarp - kExtraWarps;  // compute warps; then the reducers; the last warp loads
    const uint32_t row_bytes = KC ? (uint32_t)(KC / 2) : args.k / 2;
    constexpr uint32_t kSt = ring_stages<NMAT, KC>();
    const KSplitSmem<NMAT> lay{cw, ng, row_bytes, kSt};
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t red_base = smem_base + lay.off_red();
    const uint32_t bar_base = smem_base + lay.off_bar();
    // mbarriers: full[stage] | empty[stage] | part_full[r] | red_free[r]
    auto bar_full = [&](uint32_t st) { return bar_base + st * 8; };
    auto bar_empty = [&](uint32_t st) { return bar_base + (kSt + st) * 8; };
    auto bar_part_full = [&](uint32_t r) { return bar_base + (2 * kSt + r) * 8; };
    auto bar_red_free = [&](uint32_t r) { return bar_base + (2 * kSt + kRedStages + r) * 8; };

    const uint32_t tiles = args.rows / kTileRows;
    pdl_launch_dependents();
    pdl_wait();              // routing metadata and activations come from the kernels before this one
    const uint32_t total_chunks = DENSE ? (args.dense_tokens + kChunkTokens - 1) / kChunkTokens : args.counters[1];
    const uint32_t total_items = total_chunks * tiles;
    // contiguous item range per CTA: consecutive items share the chunk, whose activations stay in registers
    const uint32_t item_begin = (uint32_t)((uint64_t)total_items * blockIdx.x / gridDim.x);
    const uint32_t item_end = (uint32_t)((uint64_t)total_items * (blockIdx.x + 1) / gridDim.x);
    if (item_begin >= item_end) return;
    const uint32_t n_items = item_end - item_begin;

    if (threadIdx.x == 0) {
        for (uint32_t st = 0; st < kSt; ++st) { mbar_init(bar_full(st), 1); mbar_init(bar_empty(st), cw); }
        for (uint32_t r = 0; r < (uint32_t)kRedStages; ++r) { mbar_init(bar_part_full(r), cw); mbar_init(bar_red_free(r), 1); }
        fence_proxy_async();
    }
    __syncthreads();

    auto advance = [&](ItemCursor<NMAT>& c) {
        if (++c.tile == tiles) {
            c.tile = 0;
            ++c.chunk;
            if (c.chunk < total_chunks) resolve_chunk<NMAT, DENSE>(args, c);
        }
    };

    auto advance_by = [&](ItemCursor<NMAT>& c, uint32_t n) {
        for (uint32_t i = 0; i < n; ++i) advance(c);
    };

    if ((uint32_t)warp < cw) {
        // =========================== compute warp ===========================
        const uint32_t g0 = warp * kGPW;
        const uint32_t ngw = ng - g0 < (uint32_t)kGPW ? ng - g0 : (uint32_t)kGPW;     // g0 < ng by construction
        const bool sb_vec = (ng % 4) == 0;
        const uint32_t r_lo = lay.mma_row(g), r_hi = lay.mma_row(g + 8);                       // weight rows behind MMA rows g and g + 8
        const uint32_t sb_row0 = (r_lo * ng + g0) * 2, sb_row1 = (r_hi * ng + g0) * 2;   // their scale rows
        const uint32_t lane_code_off = lay.row_off(r_lo) + g0 * 32 + t * 8;              // this lane's codes of MMA row g within a matrix tile
        const uint32_t row8_off = lay.row_off(r_hi) - lay.row_off(r_lo);                 // MMA row g + 8

        ItemCursor<NMAT> cur;
        cur.chunk = item_begin / tiles;
        cur.tile = item_begin % tiles;
        resolve_chunk<NMAT, DENSE>(args, cur);

        // Four registers that stay zero: the accumulator input of every group's first MMA (a literal zero makes the
        // compiler clear four fresh registers per MMA).
        float zc[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) asm volatile("mov.f32 %0, 0f00000000;" : "=f"(zc[j]));
        uint2 xb[kGPW][4];          // B fragments of token g: [group][MMA j] = {b0, b1}
        float2 xsum[kGPW];          // fp32 sums of the 64 activations of the group for tokens 2t and 2t + 1
        uint32_t loaded_chunk = 0xFFFFFFFFu;
        uint32_t fail = 0;

        uint32_t st = 0, use = 0;            // ring slot of item li and how often the ring has wrapped
        for (uint32_t li = 0; li < n_items; ++li, st = st + 1 == kSt ? 0u : st + 1, use += st == 0 ? 1u : 0u) {
            if (cur.chunk != loaded_chunk) {
                // activations of this warp's columns for the chunk's token g, in MMA operand order: the 16 values
                // x0..x15 at columns 64 G + 16 t feed four MMAs,
                //   j = 0: (x0,x4),(x2,x6)   j = 1: (x1,x5)/16,(x3,x7)/16   j = 2, 3: the same for x8..x15;
                // odd columns are pre-scaled by 1/16 because their codes sit four mantissa bits higher.
                loaded_chunk = cur.chunk;
#pragma unroll
                for (int i = 0; i < kGPW; ++i) {
                    uint32_t r[8];
                    if ((uint32_t)i < ngw && (uint32_t)g < cur.ntok) {
                        const uint32_t rr = (DENSE || NMAT == 1) ? cur.row_base + g : args.sorted_pairs[cur.row_base + g].token;
                        const uint4* p = reinterpret_cast<const uint4*>(args.x + (size_t)rr * args.x_stride + (g0 + i) * kGroup + t * 16);
                        const uint4 lo = __ldg(p), hi = __ldg(p + 1);
                        r[0] = lo.x; r[1] = lo.y; r[2] = lo.z; r[3] = lo.w;
                        r[4] = hi.x; r[5] = hi.y; r[6] = hi.z; r[7] = hi.w;
                    } else {
#pragma unroll
                        for (int q = 0; q < 8; ++q) r[q] = 0;
                    }
                    float sum = 0.0f;
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&r[q]));
                        sum += v.x + v.y;
                    }
                    sum += __shfl_xor_sync(kFullMask, sum, 1);
                    sum += __shfl_xor_sync(kFullMask, sum, 2);        // every lane of quad g holds token g's group sum
                    // The codes enter the MMA as q * 2^-24, so the whole row sum is carried at 2^-24 of its value (the group
                    // sums are scaled to match here, once per chunk) and multiplied back once per item: powers of two, exact.
                    sum *= 5.9604644775390625e-08f;
                    xsum[i] = make_float2(__shfl_sync(kFullMask, sum, 8 * t), __shfl_sync(kFullMask, sum, 8 * t + 4));
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        const int o = 4 * h2;
                        xb[i][2 * h2] = make_uint2(prmt(r[o], r[o + 2], 0x5410), prmt(r[o + 1], r[o + 3], 0x5410));
                        xb[i][2 * h2 + 1] = make_uint2(hmul2_sixteenth(prmt(r[o], r[o + 2], 0x7632)),
                                                       hmul2_sixteenth(prmt(r[o + 1], r[o + 3], 0x7632)));
                    }
                }
            }
            if (!mbar_wait(bar_full(st), use & 1)) { fail = kErrTimeoutCodes; break; }

            const uint32_t ring_item = smem_base + st * lay.stage_bytes() + lane_code_off;
            const uint32_t sb_item = smem_base + st * lay.stage_bytes() + lay.off_sb_in_stage();
            // All codes of the item first, then the MMAs interleaved over the (matrix, group) pairs: the four
            // MMAs of one group form a dependent chain through its accumulator, so consecutive instructions
            // always belong to different chains and the tensor pipe stays full.
            uint2 wa[NMAT][kGPW], wb[NMAT][kGPW];          // codes of rows g and g + 8
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
#pragma unroll
                for (int i = 0; i < kGPW; ++i) {
                    // Groups past this warp's range (the last warp of a K that is not a multiple of 256) read the bytes that
                    // follow the row inside the stage (padding, the next row, the scale planes): masked nibbles are finite
                    // and meet zero activations, so they add exact zeros and need no predicate.
                    wa[m][i] = lds64(ring_item + m * lay.mat_bytes() + i * 32);
                    wb[m][i] = lds64(ring_item + m * lay.mat_bytes() + row8_off + i * 32);
                }
            }
            float c[NMAT][kGPW][4];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
#pragma unroll
                for (int i = 0; i < kGPW; ++i)
                    mma16816_first(c[m][i], wa[m][i].x & 0x000F000Fu, wb[m][i].x & 0x000F000Fu,
                                   (wa[m][i].x >> 8) & 0x000F000Fu, (wb[m][i].x >> 8) & 0x000F000Fu, xb[i][0], zc);
            }
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
#pragma unroll
                for (int i = 0; i < kGPW; ++i)
                    mma16816_acc(c[m][i], wa[m][i].x & 0x00F000F0u, wb[m][i].x & 0x00F000F0u,
                                 (wa[m][i].x >> 8) & 0x00F000F0u, (wb[m][i].x >> 8) & 0x00F000F0u, xb[i][1]);
            }
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
#pragma unroll
                for (int i = 0; i < kGPW; ++i)
                    mma16816_acc(c[m][i], wa[m][i].y & 0x000F000Fu, wb[m][i].y & 0x000F000Fu,
                                 (wa[m][i].y >> 8) & 0x000F000Fu, (wb[m][i].y >> 8) & 0x000F000Fu, xb[i][2]);
            }
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
#pragma unroll
                for (int i = 0; i < kGPW; ++i)
                    mma16816_acc(c[m][i], wa[m][i].y & 0x00F000F0u, wb[m][i].y & 0x00F000F0u,
                                 (wa[m][i].y >> 8) & 0x00F000F0u, (wb[m][i].y >> 8) & 0x00F000F0u, xb[i][3]);
            }
            float y[NMAT][4];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                const uint32_t sm_s = sb_item + (m * 2) * lay.sb_plane_bytes(), sm_b = sm_s + lay.sb_plane_bytes();
                // scale and bias of weight rows g (index 0) and g + 8 (index 1) for this warp's groups, as fp32
                float sf[2][kGPW], bf[2][kGPW];
                if (sb_vec) {
                    const uint2 vs0 = lds64(sm_s + sb_row0), vs1 = lds64(sm_s + sb_row1);
                    const uint2 vb0 = lds64(sm_b + sb_row0), vb1 = lds64(sm_b + sb_row1);
#pragma unroll
                    for (int i = 0; i < kGPW; ++i) {
                        const uint32_t sv0 = i < 2 ? vs0.x : vs0.y, sv1 = i < 2 ? vs1.x : vs1.y;
                        const uint32_t bv0 = i < 2 ? vb0.x : vb0.y, bv1 = i < 2 ? vb1.x : vb1.y;
                        sf[0][i] = (i & 1) ? bf16_hi(sv0) : bf16_lo(sv0); sf[1][i] = (i & 1) ? bf16_hi(sv1) : bf16_lo(sv1);
                        bf[0][i] = (i & 1) ? bf16_hi(bv0) : bf16_lo(bv0); bf[1][i] = (i & 1) ? bf16_hi(bv1) : bf16_lo(bv1);
                    }
                } else {
                    // groups beyond this warp's range carry zero activations; their scale words are forced to zero so that
                    // whatever follows the plane in the stage cannot turn 0 * x into a NaN
#pragma unroll
                    for (int i = 0; i < kGPW; ++i) {
                        const bool ok = (uint32_t)i < ngw;
                        sf[0][i] = ok ? bf16_lo(lds16(sm_s + sb_row0 + i * 2)) : 0.0f; sf[1][i] = ok ? bf16_lo(lds16(sm_s + sb_row1 + i * 2)) : 0.0f;
                        bf[0][i] = ok ? bf16_lo(lds16(sm_b + sb_row0 + i * 2)) : 0.0f; bf[1][i] = ok ? bf16_lo(lds16(sm_b + sb_row1 + i * 2)) : 0.0f;
                    }
                }
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int i = 0; i < kGPW; ++i) {
                    // c0, c1: weight row g, tokens 2t, 2t+1; c2, c3: weight row g + 8
                    acc[0] = fmaf(sf[0][i], c[m][i][0], fmaf(bf[0][i], xsum[i].x, acc[0]));
                    acc[1] = fmaf(sf[0][i], c[m][i][1], fmaf(bf[0][i], xsum[i].y, acc[1]));
                    acc[2] = fmaf(sf[1][i], c[m][i][2], fmaf(bf[1][i], xsum[i].x, acc[2]));
                    acc[3] = fmaf(sf[1][i], c[m][i][3], fmaf(bf[1][i], xsum[i].y, acc[3]));
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) y[m][j] = acc[j] * 16777216.0f;
            }
            // this warp is done with the stage (codes and scales are in registers or consumed)
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty(st));
            // hand the partial sums to the reducer
            const uint32_t r = li % kRedStages, ruse = li / kRedStages;
            if (!mbar_wait(bar_red_free(r), (ruse & 1) ^ 1)) { fail = kErrTimeoutRedFree; break; }

            const uint32_t red_w = red_base + r * lay.red_stage_bytes() + (warp * NMAT) * 512 + (g * 8 + 2 * t) * 4;
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                sts_f32x2(red_w + m * 512, y[m][0], y[m][1]);
                sts_f32x2(red_w + m * 512 + 256, y[m][2], y[m][3]);      // weight row g + 8: index (g + 8) * 8 + 2t
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_part_full(r));
            if (li + 1 < n_items) advance(cur);
        }
        if (fail && lane == 0) atomicCAS(args.error, 0u, fail);
    } else if ((uint32_t)warp == cw + kReducers) {
        // =========================== loader warp ===========================
        ItemCursor<NMAT> iss;
        iss.chunk = item_begin / tiles;
        iss.tile = item_begin % tiles;
        resolve_chunk<NMAT, DENSE>(args, iss);
        const uint32_t plane_bytes = lay.sb_plane_bytes();
        const uint32_t rpc = lay.rows_per_copy();                    // 16: the rows of a tile land as one copy
        const uint32_t tx_bytes = NMAT * kTileRows * row_bytes + NMAT * 2 * plane_bytes;
        uint32_t fail = 0, issued = 0;
        uint32_t st = 0, use = 0;
        for (uint32_t li = 0; li < n_items; ++li, st = st + 1 == kSt ? 0u : st + 1, use += st == 0 ? 1u : 0u) {
            if (use > 0 && !mbar_wait(bar_empty(st), (use - 1) & 1)) { fail = kErrTimeoutStageFree; break; }
            const uint32_t mbar = bar_full(st);
            const uint32_t stage = smem_base + st * lay.stage_bytes();
            if (lane == 0) {
                fence_proxy_async();          // the stage was last read through the generic proxy
                mbar_arrive_expect_tx(mbar, tx_bytes);
            }
            __syncwarp();
            for (uint32_t j = lane; j < (uint32_t)(NMAT * kTileRows) / rpc; j += kWarp) {
                const uint32_t per_mat = kTileRows / rpc, m = j / per_mat, r = (j % per_mat) * rpc;
                const MatPlanes& mp = m ? iss.pl[NMAT - 1] : iss.pl[0];
                bulk_copy_g2s(stage + m * lay.mat_bytes() + lay.row_off(r),
                              mp.W + (size_t)(iss.tile * kTileRows + r) * row_bytes, rpc * row_bytes, mbar);
            }
            if (lane < NMAT * 2) {
                const uint32_t m = lane >> 1, which = lane & 1;
                const MatPlanes& mp = m ? iss.pl[NMAT - 1] : iss.pl[0];
                const uint16_t* plane = which ? mp.B : mp.S;
                bulk_copy_g2s(stage + lay.off_sb_in_stage() + lane * plane_bytes, plane + (size_t)iss.tile * kTileRows * ng,
                              plane_bytes, mbar);
            }
            ++issued;
            if (li + 1 < n_items) advance(iss);
        }
        if (fail) {
            if (lane == 0) atomicCAS(args.error, 0u, fail);
            // let the copies already issued land before the CTA's shared memory goes away (bounded)
            for (uint32_t st = 0; st < kSt && st < issued; ++st)
                for (uint32_t par = 0; par < 2; ++par) mbar_wait(bar_full(st), par);
        }
    } else {
        // =========================== reducer warp q ===========================
        // Reducer q handles the items of parity q (and with them partial buffer q and scale stages q, q + 2).
        const uint32_t q = warp - cw;
        ItemCursor<NMAT> cur;
        cur.chunk = item_begin / tiles;
        cur.tile = item_begin % tiles;
        resolve_chunk<NMAT, DENSE>(args, cur);
        if (q < n_items) advance_by(cur, q);
        uint32_t fail = 0;
        const uint32_t row = lay.mma_row(lane >> 1), tok4 = (lane & 1) * 4;      // this lane sums one weight row (MMA row lane / 2) for 4 consecutive tokens
        const uint32_t red_q = red_base + q * lay.red_stage_bytes() + lane * 16;
        uint32_t pair_chunk = 0xFFFFFFFFu;
        uint32_t pair_base[4] = {0u, 0u, 0u, 0u};                   // (token * top_k + rank) of this lane's 4 tokens
        for (uint32_t li = q; li < n_items; li += kReducers) {
            const uint32_t ruse = li / kRedStages;
            if (OUT_MODE == kOutPartialF16 || OUT_MODE == kOutPartialF32) {
                if (cur.chunk != pair_chunk) {       // the pair of a token is the same for every tile of the chunk
                    pair_chunk = cur.chunk;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (tok4 + j < cur.ntok) {
                            const tf_pair pr = args.sorted_pairs[cur.row_base + tok4 + j];
                            pair_base[j] = pr.token * args.top_k + pr.rank;
                        }
                    }
                }
            }
            if (!mbar_wait(bar_part_full(q), ruse & 1)) { fail = kErrTimeoutPartials; break; }
            float4 acc[NMAT];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                // independent loads first, then the sum in warp order (deterministic)
                float4 v[kMaxComputeWarps];
#pragma unroll
                for (int w2 = 0; w2 < kMaxComputeWarps; ++w2)
                    v[w2] = (uint32_t)w2 < cw ? lds_f32x4(red_q + (w2 * NMAT + m) * 512) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                acc[m] = v[0];
#pragma unroll
                for (int w2 = 1; w2 < kMaxComputeWarps; ++w2) {
                    if ((uint32_t)w2 < cw) { acc[m].x += v[w2].x; acc[m].y += v[w2].y; acc[m].z += v[w2].z; acc[m].w += v[w2].w; }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_red_free(q));
            const uint32_t out_row = cur.tile * kTileRows + row;
            const float o0[4] = {acc[0].x, acc[0].y, acc[0].z, acc[0].w};
            const float o1[4] = {acc[NMAT - 1].x, acc[NMAT - 1].y, acc[NMAT - 1].z, acc[NMAT - 1].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t tok = tok4 + j;
                if (tok < cur.ntok) {
                    if constexpr (OUT_MODE == kOutActs) {
                        float gt = o0[j], up = o1[j];
                        if constexpr (DENSE) {
                            // shared expert: gate and up are stored as fp16 before the activation
                            // (Kernels/MoE/SharedExpertInt4.swift:62-93; Metal/Primitives/utility.metal:15-17)
                            gt = __half2float(__float2half_rn(gt));
                            up = __half2float(__float2half_rn(up));
                        }
                        // routed: act = half(gelu_tanh(gate) * up), gate and up in fp32 (prefill.metal:634-636; moe.metal:368)
                        static_cast<uint16_t*>(args.out)[(size_t)(cur.row_base + tok) * args.out_stride + out_row] =
                            __half_as_ushort(__float2half_rn(gelu_tanh(gt) * up));
                    } else if constexpr (OUT_MODE == kOutDenseF16) {
                        static_cast<uint16_t*>(args.out)[(size_t)(cur.row_base + tok) * args.out_stride + out_row] =
                            __half_as_ushort(__float2half_rn(o0[j]));
                    } else {
                        const size_t idx = (size_t)pair_base[j] * args.out_stride + out_row;
                        if constexpr (OUT_MODE == kOutPartialF16)       // prefill.metal:666-669
                            static_cast<uint16_t*>(args.out)[idx] = __half_as_ushort(__float2half_rn(o0[j]));
                        else
                            static_cast<float*>(args.out)[idx] = o0[j];
                    }
                }
            }
            if (li + kReducers < n_items) advance_by(cur, kReducers);
        }
        if (fail && lane == 0) atomicCAS(args.error, 0u, fail);
    }
}

}  // namespace tf

// ---------------------------------------------------------------------------
// combine
// ---------------------------------------------------------------------------
namespace tf {

// PARTIAL_F32 = false: the reference's token-major reduce (Metal/Prefill/prefill.metal:575-596):
//     h2[t,d] = half(sum_r fma(float(w[t,r]), float(partial[t,r,d]), acc)) (+ residual in fp32 when given)
// PARTIAL_F32 = true: the decode kernel's order (Metal/MoE/moe.metal:473-480):
//     acc = float(residual[d]); acc += float(w_r) * partial_r, r = 0..K-1; y = half(acc)
template <bool PARTIAL_F32>
__global__ void reduce_token_major_kernel(const void* __restrict__ partials, const uint16_t* __restrict__ weights,
                                          const uint16_t* __restrict__ residual, uint32_t residual_stride,
                                          uint16_t* __restrict__ out, uint32_t out_stride,
                                          uint32_t T, uint32_t K, uint32_t D) {
    const uint32_t d = blockIdx.y * blockDim.x + threadIdx.x;      // rows in grid.x: no 65535 limit on the token count
    const uint32_t t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (d >= D || t >= T) return;
    float acc;
    if constexpr (PARTIAL_F32) {
        acc = residual ? f16_bits_to_float(residual[(size_t)t * residual_stride + d]) : 0.0f;
        const float* p = static_cast<const float*>(partials);
        for (uint32_t r = 0; r < K; ++r)
            acc = __fadd_rn(acc, __fmul_rn(f16_bits_to_float(weights[(size_t)t * K + r]), p[((size_t)t * K + r) * D + d]));
    } else {
        acc = 0.0f;
        const uint16_t* p = static_cast<const uint16_t*>(partials);
        for (uint32_t r = 0; r < K; ++r)
            acc = fmaf(f16_bits_to_float(weights[(size_t)t * K + r]), f16_bits_to_float(p[((size_t)t * K + r) * D + d]), acc);
        if (residual) acc += f16_bits_to_float(residual[(size_t)t * residual_stride + d]);
    }
    out[(size_t)t * out_stride + d] = __half_as_ushort(__float2half_rn(acc));
}

template <int NMAT, bool DENSE, int OUT_MODE, int KC>
static tf_status launch_grouped_k(tf_context* ctx, void* stream, GroupedArgs& args, const char* name) {
    const uint32_t ng = args.k / kGroup;
    const uint32_t cw = (ng + kGPW - 1) / kGPW;
    const KSplitSmem<NMAT> lay{cw, ng, args.k / 2, ring_stages<NMAT, KC>()};
    const size_t smem = lay.total();
    TF_REQUIRE(ctx, smem <= 200 * 1024, TF_ERR_UNSUPPORTED, "%s: K=%u needs %zu bytes of shared memory (limit 200 KB)", name, args.k, smem);
    auto kern = grouped_ksplit_kernel<NMAT, DENSE, OUT_MODE, KC>;
    // Attribute and occupancy are queried once per (instantiation, device, warp count) and cached, so
    // steady-state calls are a bare launch (and safe inside stream capture).
    static std::mutex cache_mu;
    static int cached_per_sm[kMaxDevices][kMaxComputeWarps + 1] = {};
    const int dev = ctx->device >= 0 && ctx->device < kMaxDevices ? ctx->device : -1;
    int per_sm = 0;
    {
        std::lock_guard<std::mutex> lock(cache_mu);
        if (dev >= 0) per_sm = cached_per_sm[dev][cw];
        if (per_sm == 0) {
            TF_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            TF_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, (int)((cw + kExtraWarps) * kWarp), smem));
            if (per_sm < 1) per_sm = 1;
            if (per_sm > 8) per_sm = 8;
            if (dev >= 0) cached_per_sm[dev][cw] = per_sm;
        }
    }
    args.error = ctx->device_error;
    uint32_t grid = (uint32_t)ctx->sm_count * (uint32_t)per_sm;
    if (DENSE) {
        const uint64_t items = (uint64_t)((args.dense_tokens + kChunkTokens - 1) / kChunkTokens) * (args.rows / kTileRows);
        if (items == 0) return TF_OK;
        if (items < grid) grid = (uint32_t)items;
    }
    launch_pdl(kern, dim3(grid), dim3((cw + kExtraWarps) * kWarp), smem, static_cast<cudaStream_t>(stream), args);
    return check_launch(ctx, name);
}

// KSPEC: the column count this instantiation is specialised for (the Gemma-4 shape of its role); other
// column counts take the generic kernel.
template <int NMAT, bool DENSE, int OUT_MODE, int KSPEC>
static tf_status launch_grouped(tf_context* ctx, void* stream, GroupedArgs& args, const char* name) {
    const uint32_t ng = args.k / kGroup;
    TF_REQUIRE(ctx, ng >= 1 && args.k % kGroup == 0, TF_ERR_INVALID_ARGUMENT, "%s: K must be a positive multiple of 64", name);
    const uint32_t cw = (ng + kGPW - 1) / kGPW;
    TF_REQUIRE(ctx, cw <= (uint32_t)kMaxComputeWarps, TF_ERR_UNSUPPORTED, "%s: K=%u outside the supported range (64..3072)", name, args.k);
    TF_REQUIRE(ctx, args.rows % kTileRows == 0, TF_ERR_UNSUPPORTED, "%s: row count %u must be a multiple of 16", name, args.rows);
    if (args.k == (uint32_t)KSPEC) return launch_grouped_k<NMAT, DENSE, OUT_MODE, KSPEC>(ctx, stream, args, name);
    return launch_grouped_k<NMAT, DENSE, OUT_MODE, 0>(ctx, stream, args, name);
}

static tf_status check_blob_alignment(tf_context* ctx, const void* pool, uint64_t stride, const tf_expert_offsets* o, const char* name) {
    TF_REQUIRE(ctx, o != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: offsets is NULL", name);
    TF_REQUIRE(ctx, aligned(pool, 16) && stride % 16 == 0, TF_ERR_ALIGNMENT, "%s: expert pool base and stride must be 16-byte aligned", name);
    const uint32_t all[9] = {o->gate_w_off, o->gate_s_off, o->gate_b_off, o->up_w_off, o->up_s_off, o->up_b_off,
                             o->down_w_off, o->down_s_off, o->down_b_off};
    for (uint32_t v : all)
        TF_REQUIRE(ctx, v % 16 == 0, TF_ERR_ALIGNMENT, "%s: blob sub-tensor offset %u is not a multiple of 16 bytes", name, v);
    return TF_OK;
}

// ---------------------------------------------------------------------------
// Scratch that lives in the library image, for tf_shared_expert_int4_block_noalloc
// ---------------------------------------------------------------------------
// Every GPU that loads this library carries these arrays from load until the process exits.
constexpr size_t kNoAllocScratchBytes = 1u << 20;          // 1 MiB of fp16 activations: rows * gate.rows * 2 bytes
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
static __device__ __align__(256) uint32_t g_noalloc_error_word[1];

// In host code the two names above are stand-ins, not device addresses; the addresses a kernel can use come
// from cudaGetSymbolAddress, asked once per device with that device current.
struct NoAllocDevice {
    bool ready = false;
    void* scratch = nullptr;
    uint32_t* error_word = nullptr;
    int sm_count = 0;
};
constexpr int kNoAllocMaxDevices = 64;
static NoAllocDevice g_noalloc_devices[kNoAllocMaxDevices];
static std::mutex g_noalloc_mutex;

static tf_status noalloc_device(NoAllocDevice** out, const char* name) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(nullptr, TF_ERR_NO_DEVICE, "%s: cudaGetDevice: %s", name, cudaGetErrorString(e));
    if (dev < 0 || dev >= kNoAllocMaxDevices) return fail(nullptr, TF_ERR_UNSUPPORTED, "%s: device ordinal %d is out of range", name, dev);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    NoAllocDevice& d = g_noalloc_devices[dev];
    if (!d.ready) {
        int major = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return fail(nullptr, TF_ERR_CUDA, "%s: cudaDeviceGetAttribute: %s", name, cudaGetErrorString(e));
        if (major != 10) return fail(nullptr, TF_ERR_UNSUPPORTED, "%s: device %d is not sm_100; this library is built for sm_100a only", name, dev);
        e = cudaGetSymbolAddress(&d.scratch, g_noalloc_scratch);
        if (e != cudaSuccess) return fail(nullptr, TF_ERR_CUDA, "%s: cudaGetSymbolAddress(scratch): %s", name, cudaGetErrorString(e));
        void* w = nullptr;
        e = cudaGetSymbolAddress(&w, g_noalloc_error_word);
        if (e != cudaSuccess) return fail(nullptr, TF_ERR_CUDA, "%s: cudaGetSymbolAddress(error word): %s", name, cudaGetErrorString(e));
        d.error_word = static_cast<uint32_t*>(w);
        d.ready = true;
    }
    *out = &d;
    return TF_OK;
}

}  // namespace tf

extern "C" {

}  // extern "C"

namespace tf {

// tf_group_routes_device with the ids read at a stride of `idx_stride` 32-bit words (the id tails of exchanged rows)
// and, when ids_out is given, also written out densely.
tf_status group_routes_strided(tf_context* ctx, void* stream, const uint32_t* indices, uint32_t idx_stride, uint32_t* ids_out,
                               const void* weights_f16, uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                               const tf_device_routes* routes, const char* name, const PeerWait* peer_wait) {
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, indices && weights_f16 && routes, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, routes->sorted_pairs && routes->per_expert_offsets && routes->per_expert_counts && routes->groups &&
                        routes->chunk_group && routes->chunk_start && routes->counters,
               TF_ERR_INVALID_ARGUMENT, "%s: NULL route buffer", name);
    TF_REQUIRE(ctx, top_k > 0, TF_ERR_GROUPING_INVALID_TOP_K, "topK must be positive, got %u", top_k);
    TF_REQUIRE(ctx, num_experts > 0 && num_experts <= TF_MAX_ROUTER_EXPERTS, TF_ERR_GROUPING_INVALID_NUM_EXPERTS,
               "numExperts must be in 1...256, got %u", num_experts);
    TF_REQUIRE(ctx, (uint64_t)query_count * top_k < (1ull << 31), TF_ERR_INVALID_ARGUMENT, "%s: too many pairs", name);
    TF_REQUIRE(ctx, idx_stride > 0, TF_ERR_INVALID_ARGUMENT, "%s: the id stride must be positive", name);
    const uint32_t n = query_count * top_k;
    if (n >= kGrpLargePairs && ctx->group_scratch) {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        uint32_t slices = (n + kGrpSliceThreads - 1) / kGrpSliceThreads;
        const uint32_t want = (uint32_t)ctx->sm_count;
        if (slices > want) slices = want;
        if (slices > (uint32_t)kGrpMaxSlices) slices = kGrpMaxSlices;
        const uint32_t slice_len = grp_slice_len(n, slices);
        slices = (n + slice_len - 1) / slice_len;
        const PeerWait pw = peer_wait ? *peer_wait : PeerWait{nullptr, nullptr, nullptr, 0u};
        tf::launch_pdl(tf::group_count_kernel, dim3(slices), dim3(kGrpSliceThreads), 0, st, indices, idx_stride, ids_out, n, num_experts,
                       slice_len, ctx->group_scratch, pw);
        if (tf_status s = tf::check_launch(ctx, name)) return s;
        uint32_t* slice_start = ctx->group_scratch + (size_t)kGrpMaxSlices * TF_MAX_ROUTER_EXPERTS;
        tf::launch_pdl(tf::group_scan_kernel, dim3(1), dim3(TF_MAX_ROUTER_EXPERTS), 0, st, static_cast<const uint32_t*>(ctx->group_scratch),
                       slice_start, slices, n, num_experts,
                       routes->per_expert_offsets, routes->per_expert_counts, routes->groups, routes->chunk_group, routes->chunk_start,
                       routes->counters);
        if (tf_status s = tf::check_launch(ctx, name)) return s;
        tf::launch_pdl(tf::group_place_kernel, dim3(slices), dim3(kGrpSliceThreads), 0, st, indices, idx_stride,
                       static_cast<const uint16_t*>(weights_f16), n, top_k, num_experts, slice_len,
                       static_cast<const uint32_t*>(slice_start), routes->sorted_pairs);
        return tf::check_launch(ctx, name);
    }
    tf::launch_pdl(tf::group_routes_kernel, dim3(num_experts), dim3(tf::kGroupThreads), 0, static_cast<cudaStream_t>(stream),
                   indices, idx_stride, ids_out, static_cast<const uint16_t*>(weights_f16), query_count, top_k, num_experts,
                   routes->sorted_pairs, routes->per_expert_offsets, routes->per_expert_counts, routes->groups, routes->chunk_group,
                   routes->chunk_start, routes->counters, peer_wait ? *peer_wait : PeerWait{nullptr, nullptr, nullptr, 0u});
    return tf::check_launch(ctx, name);
}

}  // namespace tf

extern "C" {

tf_status tf_group_routes_device(tf_context* ctx, void* stream, const uint32_t* indices, const void* weights_f16,
                                 uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                                 const tf_device_routes* routes) {
    return tf::group_routes_strided(ctx, stream, indices, 1, nullptr, weights_f16, query_count, top_k, num_experts, routes,
                                    "tf_group_routes_device", nullptr);
}

tf_status tf_grouped_moe_batched(tf_context* ctx, void* stream, const void* hidden, uint64_t hidden_off,
                                 uint32_t hidden_stride_elements, const void* pool_layer_base, uint64_t expert_stride,
                                 const tf_expert_offsets* offsets, const tf_device_routes* routes,
                                 void* acts_scratch, void* route_partials, int partials_f32,
                                 uint32_t query_count, uint32_t d, uint32_t f, uint32_t top_k) {
    const char* name = "tf_grouped_moe_batched";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, hidden && pool_layer_base && routes && acts_scratch && route_partials, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    if (tf_status s = tf::check_blob_alignment(ctx, pool_layer_base, expert_stride, offsets, name)) return s;
    TF_REQUIRE(ctx, d % tf::kGroup == 0 && f % tf::kGroup == 0 && d > 0 && f > 0, TF_ERR_INVALID_ARGUMENT,
               "%s: D and F must be positive multiples of 64", name);
    TF_REQUIRE(ctx, top_k > 0 && hidden_stride_elements >= d, TF_ERR_INVALID_ARGUMENT, "%s: bad topK or hidden stride", name);
    const uint8_t* hp = tf::byte_ptr(hidden, hidden_off);
    TF_REQUIRE(ctx, tf::aligned(hp, 16) && (hidden_stride_elements * 2) % 16 == 0 && tf::aligned(acts_scratch, 16),
               TF_ERR_ALIGNMENT, "%s: hidden rows and acts scratch must be 16-byte aligned", name);
    if (query_count == 0) return TF_OK;
    tf::GroupedArgs a{};
    a.pool_base = static_cast<const uint8_t*>(pool_layer_base);
    a.expert_stride = expert_stride;
    a.w_off[0] = offsets->gate_w_off; a.s_off[0] = offsets->gate_s_off; a.b_off[0] = offsets->gate_b_off;
    a.w_off[1] = offsets->up_w_off;   a.s_off[1] = offsets->up_s_off;   a.b_off[1] = offsets->up_b_off;
    a.sorted_pairs = routes->sorted_pairs; a.groups = routes->groups; a.chunk_group = routes->chunk_group;
    a.chunk_start = routes->chunk_start; a.counters = routes->counters;
    a.x = reinterpret_cast<const uint16_t*>(hp); a.x_stride = hidden_stride_elements;
    a.out = acts_scratch; a.out_stride = f; a.rows = f; a.k = d; a.top_k = top_k;
    tf_status s = tf::launch_grouped<2, false, tf::kOutActs, 2816>(ctx, stream, a, "tf_grouped_moe_batched(gate/up)");
    if (s) return s;

    tf::GroupedArgs b{};
    b.pool_base = a.pool_base; b.expert_stride = expert_stride;
    b.w_off[0] = offsets->down_w_off; b.s_off[0] = offsets->down_s_off; b.b_off[0] = offsets->down_b_off;
    b.sorted_pairs = routes->sorted_pairs; b.groups = routes->groups; b.chunk_group = routes->chunk_group;
    b.chunk_start = routes->chunk_start; b.counters = routes->counters;
    b.x = static_cast<const uint16_t*>(acts_scratch); b.x_stride = f;
    b.out = route_partials; b.out_stride = d; b.rows = d; b.k = f; b.top_k = top_k;
    if (partials_f32) return tf::launch_grouped<1, false, tf::kOutPartialF32, 704>(ctx, stream, b, "tf_grouped_moe_batched(down)");
    return tf::launch_grouped<1, false, tf::kOutPartialF16, 704>(ctx, stream, b, "tf_grouped_moe_batched(down)");
}

}  // extern "C"

namespace tf {

constexpr uint32_t kStreamedMaxPairs = 65536;       // pairs of one tf_grouped_moe_streamed call
constexpr uint32_t kErrUnboundExpert = 0x7F000031u; // a pair's expert is not among the tile's bound experts

// Scratch layout of the streamed form inside tf_context::streamed_scratch.
struct StreamedScratch {
    tf_group groups[TF_STREAMED_MAX_EXPERTS];
    uint32_t chunk_start[TF_STREAMED_MAX_EXPERTS];
    uint32_t counters[4];
    uint32_t chunk_group[kStreamedMaxPairs / kChunkTokens + TF_STREAMED_MAX_EXPERTS];
};
size_t streamed_scratch_bytes() { return sizeof(StreamedScratch); }

struct StreamedBinding {
    uint32_t expert[TF_STREAMED_MAX_EXPERTS];       // params.local_expert
    uint32_t blob16[TF_STREAMED_MAX_EXPERTS];       // (blob - lowest blob) / 16
    uint32_t live;
};

// The pairs of one tile are sorted by expert, so a bound expert's pairs are one run. One block: count the run of
// every bound expert, then emit the groups in order of appearance with the blob's encoded address in the expert
// field (the grouped kernel computes blob = base + expert * 16), and the 8-token chunk table.
__global__ void streamed_routes_kernel(const tf_pair* __restrict__ pairs, uint32_t count, const StreamedBinding bind,
                                       StreamedScratch* out, uint32_t* error) {
    __shared__ uint32_t hist[TF_STREAMED_MAX_EXPERTS], first[TF_STREAMED_MAX_EXPERTS];
    if (threadIdx.x < TF_STREAMED_MAX_EXPERTS) { hist[threadIdx.x] = 0u; first[threadIdx.x] = 0xFFFFFFFFu; }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) {
        const uint32_t e = pairs[i].expert;
        uint32_t slot = 0xFFFFFFFFu;
        for (uint32_t sl = 0; sl < bind.live; ++sl)
            if (bind.expert[sl] == e) { slot = sl; break; }
        if (slot == 0xFFFFFFFFu) { atomicCAS(error, 0u, kErrUnboundExpert); continue; }
        atomicAdd(&hist[slot], 1u);
        atomicMin(&first[slot], i);
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    uint32_t ng = 0, nch = 0;
    uint32_t last_first = 0;
    for (uint32_t round = 0; round < bind.live; ++round) {
        // next bound expert in order of appearance
        uint32_t best = 0xFFFFFFFFu, best_first = 0xFFFFFFFFu;
        for (uint32_t sl = 0; sl < bind.live; ++sl)
            if (hist[sl] && first[sl] < best_first && (round == 0 || first[sl] > last_first)) { best = sl; best_first = first[sl]; }
        if (best == 0xFFFFFFFFu) break;
        last_first = best_first;
        const uint32_t cnt = hist[best], ch = (cnt + kChunkTokens - 1) / kChunkTokens;
        out->groups[ng] = tf_group{bind.blob16[best], best_first, cnt};
        out->chunk_start[ng] = nch;
        for (uint32_t j = 0; j < ch; ++j) out->chunk_group[nch + j] = ng;
        ++ng; nch += ch;
    }
    out->counters[0] = ng; out->counters[1] = nch; out->counters[2] = count; out->counters[3] = count;
}

}  // namespace tf

extern "C" {

tf_status tf_grouped_moe_streamed(tf_context* ctx, void* stream, const void* hidden, uint64_t hidden_off,
                                  const void* sorted_pairs, uint64_t sorted_pairs_off,
                                  void* route_partials, uint64_t route_partials_off,
                                  void* gate_up_act_scratch, uint64_t gate_up_act_scratch_off,
                                  const void* const* blobs, uint32_t blob_count, const tf_streamed_params* params,
                                  uint32_t pair_microbatch_rows, uint32_t* microbatches_out) {
    const char* name = "tf_grouped_moe_streamed";
    if (microbatches_out) *microbatches_out = 0;
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, params != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: params is NULL", name);
    // PrefillGroupedRoutedMoE.swift:402-404: nothing to do, no error
    if (params->pair_count == 0 || params->live_expert_count != blob_count || pair_microbatch_rows == 0) return TF_OK;
    TF_REQUIRE(ctx, hidden && sorted_pairs && route_partials && gate_up_act_scratch && blobs, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, blob_count >= 1 && blob_count <= TF_STREAMED_MAX_EXPERTS, TF_ERR_INVALID_ARGUMENT,
               "tile binding has %u experts; expected 1...%d", blob_count, TF_STREAMED_MAX_EXPERTS);       // :188-195
    TF_REQUIRE(ctx, params->pair_count <= tf::kStreamedMaxPairs, TF_ERR_SCRATCH_TOO_SMALL, "%s: %u pairs exceed the %u a call can take",
               name, params->pair_count, tf::kStreamedMaxPairs);
    const uint32_t d = params->d, f = params->routed_intermediate;
    TF_REQUIRE(ctx, d % tf::kGroup == 0 && f % tf::kGroup == 0 && d > 0 && f > 0, TF_ERR_INVALID_ARGUMENT,
               "%s: D and F must be positive multiples of 64", name);
    TF_REQUIRE(ctx, params->top_k > 0 && params->hidden_stride_elements >= d, TF_ERR_INVALID_ARGUMENT, "%s: bad topK or hidden stride", name);
    const tf_expert_offsets offsets{params->gate_w_off, params->gate_s_off, params->gate_b_off, params->up_w_off, params->up_s_off,
                                    params->up_b_off, params->down_w_off, params->down_s_off, params->down_b_off};
    // blob addresses relative to the lowest one, in units of 16 bytes (the grouped kernel's expert stride)
    const uint8_t* lowest = static_cast<const uint8_t*>(blobs[0]);
    for (uint32_t i = 0; i < blob_count; ++i) {
        TF_REQUIRE(ctx, blobs[i] != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: blob %u is NULL", name, i);
        for (uint32_t j = 0; j < i; ++j)
            TF_REQUIRE(ctx, params->local_expert[i] != params->local_expert[j], TF_ERR_INVALID_ARGUMENT,
                       "duplicate expert id %u in tile binding", params->local_expert[i]);                 // :204-207
        if (static_cast<const uint8_t*>(blobs[i]) < lowest) lowest = static_cast<const uint8_t*>(blobs[i]);
    }
    if (tf_status s = tf::check_blob_alignment(ctx, lowest, 16, &offsets, name)) return s;
    tf::StreamedBinding bind{};
    bind.live = blob_count;
    for (uint32_t i = 0; i < blob_count; ++i) {
        const uint64_t delta = (uint64_t)(static_cast<const uint8_t*>(blobs[i]) - lowest);
        TF_REQUIRE(ctx, delta % 16 == 0, TF_ERR_ALIGNMENT, "%s: blobs must be 16-byte aligned", name);
        TF_REQUIRE(ctx, delta / 16 <= 0xFFFFFFFFull, TF_ERR_UNSUPPORTED, "%s: the bound blobs span more than 64 GiB", name);
        bind.expert[i] = params->local_expert[i];
        bind.blob16[i] = (uint32_t)(delta / 16);
    }
    const uint8_t* hp = tf::byte_ptr(hidden, hidden_off);
    uint8_t* acts = tf::byte_ptr(gate_up_act_scratch, gate_up_act_scratch_off);
    const tf_pair* pairs = reinterpret_cast<const tf_pair*>(tf::byte_ptr(sorted_pairs, sorted_pairs_off)) + params->pair_start;
    TF_REQUIRE(ctx, tf::aligned(hp, 16) && (params->hidden_stride_elements * 2) % 16 == 0 && tf::aligned(acts, 16) && tf::aligned(pairs, 4),
               TF_ERR_ALIGNMENT, "%s: hidden rows and the activation scratch must be 16-byte aligned", name);
    TF_REQUIRE(ctx, ctx->streamed_scratch != nullptr, TF_ERR_OUT_OF_MEMORY, "%s: context scratch missing", name);
    auto* scratch = static_cast<tf::StreamedScratch*>(ctx->streamed_scratch);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    tf::streamed_routes_kernel<<<1, 256, 0, st>>>(pairs, params->pair_count, bind, scratch, ctx->device_error);
    if (tf_status s = tf::check_launch(ctx, name)) return s;

    tf::GroupedArgs a{};
    a.pool_base = lowest; a.expert_stride = 16;
    a.w_off[0] = offsets.gate_w_off; a.s_off[0] = offsets.gate_s_off; a.b_off[0] = offsets.gate_b_off;
    a.w_off[1] = offsets.up_w_off;   a.s_off[1] = offsets.up_s_off;   a.b_off[1] = offsets.up_b_off;
    a.sorted_pairs = pairs; a.groups = scratch->groups; a.chunk_group = scratch->chunk_group;
    a.chunk_start = scratch->chunk_start; a.counters = scratch->counters;
    a.x = reinterpret_cast<const uint16_t*>(hp); a.x_stride = params->hidden_stride_elements;
    a.out = acts; a.out_stride = f; a.rows = f; a.k = d; a.top_k = params->top_k;
    if (tf_status s = tf::launch_grouped<2, false, tf::kOutActs, 2816>(ctx, stream, a, "tf_grouped_moe_streamed(gate/up)")) return s;
    tf::GroupedArgs b{};
    b.pool_base = lowest; b.expert_stride = 16;
    b.w_off[0] = offsets.down_w_off; b.s_off[0] = offsets.down_s_off; b.b_off[0] = offsets.down_b_off;
    b.sorted_pairs = pairs; b.groups = scratch->groups; b.chunk_group = scratch->chunk_group;
    b.chunk_start = scratch->chunk_start; b.counters = scratch->counters;
    b.x = reinterpret_cast<const uint16_t*>(acts); b.x_stride = f;
    b.out = tf::byte_ptr(route_partials, route_partials_off); b.out_stride = d; b.rows = d; b.k = f; b.top_k = params->top_k;
    if (tf_status s = tf::launch_grouped<1, false, tf::kOutPartialF16, 704>(ctx, stream, b, "tf_grouped_moe_streamed(down)")) return s;
    if (microbatches_out) *microbatches_out = (params->pair_count + pair_microbatch_rows - 1) / pair_microbatch_rows;
    return TF_OK;
}

tf_status tf_moe_reduce_token_major(tf_context* ctx, void* stream, const void* route_partials, int partials_f32,
                                    const void* route_weights, const void* residual, uint32_t residual_stride_elements,
                                    void* h2, uint32_t h2_stride_elements,
                                    uint32_t query_count, uint32_t top_k, uint32_t d) {
    const char* name = "tf_moe_reduce_token_major";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, route_partials && route_weights && h2, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, top_k > 0 && d > 0 && h2_stride_elements >= d, TF_ERR_INVALID_ARGUMENT, "%s: bad dimensions", name);
    if (query_count == 0) return TF_OK;
    dim3 grid(query_count, (d + 255) / 256);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (partials_f32)
        tf::launch_pdl(tf::reduce_token_major_kernel<true>, grid, dim3(256), 0, st, route_partials, static_cast<const uint16_t*>(route_weights),
                                                                  static_cast<const uint16_t*>(residual), residual_stride_elements,
                                                                  static_cast<uint16_t*>(h2), h2_stride_elements, query_count, top_k, d);
    else
        tf::launch_pdl(tf::reduce_token_major_kernel<false>, grid, dim3(256), 0, st, route_partials, static_cast<const uint16_t*>(route_weights),
                                                                   static_cast<const uint16_t*>(residual), residual_stride_elements,
                                                                   static_cast<uint16_t*>(h2), h2_stride_elements, query_count, top_k, d);
    return tf::check_launch(ctx, name);
}

tf_status tf_shared_expert_int4_block(tf_context* ctx, void* stream, const void* x, uint64_t x_off,
                                      uint32_t x_stride_elements, const tf_projection* gate, const tf_projection* up,
                                      const tf_projection* down, void* y, uint64_t y_off, uint32_t y_stride_elements,
                                      void* scratch_act, uint32_t rows) {
    const char* name = "tf_shared_expert_int4_block";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, x && gate && up && down && y && scratch_act, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, gate->rows == up->rows && gate->cols == up->cols && down->rows == gate->cols && down->cols == gate->rows,
               TF_ERR_DIMENSION_MISMATCH, "SharedExpert dimension mismatch: gate=(%u,%u) up=(%u,%u) down=(%u,%u)",
               gate->rows, gate->cols, up->rows, up->cols, down->rows, down->cols);
    const uint32_t fs = gate->rows, d = gate->cols;
    TF_REQUIRE(ctx, d % tf::kGroup == 0 && fs % tf::kGroup == 0, TF_ERR_INVALID_ARGUMENT, "%s: dimensions must be multiples of 64", name);
    TF_REQUIRE(ctx, x_stride_elements >= d && y_stride_elements >= d, TF_ERR_INVALID_ARGUMENT, "%s: stride is too small", name);
    const tf_projection* ps[3] = {gate, up, down};
    tf::MatPlanes mp[3];
    for (int i = 0; i < 3; ++i) {
        mp[i].W = tf::byte_ptr(ps[i]->weights, ps[i]->weights_off);
        mp[i].S = reinterpret_cast<const uint16_t*>(tf::byte_ptr(ps[i]->scales, ps[i]->scales_off));
        mp[i].B = reinterpret_cast<const uint16_t*>(tf::byte_ptr(ps[i]->biases, ps[i]->biases_off));
        TF_REQUIRE(ctx, tf::aligned(mp[i].W, 16) && tf::aligned(mp[i].S, 16) && tf::aligned(mp[i].B, 16), TF_ERR_ALIGNMENT,
                   "%s: projection planes must be 16-byte aligned (use tf_shared_expert_int4 for 2-byte aligned planes)", name);
    }
    const uint8_t* xp = tf::byte_ptr(x, x_off);
    TF_REQUIRE(ctx, tf::aligned(xp, 16) && (x_stride_elements * 2) % 16 == 0 && tf::aligned(scratch_act, 16), TF_ERR_ALIGNMENT,
               "%s: x rows and scratch must be 16-byte aligned", name);
    if (rows == 0) return TF_OK;
    tf::GroupedArgs a{};
    a.dense[0] = mp[0]; a.dense[1] = mp[1];
    a.x = reinterpret_cast<const uint16_t*>(xp); a.x_stride = x_stride_elements;
    a.out = scratch_act; a.out_stride = fs; a.rows = fs; a.k = d; a.dense_tokens = rows;
    tf_status s = tf::launch_grouped<2, true, tf::kOutActs, 2816>(ctx, stream, a, "tf_shared_expert_int4_block(gate/up)");
    if (s) return s;
    tf::GroupedArgs b{};
    b.dense[0] = mp[2];
    b.x = static_cast<const uint16_t*>(scratch_act); b.x_stride = fs;
    b.out = tf::byte_ptr(y, y_off); b.out_stride = y_stride_elements; b.rows = d; b.k = fs; b.dense_tokens = rows;
    return tf::launch_grouped<1, true, tf::kOutDenseF16, 2112>(ctx, stream, b, "tf_shared_expert_int4_block(down)");
}

// The shared expert for callers that must not allocate. Same kernels as tf_shared_expert_int4_block; the
// activation scratch between the gate/up kernel and the down kernel is the array built into the library.
tf_status tf_shared_expert_int4_block_noalloc(void* stream, const void* x, uint64_t x_off, uint32_t x_stride_elements,
                                              const tf_projection* gate, const tf_projection* up, const tf_projection* down,
                                              void* y, uint64_t y_off, uint32_t y_stride_elements, uint32_t rows,
                                              uint32_t* device_status) {
    const char* name = "tf_shared_expert_int4_block_noalloc";
    if (!gate || !up || !down) return tf::fail(nullptr, TF_ERR_INVALID_ARGUMENT, "%s: NULL projection", name);
    const uint64_t need = (uint64_t)rows * gate->rows * 2;
    if (need > tf::kNoAllocScratchBytes)
        return tf::fail(nullptr, TF_ERR_SCRATCH_TOO_SMALL,
                        "%s: %u rows x %u activations need %llu bytes of scratch; the built-in scratch holds %zu bytes "
                        "(use tf_shared_expert_int4_block with your own scratch for larger blocks)",
                        name, rows, gate->rows, (unsigned long long)need, tf::kNoAllocScratchBytes);
    tf::NoAllocDevice* dev = nullptr;
    if (tf_status s = tf::noalloc_device(&dev, name)) return s;      // first call on a device: the one-time set-up
    // A context on the stack: nothing in it is allocated on the device. tf_shared_expert_int4_block and the launch
    // code under it use only device, sm_count, device_error, launches and last_error; the side stream, the router
    // and tensor-core scratch stay NULL and must not be touched on this path.
    tf_context local;
    cudaGetDevice(&local.device);
    local.sm_count = dev->sm_count;
    local.device_error = device_status ? device_status : dev->error_word;
    // The scratch keeps what the previous call left. The activations need no clearing (the first kernel writes
    // every element the second reads); the status word must start at zero.
    cudaError_t e = cudaMemsetAsync(local.device_error, 0, sizeof(uint32_t), static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return tf::fail(nullptr, TF_ERR_CUDA, "%s: clearing the status word: %s", name, cudaGetErrorString(e));
    return tf_shared_expert_int4_block(&local, stream, x, x_off, x_stride_elements, gate, up, down, y, y_off, y_stride_elements,
                                       dev->scratch, rows);
}

}  // extern "C"
