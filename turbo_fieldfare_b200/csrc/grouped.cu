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
// Kernel design (memory-bound; HBM roofline): weights are the B operand of
// mma.sync.m16n8k16 (8 weight rows per warp tile), up to 16 tokens are the A
// operand. A 4-bit code q placed in the low mantissa bits of an fp16 IS
// the subnormal q * 2^-24, so "dequantisation" is one AND per two codes and the
// tensor core multiplies exact integers by fp16 activations with fp32
// accumulation. Scale and bias are applied per 64-column group after the MMAs:
//     y += (s * 2^24) * acc + b * sum_k x_k
// i.e. the reference's group factoring (Metal/Quant/dequant_int4.metal:14-19).
// The activations of a chunk (<= 16 tokens of one expert) are staged once per
// CTA in shared memory, already permuted into MMA fragment order; every warp
// then streams whole 8-row tiles on its own: packed codes and scale rows come
// straight from global memory into registers, prefetched one step (4 groups)
// ahead, with no block-wide barrier in the steady state. For very small
// batches a tile is split along K over `ks` warps that meet at a named barrier
// and are summed in warp order, so results stay deterministic.
#include "tf_common.cuh"

namespace tf {

// ---------------------------------------------------------------------------
// route grouping on the device
// ---------------------------------------------------------------------------

constexpr int kGroupThreads = 256;
constexpr int kGroupPerThread = 4;
constexpr int kChunkTokens = 16;      // tokens per work chunk of the grouped kernels (the m of m16n8k16)

// counters: [0] group count, [1] total chunks (sum over groups of ceil(count/16)), [2] pair count
__global__ void __launch_bounds__(kGroupThreads)
group_routes_kernel(const uint32_t* __restrict__ indices, const uint16_t* __restrict__ weights,
                    uint32_t T, uint32_t K, uint32_t E,
                    tf_pair* __restrict__ sorted_pairs, uint32_t* __restrict__ per_expert_offsets,
                    uint32_t* __restrict__ per_expert_counts, tf_group* __restrict__ groups,
                    uint32_t* __restrict__ chunk_group, uint32_t* __restrict__ chunk_start,
                    uint32_t* __restrict__ counters) {
    __shared__ uint32_t hist[TF_MAX_ROUTER_EXPERTS];
    __shared__ uint32_t warp_tot[kGroupThreads / kWarp];
    __shared__ uint32_t s_offset, s_gi, s_chunk0;
    const uint32_t e = blockIdx.x;
    const uint32_t n = T * K;
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        uint32_t ex = indices[i];
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
        s_offset = off; s_gi = gi; s_chunk0 = ch;
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
                uint32_t ex = indices[i];
                if (ex >= E) ex = E - 1;
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

// ---------------------------------------------------------------------------
// grouped small-batch expert kernels
// ---------------------------------------------------------------------------

constexpr int kStep = 4;               // 64-column groups per prefetch step
constexpr int kTileRows = 8;           // weight rows per MMA tile (the n of m16n8k16)
constexpr float kTwo24 = 16777216.0f;
constexpr int kStreamWarps = 16;       // warps per CTA
constexpr int kStreamThreads = kStreamWarps * kWarp;
constexpr int kMaxKSplit = 8;

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
    uint32_t ks;               // warps that share one tile along K (1, 2, 4 or 8)
};

// D = A * B + C with C either the constant zero (first MMA of a group) or D itself. The four A
// registers and the four accumulators are always real fragments (tokens g and g + 8), so the
// operands need no marshalling moves.
__device__ __forceinline__ void mma16816_first(float (&c)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void mma16816_acc(float (&c)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
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
__device__ __forceinline__ uint2 ldg_nc_u2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds_f32x2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void named_barrier(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

enum OutMode { kOutActs = 0, kOutPartialF16 = 1, kOutPartialF32 = 2, kOutDenseF16 = 3 };

// Shared memory:
//   xq[ng][4][32] uint4    A fragments: entry (G, j, lane) = {a0, a1, a2, a3} of MMA j of group G for lane (g, t):
//                          tokens g (a0, a2) and g + 8 (a1, a3), this lane's columns 64 G + 16 t + {..}
//   xsum[ng][8] float2     fp32 sums of the 64 activations of group G for tokens g and g + 8
//   red[2][warps][NMAT][128] float   K-split partials, double buffered
__host__ __device__ inline size_t stream_smem_bytes(uint32_t ng, int nmat) {
    return (size_t)ng * 4 * 32 * 16 + (size_t)ng * 8 * 8 + (size_t)2 * kStreamWarps * nmat * 128 * 4;
}

// What one step (up to kStep groups of one 8-row tile) needs from global memory.
template <int NMAT>
struct StepRegs {
    uint2 w[NMAT][kStep];          // this lane's 16 codes of each group (row g, bytes [8t, 8t+8) of the group)
    uint2 s0[NMAT], s1[NMAT];      // 4 consecutive bf16 scales of rows 2t and 2t+1
    uint2 b0[NMAT], b1[NMAT];      // and biases
};

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
// bf16 scale times 2^24 (the codes enter the MMA as q * 2^-24): add 24 to the exponent field.
// A zero scale becomes 2^-103, whose product with the accumulator is far below fp32 resolution.
__device__ __forceinline__ float bf16_lo_x2p24(uint32_t v) { return __uint_as_float((v << 16) + 0x0C000000u); }
__device__ __forceinline__ float bf16_hi_x2p24(uint32_t v) { return __uint_as_float((v & 0xFFFF0000u) + 0x0C000000u); }

template <int NMAT, bool DENSE, int OUT_MODE>
__global__ void __launch_bounds__(kStreamThreads)
grouped_stream_kernel(const GroupedArgs args) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t ng = args.k / kGroup;
    const uint32_t ks = args.ks;
    const uint32_t row_bytes = args.k / 2;
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t xq_addr = smem_base + lane * 16;                    // + G * 2048 + j * 512
    const uint32_t xsum_addr = smem_base + ng * 2048 + g * 8;          // + G * 64
    uint4* xq = reinterpret_cast<uint4*>(smem);
    float2* xsum = reinterpret_cast<float2*>(smem + (size_t)ng * 2048);
    float* red = reinterpret_cast<float*>(smem + (size_t)ng * 2048 + (size_t)ng * 64);

    const uint32_t tiles = args.rows / kTileRows;
    const uint32_t total_chunks = DENSE ? (args.dense_tokens + kChunkTokens - 1) / kChunkTokens : args.counters[1];
    const uint32_t total_items = total_chunks * tiles;
    // contiguous item range per CTA: consecutive items share the chunk whose activations sit in shared memory
    uint32_t item = (uint32_t)((uint64_t)total_items * blockIdx.x / gridDim.x);
    const uint32_t item_end = (uint32_t)((uint64_t)total_items * (blockIdx.x + 1) / gridDim.x);

    // K split: warp group `grp` of ks warps shares a tile; warp `kw` of the group owns groups [k_begin, k_end)
    const uint32_t ngroups = kStreamWarps / ks;
    const uint32_t grp = warp / ks, kw = warp % ks;
    const uint32_t steps_total = (ng + kStep - 1) / kStep;
    const uint32_t steps_per_warp = (steps_total + ks - 1) / ks;
    const uint32_t k_begin = kw * steps_per_warp * kStep < ng ? kw * steps_per_warp * kStep : ng;
    const uint32_t k_end = (kw + 1) * steps_per_warp * kStep < ng ? (kw + 1) * steps_per_warp * kStep : ng;
    const uint32_t nsteps = k_end > k_begin ? (k_end - k_begin + kStep - 1) / kStep : 0;
    const bool sb_vec = (ng % 4) == 0;        // 4 consecutive bf16 of a scale row are 8-byte aligned
    const uint32_t out_stride = args.out_stride, top_k = args.top_k;

    while (item < item_end) {
        // ---- segment: the items of this CTA that belong to one chunk ----
        const uint32_t chunk = item / tiles;
        const uint32_t tile_begin = item % tiles;
        const uint32_t seg_items = (item_end - item) < (tiles - tile_begin) ? (item_end - item) : (tiles - tile_begin);
        MatPlanes pl[NMAT];
        uint32_t ntok, row_base;
        if constexpr (DENSE) {
#pragma unroll
            for (int m = 0; m < NMAT; ++m) pl[m] = args.dense[m];
            row_base = chunk * kChunkTokens;
            const uint32_t left = args.dense_tokens - row_base;
            ntok = left < (uint32_t)kChunkTokens ? left : (uint32_t)kChunkTokens;
        } else {
            const uint32_t gi = args.chunk_group[chunk];
            const tf_group grpinfo = args.groups[gi];
            const uint32_t cin = chunk - args.chunk_start[gi];
            const uint8_t* blob = args.pool_base + (uint64_t)grpinfo.expert * args.expert_stride;
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                pl[m].W = blob + args.w_off[m];
                pl[m].S = reinterpret_cast<const uint16_t*>(blob + args.s_off[m]);
                pl[m].B = reinterpret_cast<const uint16_t*>(blob + args.b_off[m]);
            }
            row_base = grpinfo.pair_start + cin * kChunkTokens;
            const uint32_t left = grpinfo.pair_count - cin * kChunkTokens;
            ntok = left < (uint32_t)kChunkTokens ? left : (uint32_t)kChunkTokens;
        }

        __syncthreads();        // every warp is done with the previous chunk's fragments
        // Stage the chunk's activations as MMA A fragments. Work item (G, half, lane): token g + 8 * half,
        // columns 64 G + 16 t .. + 15. The 16 values x0..x15 feed four MMAs:
        //   j = 0: (x0,x4),(x2,x6)   j = 1: (x1,x5)/16,(x3,x7)/16   j = 2, 3: the same for x8..x15.
        // Odd columns are pre-scaled by 1/16 because their codes sit four mantissa bits higher.
        for (uint32_t idx = threadIdx.x; idx < ng * 64; idx += blockDim.x) {
            const uint32_t G = idx >> 6, half = (idx >> 5) & 1, ln = idx & 31, tok = (ln >> 2) + 8 * half, tt = ln & 3;
            uint32_t r[8];
            if (tok < ntok) {
                const uint32_t rr = (DENSE || NMAT == 1) ? row_base + tok : args.sorted_pairs[row_base + tok].token;
                const uint4* p = reinterpret_cast<const uint4*>(args.x + (size_t)rr * args.x_stride + G * kGroup + tt * 16);
                const uint4 lo = __ldg(p), hi = __ldg(p + 1);
                r[0] = lo.x; r[1] = lo.y; r[2] = lo.z; r[3] = lo.w;
                r[4] = hi.x; r[5] = hi.y; r[6] = hi.z; r[7] = hi.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) r[i] = 0;
            }
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&r[i]));
                sum += v.x + v.y;
            }
            sum += __shfl_xor_sync(kFullMask, sum, 1);
            sum += __shfl_xor_sync(kFullMask, sum, 2);
            uint32_t* q = reinterpret_cast<uint32_t*>(xq + (size_t)G * 128 + ln) + half;     // a0/a1 slot; a2/a3 at +2
            q[0 * 128 + 0] = prmt(r[0], r[2], 0x5410);                      q[0 * 128 + 2] = prmt(r[1], r[3], 0x5410);
            q[1 * 128 + 0] = hmul2_sixteenth(prmt(r[0], r[2], 0x7632));     q[1 * 128 + 2] = hmul2_sixteenth(prmt(r[1], r[3], 0x7632));
            q[2 * 128 + 0] = prmt(r[4], r[6], 0x5410);                      q[2 * 128 + 2] = prmt(r[5], r[7], 0x5410);
            q[3 * 128 + 0] = hmul2_sixteenth(prmt(r[4], r[6], 0x7632));     q[3 * 128 + 2] = hmul2_sixteenth(prmt(r[5], r[7], 0x7632));
            if (tt == 0) reinterpret_cast<float*>(xsum + G * 8 + (ln >> 2))[half] = sum;
        }
        __syncthreads();

        // ---- this warp group's tiles of the segment: tile_begin + grp, + ngroups, ... ----
        const uint32_t my_tiles = grp < seg_items ? (seg_items - grp + ngroups - 1) / ngroups : 0;
        const uint32_t total_steps = my_tiles * nsteps;

        // lane pointers at (first tile, k_begin); a step advances them by kStep groups, a tile change rewinds K
        const uint8_t* wp[NMAT];
        const uint16_t* sp[NMAT];
        const uint16_t* bp[NMAT];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
            const uint32_t tile0 = tile_begin + grp;
            wp[m] = pl[m].W + (size_t)(tile0 * kTileRows + g) * row_bytes + k_begin * 32 + t * 8;
            sp[m] = pl[m].S + (size_t)(tile0 * kTileRows + 2 * t) * ng + k_begin;
            bp[m] = pl[m].B + (size_t)(tile0 * kTileRows + 2 * t) * ng + k_begin;
        }
        const uint32_t w_tile_jump = ngroups * kTileRows * row_bytes - (nsteps - 1) * kStep * 32;   // last step -> next tile's first
        const uint32_t sb_tile_jump = ngroups * kTileRows * ng - (nsteps - 1) * kStep;
        uint32_t load_st = 0;       // step index (within the tile) of the next load

        // L2 prefetch of one whole tile (this warp's K range of the 8 rows, and the scale rows): issued
        // one tile ahead so that DRAM latency is paid long before the register loads need the data.
        const uint32_t pf_line0 = (k_begin * 32) / 128, pf_line1 = (k_end * 32 + 127) / 128;
        const uint32_t pf_lines = (pf_line1 - pf_line0) * kTileRows;
        const uint32_t sb_lines = (kTileRows * ng * 2 + 127) / 128;
        uint32_t load_tile = tile_begin + grp;
        auto prefetch_tile = [&](uint32_t tile) {
            if (tile >= tile_begin + seg_items) return;
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                const uint8_t* wt = pl[m].W + (size_t)tile * kTileRows * row_bytes;
                for (uint32_t l = lane; l < pf_lines; l += kWarp) {
                    const uint32_t r = l / (pf_line1 - pf_line0), c = pf_line0 + l % (pf_line1 - pf_line0);
                    prefetch_l2(wt + (size_t)r * row_bytes + c * 128);
                }
                if (kw == 0 && lane < sb_lines) {
                    prefetch_l2(reinterpret_cast<const uint8_t*>(pl[m].S + (size_t)tile * kTileRows * ng) + lane * 128);
                    prefetch_l2(reinterpret_cast<const uint8_t*>(pl[m].B + (size_t)tile * kTileRows * ng) + lane * 128);
                }
            }
        };
        if (my_tiles > 0 && nsteps > 0) prefetch_tile(load_tile);

        auto load_step = [&](StepRegs<NMAT>& sr) {
            const uint32_t g_first = k_begin + load_st * kStep;
            if (load_st == 0) {
                prefetch_tile(load_tile + ngroups);
                load_tile += ngroups;
            }
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
#pragma unroll
                for (int i = 0; i < kStep; ++i)
                    sr.w[m][i] = (g_first + i < k_end) ? ldg_nc_u2(wp[m] + i * 32) : make_uint2(0u, 0u);
                if (sb_vec) {
                    sr.s0[m] = __ldg(reinterpret_cast<const uint2*>(sp[m]));
                    sr.s1[m] = __ldg(reinterpret_cast<const uint2*>(sp[m] + ng));
                    sr.b0[m] = __ldg(reinterpret_cast<const uint2*>(bp[m]));
                    sr.b1[m] = __ldg(reinterpret_cast<const uint2*>(bp[m] + ng));
                } else {
                    uint32_t v[4][4];
#pragma unroll
                    for (int i = 0; i < kStep; ++i) {
                        const bool ok = g_first + i < k_end;
                        v[0][i] = ok ? sp[m][i] : 0u; v[1][i] = ok ? sp[m][ng + i] : 0u;
                        v[2][i] = ok ? bp[m][i] : 0u; v[3][i] = ok ? bp[m][ng + i] : 0u;
                    }
                    sr.s0[m] = make_uint2(v[0][0] | (v[0][1] << 16), v[0][2] | (v[0][3] << 16));
                    sr.s1[m] = make_uint2(v[1][0] | (v[1][1] << 16), v[1][2] | (v[1][3] << 16));
                    sr.b0[m] = make_uint2(v[2][0] | (v[2][1] << 16), v[2][2] | (v[2][3] << 16));
                    sr.b1[m] = make_uint2(v[3][0] | (v[3][1] << 16), v[3][2] | (v[3][3] << 16));
                }
            }
            if (++load_st == nsteps) {
                load_st = 0;
#pragma unroll
                for (int m = 0; m < NMAT; ++m) { wp[m] += w_tile_jump; sp[m] += sb_tile_jump; bp[m] += sb_tile_jump; }
            } else {
#pragma unroll
                for (int m = 0; m < NMAT; ++m) { wp[m] += kStep * 32; sp[m] += kStep; bp[m] += kStep; }
            }
        };

        float ya[NMAT][4];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
#pragma unroll
            for (int j = 0; j < 4; ++j) ya[m][j] = 0.0f;
        }
        uint32_t comp_st = 0, comp_tile = tile_begin + grp, comp_ti = 0;

        auto compute_step = [&](const StepRegs<NMAT>& sr) {
            const uint32_t g_first = k_begin + comp_st * kStep;
#pragma unroll
            for (int i = 0; i < kStep; ++i) {
                if (g_first + i < k_end) {          // warp-uniform
                    const uint32_t G = g_first + i;
                    const uint4 a0 = lds128(xq_addr + G * 2048), a1 = lds128(xq_addr + G * 2048 + 512);
                    const uint4 a2 = lds128(xq_addr + G * 2048 + 1024), a3 = lds128(xq_addr + G * 2048 + 1536);
                    const float2 xs = lds_f32x2(xsum_addr + G * 64);
#pragma unroll
                    for (int m = 0; m < NMAT; ++m) {
                        const uint32_t w0 = sr.w[m][i].x, w1 = sr.w[m][i].y, w0s = w0 >> 8, w1s = w1 >> 8;
                        float c[4];
                        mma16816_first(c, a0, w0 & 0x000F000Fu, w0s & 0x000F000Fu);
                        mma16816_acc(c, a1, w0 & 0x00F000F0u, w0s & 0x00F000F0u);
                        mma16816_acc(c, a2, w1 & 0x000F000Fu, w1s & 0x000F000Fu);
                        mma16816_acc(c, a3, w1 & 0x00F000F0u, w1s & 0x00F000F0u);
                        const uint32_t sv0 = i < 2 ? sr.s0[m].x : sr.s0[m].y, sv1 = i < 2 ? sr.s1[m].x : sr.s1[m].y;
                        const uint32_t bv0 = i < 2 ? sr.b0[m].x : sr.b0[m].y, bv1 = i < 2 ? sr.b1[m].x : sr.b1[m].y;
                        const float s0 = (i & 1) ? bf16_hi_x2p24(sv0) : bf16_lo_x2p24(sv0);
                        const float s1 = (i & 1) ? bf16_hi_x2p24(sv1) : bf16_lo_x2p24(sv1);
                        const float b0 = (i & 1) ? bf16_hi(bv0) : bf16_lo(bv0), b1 = (i & 1) ? bf16_hi(bv1) : bf16_lo(bv1);
                        // c0, c1: token g, rows 2t, 2t+1; c2, c3: token g + 8
                        ya[m][0] = fmaf(s0, c[0], fmaf(b0, xs.x, ya[m][0]));
                        ya[m][1] = fmaf(s1, c[1], fmaf(b1, xs.x, ya[m][1]));
                        ya[m][2] = fmaf(s0, c[2], fmaf(b0, xs.y, ya[m][2]));
                        ya[m][3] = fmaf(s1, c[3], fmaf(b1, xs.y, ya[m][3]));
                    }
                }
            }
            if (++comp_st < nsteps) return;
            // ---- last step of the tile: combine, reduce over the K split, store ----
            comp_st = 0;
            float y[NMAT][4];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    y[m][j] = ya[m][j];
                    ya[m][j] = 0.0f;
                }
            }
            if (ks > 1) {
                // partial sums of the group's warps, added in warp order by the group's first warp
                float* rb = red + (size_t)(comp_ti & 1) * (kStreamWarps * NMAT * 128);
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                    float* r = rb + ((size_t)warp * NMAT + m) * 128;
                    *reinterpret_cast<float2*>(r + g * 8 + 2 * t) = make_float2(y[m][0], y[m][1]);
                    *reinterpret_cast<float2*>(r + (g + 8) * 8 + 2 * t) = make_float2(y[m][2], y[m][3]);
                }
                named_barrier(1 + grp, ks * kWarp);
                if (kw == 0) {
#pragma unroll
                    for (int m = 0; m < NMAT; ++m) {
                        float2 lo = make_float2(0.0f, 0.0f), hi = make_float2(0.0f, 0.0f);
                        for (uint32_t w2 = 0; w2 < ks; ++w2) {
                            const float* r = rb + ((size_t)(warp + w2) * NMAT + m) * 128;
                            const float2 v0 = *reinterpret_cast<const float2*>(r + g * 8 + 2 * t);
                            const float2 v1 = *reinterpret_cast<const float2*>(r + (g + 8) * 8 + 2 * t);
                            lo.x += v0.x; lo.y += v0.y; hi.x += v1.x; hi.y += v1.y;
                        }
                        y[m][0] = lo.x; y[m][1] = lo.y; y[m][2] = hi.x; y[m][3] = hi.y;
                    }
                }
                // `red` is double buffered by tile parity: a buffer is rewritten two tiles later, after another
                // pass through this barrier, which the reading warp reaches only once it has finished reading.
            }
            if (kw == 0) {
                const uint32_t out_row = comp_tile * kTileRows + 2 * t;
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const uint32_t tok = g + 8 * hh;
                    if (tok < ntok) {
                        const float v0 = y[0][2 * hh], v1 = y[0][2 * hh + 1];
                        if constexpr (OUT_MODE == kOutActs) {
                            float g0v = v0, g1v = v1, u0 = y[NMAT - 1][2 * hh], u1 = y[NMAT - 1][2 * hh + 1];
                            if constexpr (DENSE) {
                                // shared expert: gate and up are stored as fp16 before the activation
                                // (Kernels/MoE/SharedExpertInt4.swift:62-93; Metal/Primitives/utility.metal:15-17)
                                g0v = __half2float(__float2half_rn(g0v)); g1v = __half2float(__float2half_rn(g1v));
                                u0 = __half2float(__float2half_rn(u0)); u1 = __half2float(__float2half_rn(u1));
                            }
                            // routed: act = half(gelu_tanh(gate) * up), gate and up in fp32 (prefill.metal:634-636; moe.metal:368)
                            *reinterpret_cast<__half2*>(static_cast<uint16_t*>(args.out) + (size_t)(row_base + tok) * out_stride + out_row) =
                                __floats2half2_rn(gelu_tanh(g0v) * u0, gelu_tanh(g1v) * u1);
                        } else if constexpr (OUT_MODE == kOutDenseF16) {
                            *reinterpret_cast<__half2*>(static_cast<uint16_t*>(args.out) + (size_t)(row_base + tok) * out_stride + out_row) =
                                __floats2half2_rn(v0, v1);
                        } else {
                            const tf_pair pr = args.sorted_pairs[row_base + tok];
                            const size_t idx = ((size_t)pr.token * top_k + pr.rank) * out_stride + out_row;
                            if constexpr (OUT_MODE == kOutPartialF16)      // prefill.metal:666-669
                                *reinterpret_cast<__half2*>(static_cast<uint16_t*>(args.out) + idx) = __floats2half2_rn(v0, v1);
                            else
                                *reinterpret_cast<float2*>(static_cast<float*>(args.out) + idx) = make_float2(v0, v1);
                        }
                    }
                }
            }
            comp_tile += ngroups;
            ++comp_ti;
        };

        if (ks > 1 && nsteps == 0) {
            // a warp of a K-split group whose K range is empty still has to meet its group at every tile
            for (uint32_t ti = 0; ti < my_tiles; ++ti) {
                float* rb = red + (size_t)(ti & 1) * (kStreamWarps * NMAT * 128);
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                    float* r = rb + ((size_t)warp * NMAT + m) * 128;
                    *reinterpret_cast<float2*>(r + g * 8 + 2 * t) = make_float2(0.0f, 0.0f);
                    *reinterpret_cast<float2*>(r + (g + 8) * 8 + 2 * t) = make_float2(0.0f, 0.0f);
                }
                named_barrier(1 + grp, ks * kWarp);
            }
        } else if (total_steps > 0) {
            // ping-pong register prefetch: while one step's registers are consumed the next step's loads are in flight
            StepRegs<NMAT> ra, rb2;
            load_step(ra);
            uint32_t gs = 0;
            for (; gs + 2 <= total_steps; gs += 2) {
                load_step(rb2);
                compute_step(ra);
                if (gs + 2 < total_steps) load_step(ra);
                compute_step(rb2);
            }
            if (gs < total_steps) compute_step(ra);
        }
        item += seg_items;
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
    const uint32_t d = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t t = blockIdx.y;
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

// Picks the K split: enough warp-tiles to occupy every warp of every CTA a few times over.
static uint32_t choose_ksplit(uint64_t expected_items, uint32_t sm_count, uint32_t ng) {
    uint32_t ks = 1;
    const uint32_t steps = (ng + kStep - 1) / kStep;
    while (ks < (uint32_t)kMaxKSplit && ks * 2 <= steps && expected_items * ks < (uint64_t)sm_count * kStreamWarps * 3) ks *= 2;
    return ks;
}

template <int NMAT, bool DENSE, int OUT_MODE>
static tf_status launch_grouped(tf_context* ctx, void* stream, GroupedArgs& args, uint64_t expected_chunks, const char* name) {
    const uint32_t ng = args.k / kGroup;
    TF_REQUIRE(ctx, ng >= 1 && args.k % kGroup == 0, TF_ERR_INVALID_ARGUMENT, "%s: K must be a positive multiple of 64", name);
    TF_REQUIRE(ctx, args.rows % kTileRows == 0, TF_ERR_UNSUPPORTED, "%s: row count %u must be a multiple of 8", name, args.rows);
    const size_t smem = stream_smem_bytes(ng, NMAT);
    TF_REQUIRE(ctx, smem <= 200 * 1024, TF_ERR_UNSUPPORTED, "%s: K=%u needs %zu bytes of shared memory (limit 200 KB)", name, args.k, smem);
    auto kern = grouped_stream_kernel<NMAT, DENSE, OUT_MODE>;
    // The attribute is set once per instantiation, so steady-state calls are a bare launch
    // (and safe inside stream capture).
    static bool configured = false;
    if (!configured) {
        TF_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = true;
    }
    const uint64_t items = expected_chunks * (args.rows / kTileRows);
    args.ks = choose_ksplit(items, (uint32_t)ctx->sm_count, ng);
    uint32_t grid = (uint32_t)ctx->sm_count;
    if (DENSE) {
        if (items == 0) return TF_OK;
        const uint64_t want = (items * args.ks + kStreamWarps - 1) / kStreamWarps;
        if (want < grid) grid = (uint32_t)want;
    }
    kern<<<grid, kStreamThreads, smem, static_cast<cudaStream_t>(stream)>>>(args);
    return check_launch(ctx, name);
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

}  // namespace tf

extern "C" {

tf_status tf_group_routes_device(tf_context* ctx, void* stream, const uint32_t* indices, const void* weights_f16,
                                 uint32_t query_count, uint32_t top_k, uint32_t num_experts,
                                 const tf_device_routes* routes) {
    const char* name = "tf_group_routes_device";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, indices && weights_f16 && routes, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, routes->sorted_pairs && routes->per_expert_offsets && routes->per_expert_counts && routes->groups &&
                        routes->chunk_group && routes->chunk_start && routes->counters,
               TF_ERR_INVALID_ARGUMENT, "%s: NULL route buffer", name);
    TF_REQUIRE(ctx, top_k > 0, TF_ERR_GROUPING_INVALID_TOP_K, "topK must be positive, got %u", top_k);
    TF_REQUIRE(ctx, num_experts > 0 && num_experts <= TF_MAX_ROUTER_EXPERTS, TF_ERR_GROUPING_INVALID_NUM_EXPERTS,
               "numExperts must be in 1...256, got %u", num_experts);
    TF_REQUIRE(ctx, (uint64_t)query_count * top_k < (1ull << 31), TF_ERR_INVALID_ARGUMENT, "%s: too many pairs", name);
    tf::group_routes_kernel<<<num_experts, tf::kGroupThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        indices, static_cast<const uint16_t*>(weights_f16), query_count, top_k, num_experts, routes->sorted_pairs,
        routes->per_expert_offsets, routes->per_expert_counts, routes->groups, routes->chunk_group, routes->chunk_start,
        routes->counters);
    return tf::check_launch(ctx, name);
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
    // The chunk count lives on the device; the K split only needs its order of magnitude:
    // every pair its own expert (at most num pairs, bounded by the pool) or 8 pairs per chunk.
    const uint64_t pairs = (uint64_t)query_count * top_k;
    const uint64_t expected_chunks = pairs < 1024 ? pairs : pairs / tf::kChunkTokens;

    tf::GroupedArgs a{};
    a.pool_base = static_cast<const uint8_t*>(pool_layer_base);
    a.expert_stride = expert_stride;
    a.w_off[0] = offsets->gate_w_off; a.s_off[0] = offsets->gate_s_off; a.b_off[0] = offsets->gate_b_off;
    a.w_off[1] = offsets->up_w_off;   a.s_off[1] = offsets->up_s_off;   a.b_off[1] = offsets->up_b_off;
    a.sorted_pairs = routes->sorted_pairs; a.groups = routes->groups; a.chunk_group = routes->chunk_group;
    a.chunk_start = routes->chunk_start; a.counters = routes->counters;
    a.x = reinterpret_cast<const uint16_t*>(hp); a.x_stride = hidden_stride_elements;
    a.out = acts_scratch; a.out_stride = f; a.rows = f; a.k = d; a.top_k = top_k;
    tf_status s = tf::launch_grouped<2, false, tf::kOutActs>(ctx, stream, a, expected_chunks, "tf_grouped_moe_batched(gate/up)");
    if (s) return s;

    tf::GroupedArgs b{};
    b.pool_base = a.pool_base; b.expert_stride = expert_stride;
    b.w_off[0] = offsets->down_w_off; b.s_off[0] = offsets->down_s_off; b.b_off[0] = offsets->down_b_off;
    b.sorted_pairs = routes->sorted_pairs; b.groups = routes->groups; b.chunk_group = routes->chunk_group;
    b.chunk_start = routes->chunk_start; b.counters = routes->counters;
    b.x = static_cast<const uint16_t*>(acts_scratch); b.x_stride = f;
    b.out = route_partials; b.out_stride = d; b.rows = d; b.k = f; b.top_k = top_k;
    if (partials_f32) return tf::launch_grouped<1, false, tf::kOutPartialF32>(ctx, stream, b, expected_chunks, "tf_grouped_moe_batched(down)");
    return tf::launch_grouped<1, false, tf::kOutPartialF16>(ctx, stream, b, expected_chunks, "tf_grouped_moe_batched(down)");
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
    dim3 grid((d + 255) / 256, query_count);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (partials_f32)
        tf::reduce_token_major_kernel<true><<<grid, 256, 0, st>>>(route_partials, static_cast<const uint16_t*>(route_weights),
                                                                  static_cast<const uint16_t*>(residual), residual_stride_elements,
                                                                  static_cast<uint16_t*>(h2), h2_stride_elements, query_count, top_k, d);
    else
        tf::reduce_token_major_kernel<false><<<grid, 256, 0, st>>>(route_partials, static_cast<const uint16_t*>(route_weights),
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
    tf_status s = tf::launch_grouped<2, true, tf::kOutActs>(ctx, stream, a, (rows + tf::kChunkTokens - 1) / tf::kChunkTokens, "tf_shared_expert_int4_block(gate/up)");
    if (s) return s;
    tf::GroupedArgs b{};
    b.dense[0] = mp[2];
    b.x = static_cast<const uint16_t*>(scratch_act); b.x_stride = fs;
    b.out = tf::byte_ptr(y, y_off); b.out_stride = y_stride_elements; b.rows = d; b.k = fs; b.dense_tokens = rows;
    return tf::launch_grouped<1, true, tf::kOutDenseF16>(ctx, stream, b, (rows + tf::kChunkTokens - 1) / tf::kChunkTokens, "tf_shared_expert_int4_block(down)");
}

}  // extern "C"
