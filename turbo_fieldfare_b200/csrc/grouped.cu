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
// operand. A 4-bit code q placed in the low mantissa bits of an fp16 IS the
// subnormal q * 2^-24, so "dequantisation" is one AND per two codes and the
// tensor core multiplies exact integers by fp16 activations with fp32
// accumulation. Scale and bias are applied per 64-column group after the MMAs:
//     y += (s * 2^24) * acc + b * sum_k x_k
// i.e. the reference's group factoring (Metal/Quant/dequant_int4.metal:14-19).
// K is split across the warps of a CTA (4 groups each); activations live in
// registers as MMA fragments; packed weights and the scale planes stream
// through a cp.async ring (16-byte copies, 4 stages); warp partials are summed
// in warp order through shared memory, so results are deterministic.
#include "tf_common.cuh"

namespace tf {

// ---------------------------------------------------------------------------
// route grouping on the device
// ---------------------------------------------------------------------------

constexpr int kGroupThreads = 256;
constexpr int kGroupPerThread = 4;
constexpr int kChunkTokens = 16;      // tokens per work chunk of the grouped kernels

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

constexpr int kGPW = 4;            // 64-column groups per warp
constexpr int kStages = 4;         // cp.async ring depth
constexpr int kTileRows = 8;       // weight rows per MMA tile (the n of m16n8k16)
constexpr float kTwo24 = 16777216.0f;
constexpr int kMaxGroupedWarps = 12;   // K <= 12 * 4 * 64 = 3072 columns
constexpr int kMaxGroupedThreads = kMaxGroupedWarps * kWarp;

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
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, bool valid) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Activation fragments of one token for one 64-column group, as held by lane
// (g, t): 16 consecutive values starting at 16 * pi(t), pi = (0, 2, 1, 3),
// rearranged to the operand order of the four MMAs; odd columns pre-scaled by
// 1/16 because their codes sit four mantissa bits higher.
struct XFrag {
    uint32_t a[8];
    float sum;       // full 64-column sum of the token's activations (quad-reduced)
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

__device__ __forceinline__ uint32_t hmul2_sixteenth(uint32_t v) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&v), __half2half2(__float2half_rn(0.0625f)));
    return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ void load_xfrag(XFrag& f, const uint16_t* __restrict__ row /* null = zero token */,
                                           uint32_t group, int t) {
    uint32_t r[8];
    if (row) {
        const int piece = ((t & 1) << 1) | (t >> 1);
        const uint4* p = reinterpret_cast<const uint4*>(row + group * kGroup + piece * 16);
        const uint4 lo = __ldg(p), hi = __ldg(p + 1);
        r[0] = lo.x; r[1] = lo.y; r[2] = lo.z; r[3] = lo.w;
        r[4] = hi.x; r[5] = hi.y; r[6] = hi.z; r[7] = hi.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] = 0;
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&r[i]));
        s += v.x + v.y;
    }
    s += __shfl_xor_sync(kFullMask, s, 1);
    s += __shfl_xor_sync(kFullMask, s, 2);
    f.sum = s;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        f.a[4 * h + 0] = prmt(r[4 * h + 0], r[4 * h + 2], 0x5410);                    // (x0, x4)
        f.a[4 * h + 1] = prmt(r[4 * h + 1], r[4 * h + 3], 0x5410);                    // (x2, x6)
        f.a[4 * h + 2] = hmul2_sixteenth(prmt(r[4 * h + 0], r[4 * h + 2], 0x7632));   // (x1, x5) / 16
        f.a[4 * h + 3] = hmul2_sixteenth(prmt(r[4 * h + 1], r[4 * h + 3], 0x7632));   // (x3, x7) / 16
    }
}

// Four MMAs of one 64-column group: piece = this lane's 16 codes (two words).
template <bool HI>
__device__ __forceinline__ void group_mma(float (&c)[4], uint32_t w0, uint32_t w1, const XFrag& lo, const XFrag& hi) {
    const uint32_t w0s = w0 >> 8, w1s = w1 >> 8;
    mma16816(c, lo.a[0], HI ? hi.a[0] : 0u, lo.a[1], HI ? hi.a[1] : 0u, w0 & 0x000F000Fu, w0s & 0x000F000Fu);
    mma16816(c, lo.a[2], HI ? hi.a[2] : 0u, lo.a[3], HI ? hi.a[3] : 0u, w0 & 0x00F000F0u, w0s & 0x00F000F0u);
    mma16816(c, lo.a[4], HI ? hi.a[4] : 0u, lo.a[5], HI ? hi.a[5] : 0u, w1 & 0x000F000Fu, w1s & 0x000F000Fu);
    mma16816(c, lo.a[6], HI ? hi.a[6] : 0u, lo.a[7], HI ? hi.a[7] : 0u, w1 & 0x00F000F0u, w1s & 0x00F000F0u);
}

enum OutMode { kOutActs = 0, kOutPartialF16 = 1, kOutPartialF32 = 2, kOutDenseF16 = 3 };

// Shared-memory layout per CTA:
//   ring[stage][warp][mat][step][lane] uint4      (packed codes, warp private)
//   sb[stage][mat][2][8 * NG] uint16              (scale and bias rows of the tile)
//   red[warp][mat][16 * 8] float                  (warp partials)
template <int NMAT>
struct SmemLayout {
    uint32_t warps, ng;
    __host__ __device__ size_t ring_bytes() const { return (size_t)kStages * warps * NMAT * (kGPW / 2) * kWarp * 16; }
    __host__ __device__ size_t sb_stage_bytes() const { return (size_t)NMAT * 2 * kTileRows * ng * 2; }
    __host__ __device__ size_t sb_bytes() const { return (size_t)kStages * sb_stage_bytes(); }
    __host__ __device__ size_t red_bytes() const { return (size_t)warps * NMAT * 128 * sizeof(float); }
    __host__ __device__ size_t total() const { return ring_bytes() + sb_bytes() + red_bytes(); }
};

template <int NMAT, bool DENSE, int OUT_MODE>
__global__ void __launch_bounds__(kMaxGroupedThreads)
grouped_mma_kernel(const GroupedArgs args) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t warps = blockDim.x / kWarp;
    const uint32_t ng = args.k / kGroup;
    const SmemLayout<NMAT> lay{warps, ng};
    uint4* ring = reinterpret_cast<uint4*>(smem);
    uint16_t* sb = reinterpret_cast<uint16_t*>(smem + lay.ring_bytes());
    float* red = reinterpret_cast<float*>(smem + lay.ring_bytes() + lay.sb_bytes());

    const uint32_t tiles = args.rows / kTileRows;
    const uint32_t total_chunks = DENSE ? (args.dense_tokens + kChunkTokens - 1) / kChunkTokens : args.counters[1];
    const uint64_t total_items = (uint64_t)total_chunks * tiles;
    // contiguous item range per CTA so that consecutive items share the chunk (activations stay in registers)
    const uint64_t item_begin = total_items * blockIdx.x / gridDim.x;
    const uint64_t item_end = total_items * (blockIdx.x + 1) / gridDim.x;
    if (item_begin >= item_end) return;

    const uint32_t g0 = warp * kGPW;                                   // first group of this warp
    const uint32_t ngw = g0 < ng ? (ng - g0 < (uint32_t)kGPW ? ng - g0 : (uint32_t)kGPW) : 0u;
    const size_t row_bytes = args.k / 2;

    // per-chunk state
    uint32_t cur_chunk = 0xFFFFFFFFu;
    MatPlanes planes[NMAT];
    uint32_t ntok = 0, row_base = 0;          // routed: first sorted-pair index; dense: first token
    XFrag xlo[kGPW], xhi[kGPW];

    auto resolve_chunk = [&](uint32_t chunk, MatPlanes (&pl)[NMAT], uint32_t& ntok_o, uint32_t& base_o) {
        if constexpr (DENSE) {
#pragma unroll
            for (int m = 0; m < NMAT; ++m) pl[m] = args.dense[m];
            base_o = chunk * kChunkTokens;
            const uint32_t left = args.dense_tokens - base_o;
            ntok_o = left < (uint32_t)kChunkTokens ? left : (uint32_t)kChunkTokens;
        } else {
            const uint32_t gi = args.chunk_group[chunk];
            const tf_group grp = args.groups[gi];
            const uint32_t cin = chunk - args.chunk_start[gi];
            const uint8_t* blob = args.pool_base + (uint64_t)grp.expert * args.expert_stride;
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                pl[m].W = blob + args.w_off[m];
                pl[m].S = reinterpret_cast<const uint16_t*>(blob + args.s_off[m]);
                pl[m].B = reinterpret_cast<const uint16_t*>(blob + args.b_off[m]);
            }
            base_o = grp.pair_start + cin * kChunkTokens;
            const uint32_t left = grp.pair_count - cin * kChunkTokens;
            ntok_o = left < (uint32_t)kChunkTokens ? left : (uint32_t)kChunkTokens;
        }
    };

    // issue the cp.async copies of one item into a ring stage
    auto issue = [&](uint64_t item, int stage) {
        if (item < item_end) {
            const uint32_t chunk = (uint32_t)(item / tiles), tile = (uint32_t)(item % tiles);
            MatPlanes pl[NMAT];
            uint32_t nt, rb;
            resolve_chunk(chunk, pl, nt, rb);
            const uint32_t row = tile * kTileRows + g;
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
#pragma unroll
                for (int s = 0; s < kGPW / 2; ++s) {
                    const uint32_t grp = g0 + 2 * s + (t >> 1);
                    const bool valid = (2u * s + (t >> 1)) < ngw;
                    const uint8_t* src = pl[m].W + (size_t)row * row_bytes + (size_t)(g0 + 2 * s) * 32 + t * 16;
                    uint4* dst = ring + ((((size_t)stage * warps + warp) * NMAT + m) * (kGPW / 2) + s) * kWarp + lane;
                    cp_async16(dst, valid ? src : pl[m].W, valid);
                    (void)grp;
                }
            }
            // scale / bias rows of the tile: 8 * ng 16-bit values per plane = ng 16-byte copies
            const uint32_t copies = NMAT * 2 * ng;
            for (uint32_t c = threadIdx.x; c < copies; c += blockDim.x) {
                const uint32_t m = c / (2 * ng), rest = c % (2 * ng), which = rest / ng, j = rest % ng;
                const uint16_t* plane = which == 0 ? pl[m].S : pl[m].B;
                const uint8_t* src = reinterpret_cast<const uint8_t*>(plane + (size_t)tile * kTileRows * ng) + j * 16;
                uint8_t* dst = reinterpret_cast<uint8_t*>(sb) + (size_t)stage * lay.sb_stage_bytes() +
                               ((size_t)(m * 2 + which) * kTileRows * ng) * 2 + j * 16;
                cp_async16(dst, src, true);
            }
        }
        cp_async_commit();
    };

#pragma unroll
    for (int p = 0; p < kStages - 1; ++p) issue(item_begin + p, p);

    for (uint64_t item = item_begin; item < item_end; ++item) {
        const int stage = (int)((item - item_begin) % kStages);
        issue(item + kStages - 1, (int)((item - item_begin + kStages - 1) % kStages));
        cp_async_wait<kStages - 1>();
        __syncthreads();

        const uint32_t chunk = (uint32_t)(item / tiles), tile = (uint32_t)(item % tiles);
        if (chunk != cur_chunk) {
            cur_chunk = chunk;
            resolve_chunk(chunk, planes, ntok, row_base);
#pragma unroll
            for (int i = 0; i < kGPW; ++i) {
                const bool gv = (uint32_t)i < ngw;
                const uint16_t* rlo = nullptr;
                const uint16_t* rhi = nullptr;
                if (gv && (uint32_t)g < ntok) {
                    const uint32_t r = DENSE || NMAT == 1 ? row_base + g : args.sorted_pairs[row_base + g].token;
                    rlo = args.x + (size_t)r * args.x_stride;
                }
                if (gv && (uint32_t)(g + 8) < ntok) {
                    const uint32_t r = DENSE || NMAT == 1 ? row_base + g + 8 : args.sorted_pairs[row_base + g + 8].token;
                    rhi = args.x + (size_t)r * args.x_stride;
                }
                load_xfrag(xlo[i], rlo, g0 + i, t);
                load_xfrag(xhi[i], rhi, g0 + i, t);
            }
        }

        float y[NMAT][4];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) { y[m][0] = y[m][1] = y[m][2] = y[m][3] = 0.0f; }
        const bool hi_tokens = ntok > 8;
        const uint16_t* sb_stage = reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(sb) +
                                                                     (size_t)stage * lay.sb_stage_bytes());
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
            const uint16_t* sm_s = sb_stage + (size_t)(m * 2 + 0) * kTileRows * ng;
            const uint16_t* sm_b = sb_stage + (size_t)(m * 2 + 1) * kTileRows * ng;
#pragma unroll
            for (int s = 0; s < kGPW / 2; ++s) {
                if (2u * s >= ngw) break;
                const uint4 v = ring[((((size_t)stage * warps + warp) * NMAT + m) * (kGPW / 2) + s) * kWarp + lane];
                // quad exchange: lanes t<2 hold two pieces of the even group, t>=2 of the odd group
                const bool low = t < 2;
                const uint32_t sx = low ? v.z : v.x, sy = low ? v.w : v.y;
                const uint32_t rx = __shfl_xor_sync(kFullMask, sx, 2), ry = __shfl_xor_sync(kFullMask, sy, 2);
                const uint32_t e0 = low ? v.x : rx, e1 = low ? v.y : ry;      // even group piece
                const uint32_t o0 = low ? rx : v.z, o1 = low ? ry : v.w;      // odd group piece
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int gi = 2 * s + half;
                    if ((uint32_t)gi >= ngw) break;
                    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (hi_tokens) group_mma<true>(c, half ? o0 : e0, half ? o1 : e1, xlo[gi], xhi[gi]);
                    else group_mma<false>(c, half ? o0 : e0, half ? o1 : e1, xlo[gi], xhi[gi]);
                    const uint32_t grp = g0 + gi;
                    const float s0 = bf16_bits_to_float(sm_s[(2 * t) * ng + grp]) * kTwo24;
                    const float s1 = bf16_bits_to_float(sm_s[(2 * t + 1) * ng + grp]) * kTwo24;
                    const float b0 = bf16_bits_to_float(sm_b[(2 * t) * ng + grp]);
                    const float b1 = bf16_bits_to_float(sm_b[(2 * t + 1) * ng + grp]);
                    y[m][0] = fmaf(s0, c[0], y[m][0]); y[m][0] = fmaf(b0, xlo[gi].sum, y[m][0]);
                    y[m][1] = fmaf(s1, c[1], y[m][1]); y[m][1] = fmaf(b1, xlo[gi].sum, y[m][1]);
                    if (hi_tokens) {
                        y[m][2] = fmaf(s0, c[2], y[m][2]); y[m][2] = fmaf(b0, xhi[gi].sum, y[m][2]);
                        y[m][3] = fmaf(s1, c[3], y[m][3]); y[m][3] = fmaf(b1, xhi[gi].sum, y[m][3]);
                    }
                }
            }
        }
        // warp partials -> shared, index = token * 8 + row
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
            float* r = red + ((size_t)warp * NMAT + m) * 128;
            r[g * 8 + 2 * t] = y[m][0];
            r[g * 8 + 2 * t + 1] = y[m][1];
            r[(g + 8) * 8 + 2 * t] = y[m][2];
            r[(g + 8) * 8 + 2 * t + 1] = y[m][3];
        }
        __syncthreads();
        for (uint32_t oi = threadIdx.x; oi < 128; oi += blockDim.x) {
            const uint32_t tok = oi >> 3, row = oi & 7;
            if (tok < ntok) {
                float acc[NMAT];
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                    float a = 0.0f;
                    for (uint32_t w2 = 0; w2 < warps; ++w2) a += red[((size_t)w2 * NMAT + m) * 128 + oi];
                    acc[m] = a;
                }
                const uint32_t out_row = tile * kTileRows + row;
                if constexpr (OUT_MODE == kOutActs) {
                    uint16_t* o = static_cast<uint16_t*>(args.out);
                    float gt = acc[0], up = acc[NMAT - 1];
                    if constexpr (DENSE) {
                        // shared expert: gate and up are stored as fp16 before the activation
                        // (Kernels/MoE/SharedExpertInt4.swift:62-93; Metal/Primitives/utility.metal:15-17)
                        gt = __half2float(__float2half_rn(gt));
                        up = __half2float(__float2half_rn(up));
                    }
                    // routed: act = half(gelu_tanh(gate) * up), gate and up in fp32 (prefill.metal:634-636; moe.metal:368)
                    o[(size_t)(row_base + tok) * args.out_stride + out_row] = __half_as_ushort(__float2half_rn(gelu_tanh(gt) * up));
                } else if constexpr (OUT_MODE == kOutDenseF16) {
                    uint16_t* o = static_cast<uint16_t*>(args.out);
                    o[(size_t)(row_base + tok) * args.out_stride + out_row] = __half_as_ushort(__float2half_rn(acc[0]));
                } else {
                    const tf_pair pr = args.sorted_pairs[row_base + tok];
                    const size_t idx = ((size_t)pr.token * args.top_k + pr.rank) * args.out_stride + out_row;
                    if constexpr (OUT_MODE == kOutPartialF16)
                        static_cast<uint16_t*>(args.out)[idx] = __half_as_ushort(__float2half_rn(acc[0]));   // prefill.metal:666-669
                    else
                        static_cast<float*>(args.out)[idx] = acc[0];
                }
            }
        }
        // the next iteration's first barrier orders these reads before the next writes of `red`
    }
    cp_async_wait<0>();
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

template <int NMAT, bool DENSE, int OUT_MODE>
static tf_status launch_grouped(tf_context* ctx, void* stream, const GroupedArgs& args, const char* name) {
    const uint32_t ng = args.k / kGroup;
    const uint32_t warps = (ng + kGPW - 1) / kGPW;
    TF_REQUIRE(ctx, warps >= 1 && warps <= (uint32_t)kMaxGroupedWarps, TF_ERR_UNSUPPORTED,
               "%s: K=%u outside the supported range (64..3072)", name, args.k);
    TF_REQUIRE(ctx, args.rows % kTileRows == 0, TF_ERR_UNSUPPORTED, "%s: row count %u must be a multiple of 8", name, args.rows);
    const SmemLayout<NMAT> lay{warps, ng};
    const size_t smem = lay.total();
    auto kern = grouped_mma_kernel<NMAT, DENSE, OUT_MODE>;
    // Attribute and occupancy are queried once per (instantiation, warp count) and cached,
    // so steady-state calls are a bare launch (and safe inside stream capture).
    static int cached_per_sm[kMaxGroupedWarps + 1] = {0};
    int per_sm = cached_per_sm[warps];
    if (per_sm == 0) {
        TF_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        TF_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, (int)(warps * kWarp), smem));
        if (per_sm < 1) per_sm = 1;
        if (per_sm > 8) per_sm = 8;
        cached_per_sm[warps] = per_sm;
    }
    uint32_t grid = (uint32_t)ctx->sm_count * (uint32_t)per_sm;
    if (DENSE) {
        const uint64_t items = (uint64_t)((args.dense_tokens + kChunkTokens - 1) / kChunkTokens) * (args.rows / kTileRows);
        if (items == 0) return TF_OK;
        if (items < grid) grid = (uint32_t)items;
    }
    kern<<<grid, warps * kWarp, smem, static_cast<cudaStream_t>(stream)>>>(args);
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

    tf::GroupedArgs a{};
    a.pool_base = static_cast<const uint8_t*>(pool_layer_base);
    a.expert_stride = expert_stride;
    a.w_off[0] = offsets->gate_w_off; a.s_off[0] = offsets->gate_s_off; a.b_off[0] = offsets->gate_b_off;
    a.w_off[1] = offsets->up_w_off;   a.s_off[1] = offsets->up_s_off;   a.b_off[1] = offsets->up_b_off;
    a.sorted_pairs = routes->sorted_pairs; a.groups = routes->groups; a.chunk_group = routes->chunk_group;
    a.chunk_start = routes->chunk_start; a.counters = routes->counters;
    a.x = reinterpret_cast<const uint16_t*>(hp); a.x_stride = hidden_stride_elements;
    a.out = acts_scratch; a.out_stride = f; a.rows = f; a.k = d; a.top_k = top_k;
    tf_status s = tf::launch_grouped<2, false, tf::kOutActs>(ctx, stream, a, "tf_grouped_moe_batched(gate/up)");
    if (s) return s;

    tf::GroupedArgs b{};
    b.pool_base = a.pool_base; b.expert_stride = expert_stride;
    b.w_off[0] = offsets->down_w_off; b.s_off[0] = offsets->down_s_off; b.b_off[0] = offsets->down_b_off;
    b.sorted_pairs = routes->sorted_pairs; b.groups = routes->groups; b.chunk_group = routes->chunk_group;
    b.chunk_start = routes->chunk_start; b.counters = routes->counters;
    b.x = static_cast<const uint16_t*>(acts_scratch); b.x_stride = f;
    b.out = route_partials; b.out_stride = d; b.rows = d; b.k = f; b.top_k = top_k;
    if (partials_f32) return tf::launch_grouped<1, false, tf::kOutPartialF32>(ctx, stream, b, "tf_grouped_moe_batched(down)");
    return tf::launch_grouped<1, false, tf::kOutPartialF16>(ctx, stream, b, "tf_grouped_moe_batched(down)");
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
    tf_status s = tf::launch_grouped<2, true, tf::kOutActs>(ctx, stream, a, "tf_shared_expert_int4_block(gate/up)");
    if (s) return s;
    tf::GroupedArgs b{};
    b.dense[0] = mp[2];
    b.x = static_cast<const uint16_t*>(scratch_act); b.x_stride = fs;
    b.out = tf::byte_ptr(y, y_off); b.out_stride = y_stride_elements; b.rows = d; b.k = fs; b.dense_tokens = rows;
    return tf::launch_grouped<1, true, tf::kOutDenseF16>(ctx, stream, b, "tf_shared_expert_int4_block(down)");
}

}  // extern "C"
