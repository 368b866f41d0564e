// Grouped int4 GEMM on the 5th-generation tensor cores for prefill-sized batches.
//
// Replaces mpp_prefill_affine_threadgroup_f16 (Metal/TensorCore/tensorops.metal:13-105; wrapper
// Kernels/TensorCore/MPPPrefillInt4QMM.swift:34-78), the reference's "dequantise a weight tile to half
// in threadgroup memory, then matrix-unit MMA with an fp32 accumulator" kernel, and the routed prefill
// kernels prefill_grouped_routed_moe_batched_phase1 / _down (Metal/Prefill/prefill.metal:598-670),
// which the reference runs as scalar per-thread dot products.
//
//   D[128 weight rows x N tokens] += W_tile[128 x 64] . X_tile[N x 64]^T      per 64-column group, N <= 256
//
// Weights are the A operand (M = 128), tokens the B operand (N = the tile's token count rounded up to 16,
// carried in the instruction descriptor), both K-major in shared memory with the 128-byte swizzle. Per step:
//   - one elected thread issues TMA tile loads (cp.async.bulk.tensor.2d, 64 rows each) of the activations;
//   - 256 dequantiser threads (two per weight row) read 16 packed bytes and the group's scale and bias and
//     write w = half(q * s + b), the reference's staged value (tensorops.metal:60-75), into the swizzled A tile;
//   - one elected thread issues four tcgen05.mma (K = 16 each) per matrix into TMEM accumulators and
//     commits the stage back to the producers through an mbarrier.
// After the last step eight epilogue warps read the accumulators with tcgen05.ld and apply GeGLU (gate and
// up accumulate side by side in TMEM) or a plain fp16 store, masked to the group's real tokens. The single
// matrix form double-buffers its accumulator so that the epilogue of one tile overlaps the next tile's MMAs.
// A persistent grid walks (group, token tile, weight-row tile) work items derived on the device from the
// routing metadata. Every mbarrier wait is bounded; on expiry the kernel records a code and leaves.
//
// Column order. The cheapest nibble extraction yields the eight codes of a 32-bit word in the order
// (0,4,1,5,2,6,3,7). A dot product does not care about the order as long as both operands agree, so the
// routed path stores its activations (the gathered rows and the GeGLU output) in that order within every
// eight columns (PERMUTED_K) and skips the four byte-permutes per word; the dense entry points take
// caller-owned activations in natural order and pay them.
#include <cuda.h>

#include "tf_common.cuh"

namespace tf {

constexpr int kQmmTokMax = 256;        // largest N of one MMA: tokens per tile
constexpr int kQmmBoxRows = 64;        // activation rows per TMA box
constexpr int kQmmRows = 128;          // M of the MMA: weight rows per tile
constexpr int kQmmK = 64;              // columns per step = one quantisation group = one 128-byte swizzle row
constexpr int kQmmMaxStages = 4;       // ring depth: 3 with two weight matrices per stage (64 KB), 4 with one (48 KB)
constexpr int kQmmDequantWarps = 8, kQmmEpilogueWarps = 8;
constexpr int kQmmFirstDequantWarp = 4, kQmmFirstEpilogueWarp = kQmmFirstDequantWarp + kQmmDequantWarps;
constexpr int kQmmThreads = (kQmmFirstEpilogueWarp + kQmmEpilogueWarps) * 32;   // warp 0: TMA, warp 1: MMA, 2-3 idle
constexpr int kQmmTmemCols = 512;      // the whole tensor memory: 2 x 256 accumulator columns
constexpr uint32_t kQmmSpin = 1u << 22;
constexpr uint32_t kErrQmmTimeout = 0x7E000000u;

static_assert(kQmmFirstEpilogueWarp % 4 == 0, "epilogue warp w reads TMEM lanes 32 * (w % 4)");

struct QmmGroup {
    const uint8_t* W[2];
    const uint16_t* S[2];
    const uint16_t* B[2];
    uint32_t row_start;     // first row of the group in the (sorted) activation matrix
    uint32_t count;         // tokens of the group
    uint32_t tile_start;    // first token tile of the group in the global tile order
    uint32_t pad;
};

static_assert(sizeof(QmmGroup) == 64, "the context allocates 64 bytes per group-table row");

struct QmmArgs {
    QmmGroup* groups;       // device array, filled by qmm_prepare_kernel
    uint32_t* totals;       // device: [0] group count, [1] token tiles
    // routed source (prepare kernel)
    const uint8_t* pool_base;
    uint64_t expert_stride;
    uint32_t w_off[2], s_off[2], b_off[2];
    const tf_group* route_groups;
    const uint32_t* route_counters;
    // dense source
    const uint8_t* dense_W[2];
    const uint16_t* dense_S[2];
    const uint16_t* dense_B[2];
    uint32_t dense_tokens;
    // problem
    uint32_t rows;          // weight rows (output features)
    uint32_t k;             // columns (input features)
    uint16_t* out;          // [tokens, out_stride] fp16
    uint32_t out_stride;
    uint32_t round_gate_up; // shared expert: gate and up rounded to fp16 before the activation
    uint32_t* error;
};

// ---- PTX wrappers ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void q_mbar_init(uint32_t addr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(addr), "r"(count) : "memory");
}
__device__ __forceinline__ void q_mbar_arrive(uint32_t addr) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void q_mbar_expect_tx(uint32_t addr, uint32_t bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool q_mbar_wait(uint32_t addr, uint32_t parity) {
    for (uint32_t i = 0; i < kQmmSpin; ++i) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int c0, int c1, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_dst), "l"(map), "r"(c0), "r"(c1), "r"(mbar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void q_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile with the 128-byte swizzle: rows of 128 bytes, 8-row atoms of 1024 bytes.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16, fp16 x fp16 -> fp32, both operands K-major, M = 128, N = n (a multiple of 16, at most 256).
__device__ __forceinline__ uint32_t qmm_idesc(uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((uint32_t)(kQmmRows >> 4) << 24);
}

// Builds the group table on the device: routed groups from the routing metadata, or one dense group.
__global__ void qmm_prepare_kernel(QmmArgs a, int nmat, int dense) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    uint32_t ng, tiles = 0;
    if (dense) {
        ng = 1;
        QmmGroup g{};
        for (int m = 0; m < nmat; ++m) { g.W[m] = a.dense_W[m]; g.S[m] = a.dense_S[m]; g.B[m] = a.dense_B[m]; }
        g.row_start = 0; g.count = a.dense_tokens; g.tile_start = 0;
        a.groups[0] = g;
        tiles = (a.dense_tokens + kQmmTokMax - 1) / kQmmTokMax;
    } else {
        ng = a.route_counters[0];
        for (uint32_t i = 0; i < ng; ++i) {
            const tf_group rg = a.route_groups[i];
            const uint8_t* blob = a.pool_base + (uint64_t)rg.expert * a.expert_stride;
            QmmGroup g{};
            for (int m = 0; m < nmat; ++m) {
                g.W[m] = blob + a.w_off[m];
                g.S[m] = reinterpret_cast<const uint16_t*>(blob + a.s_off[m]);
                g.B[m] = reinterpret_cast<const uint16_t*>(blob + a.b_off[m]);
            }
            g.row_start = rg.pair_start; g.count = rg.pair_count; g.tile_start = tiles;
            a.groups[i] = g;
            tiles += (rg.pair_count + kQmmTokMax - 1) / kQmmTokMax;
        }
    }
    a.totals[0] = ng;
    a.totals[1] = tiles;
}

template <int NMAT>
struct QmmSmem {
    static constexpr uint32_t kATile = kQmmRows * 128;                 // 16 KB
    static constexpr uint32_t kBTile = kQmmTokMax * 128;               // 32 KB
    static constexpr uint32_t kStage = NMAT * kATile + kBTile;         // 64 KB / 48 KB
    static constexpr int kStages = NMAT == 2 ? 3 : 4;
    static constexpr int kPrefetch = NMAT == 2 ? 3 : 4;               // k-steps of packed codes a dequantiser thread keeps in flight
    static constexpr uint32_t kRing = kStages * kStage;
    static constexpr uint32_t kBars = kRing;                           // barriers and the TMEM address
    static constexpr uint32_t kTotal = kRing + 256 + 1024;             // + barriers + slack for 1024-byte alignment
};

// Eight packed codes (one 32-bit word) -> eight fp16 weights w = half(q * s + b).
// Fast form: a nibble moved to bits 4..7 of a half is the subnormal q * 2^-20, so one HFMA2 with s * 2^20
// gives fma(q, s, b) rounded once (tensorops.metal:60-75 stores half(fma(q, s, b))); s * 2^20 is exact in
// fp16 (s is a bf16) while |s| < 2^-5. Larger scales take the two-step form (1024 + q) - 1024.
// Output order: PERMUTED (k0,k4,k1,k5,k2,k6,k3,k7), otherwise natural.
template <bool NATURAL_K>
__device__ __forceinline__ uint4 dequant8(uint32_t w, __half2 s_fast, __half2 s, __half2 b, bool fast) {
    uint32_t t0, t1, t2, t3;
    __half2 h0, h1, h2, h3;
    if (fast) {
        t0 = (w << 4) & 0x00F000F0u; t1 = w & 0x00F000F0u; t2 = (w >> 4) & 0x00F000F0u; t3 = (w >> 8) & 0x00F000F0u;
        h0 = __hfma2(*reinterpret_cast<__half2*>(&t0), s_fast, b);     // (k0, k4)
        h1 = __hfma2(*reinterpret_cast<__half2*>(&t1), s_fast, b);     // (k1, k5)
        h2 = __hfma2(*reinterpret_cast<__half2*>(&t2), s_fast, b);     // (k2, k6)
        h3 = __hfma2(*reinterpret_cast<__half2*>(&t3), s_fast, b);     // (k3, k7)
    } else {
        const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
        t0 = (w & 0x000F000Fu) | 0x64006400u; t1 = ((w >> 4) & 0x000F000Fu) | 0x64006400u;
        t2 = ((w >> 8) & 0x000F000Fu) | 0x64006400u; t3 = ((w >> 12) & 0x000F000Fu) | 0x64006400u;
        h0 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t0), k1024), s, b);
        h1 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t1), k1024), s, b);
        h2 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t2), k1024), s, b);
        h3 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t3), k1024), s, b);
    }
    const uint32_t u0 = *reinterpret_cast<uint32_t*>(&h0), u1 = *reinterpret_cast<uint32_t*>(&h1);
    const uint32_t u2 = *reinterpret_cast<uint32_t*>(&h2), u3 = *reinterpret_cast<uint32_t*>(&h3);
    if (!NATURAL_K) return make_uint4(u0, u1, u2, u3);
    uint4 o;
    asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(o.x) : "r"(u0), "r"(u1));   // (k0, k1)
    asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(o.y) : "r"(u2), "r"(u3));   // (k2, k3)
    asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(o.z) : "r"(u0), "r"(u1));   // (k4, k5)
    asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(o.w) : "r"(u2), "r"(u3));   // (k6, k7)
    return o;
}

// Position of column k within its eight-column block in the PERMUTED order.
__device__ __forceinline__ uint32_t permuted_col(uint32_t k) { return (k & ~7u) | ((k & 3u) << 1) | ((k >> 2) & 1u); }

// Accumulator placement in the 512 TMEM columns, two buffers of 256. A tile whose accumulators fit one buffer
// (one matrix, or two matrices of at most 128 tokens) takes the buffer used less often so far, so consecutive
// tiles alternate and the epilogue of one overlaps the MMAs of the next; a two-matrix tile of more than 128
// tokens takes both. The MMA issuer and the epilogue warps replay the same sequence, so they agree.
struct AccPlan {
    uint32_t uses0 = 0u, uses1 = 0u;
    bool both = false;
    uint32_t buf = 0, col0 = 0, mat_stride = 0;
    template <int NMAT>
    __device__ __forceinline__ void next(uint32_t n_mma) {
        both = NMAT == 2 && n_mma > 128u;
        buf = both ? 0u : (uses0 <= uses1 ? 0u : 1u);
        col0 = buf * 256u;
        mat_stride = both ? 256u : 128u;
    }
    __device__ __forceinline__ bool takes(uint32_t b) const { return both || b == buf; }
    __device__ __forceinline__ uint32_t uses(uint32_t b) const { return b ? uses1 : uses0; }
    __device__ __forceinline__ void done() {
        if (both || buf == 0) ++uses0;
        if (both || buf == 1) ++uses1;
    }
};

template <int NMAT, bool NATURAL_K>
__global__ void __launch_bounds__(kQmmThreads, 1)
qmm_tcgen05_kernel(const __grid_constant__ CUtensorMap x_map, const QmmArgs args) {
    extern __shared__ uint8_t smem_raw[];
    using L = QmmSmem<NMAT>;
    constexpr int kQmmStages = L::kStages;
    constexpr int kQmmPrefetch = L::kPrefetch;
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                      // swizzle atoms need 1024-byte alignment
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t bars = base + L::kBars;
    auto bar_full_a = [&](uint32_t s) { return bars + s * 8; };
    auto bar_full_b = [&](uint32_t s) { return bars + (kQmmMaxStages + s) * 8; };
    auto bar_empty = [&](uint32_t s) { return bars + (2 * kQmmMaxStages + s) * 8; };
    auto bar_acc_full = [&](uint32_t b) { return bars + (3 * kQmmMaxStages + b) * 8; };
    auto bar_acc_empty = [&](uint32_t b) { return bars + (3 * kQmmMaxStages + 2 + b) * 8; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + L::kBars + (3 * kQmmMaxStages + 4) * 8);

    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t ksteps = args.k / kQmmK;
    const uint32_t groups_per_row = args.k / kGroup;
    const uint32_t row_bytes = args.k / 2;
    const uint32_t wrow_tiles = (args.rows + kQmmRows - 1) / kQmmRows;
    const uint32_t ngroups = args.totals[0];
    const uint32_t total_tiles = args.totals[1] * wrow_tiles;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < (uint32_t)kQmmStages; ++s) {
            q_mbar_init(bar_full_a(s), kQmmDequantWarps);   // one arrival per dequantiser warp
            q_mbar_init(bar_full_b(s), 1);                  // the TMA thread's expect_tx
            q_mbar_init(bar_empty(s), 1);                   // tcgen05.commit
        }
        for (uint32_t b = 0; b < 2; ++b) {
            q_mbar_init(bar_acc_full(b), 1);                // tcgen05.commit after the last step
            q_mbar_init(bar_acc_empty(b), kQmmEpilogueWarps);
        }
        q_fence_async_smem();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(const_cast<uint32_t*>(tmem_slot))), "r"((uint32_t)kQmmTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // maps a work item to (group, token tile within the group, weight-row tile)
    auto locate = [&](uint32_t tile, uint32_t& gi, uint32_t& tt, uint32_t& wt) {
        const uint32_t tglob = tile / wrow_tiles;
        wt = tile % wrow_tiles;
        uint32_t lo = 0, hi = ngroups;                                 // last group with tile_start <= tglob
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (args.groups[mid].tile_start <= tglob) lo = mid; else hi = mid;
        }
        gi = lo;
        tt = tglob - args.groups[lo].tile_start;
    };
    // tokens of a tile, and the MMA's N (rounded up to 16)
    auto tile_tokens = [&](uint32_t count, uint32_t tt) {
        const uint32_t left = count - tt * kQmmTokMax;
        return left < (uint32_t)kQmmTokMax ? left : (uint32_t)kQmmTokMax;
    };

    uint32_t fail = 0;
    uint32_t it = 0;         // running k-step index over all of this CTA's tiles (ring position)

    if (warp == 0) {
        // ===================== TMA producer: activation tiles =====================
        for (uint32_t tile = blockIdx.x; tile < total_tiles && !fail; tile += gridDim.x) {
            uint32_t gi, tt, wt;
            locate(tile, gi, tt, wt);
            const uint32_t row0 = args.groups[gi].row_start + tt * kQmmTokMax;
            const uint32_t boxes = (tile_tokens(args.groups[gi].count, tt) + kQmmBoxRows - 1) / kQmmBoxRows;
            for (uint32_t ks = 0; ks < ksteps; ++ks, ++it) {
                const uint32_t s = it % kQmmStages, use = it / kQmmStages;
                if (use > 0 && !q_mbar_wait(bar_empty(s), (use - 1) & 1)) { fail = kErrQmmTimeout | 1; break; }
                if (lane == 0) {
                    q_mbar_expect_tx(bar_full_b(s), boxes * kQmmBoxRows * 128);
                    for (uint32_t b = 0; b < boxes; ++b)
                        tma_load_2d(base + s * L::kStage + NMAT * L::kATile + b * kQmmBoxRows * 128, &x_map, (int)(ks * kQmmK),
                                    (int)(row0 + b * kQmmBoxRows), bar_full_b(s));
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        AccPlan plan;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && !fail; tile += gridDim.x) {
            uint32_t gi, tt, wt;
            locate(tile, gi, tt, wt);
            const uint32_t n_mma = (tile_tokens(args.groups[gi].count, tt) + 15u) & ~15u;
            const uint32_t idesc = qmm_idesc(n_mma);
            plan.next<NMAT>(n_mma);
#pragma unroll
            for (uint32_t b = 0; b < 2; ++b) {
                if (plan.takes(b) && plan.uses(b) > 0 && !q_mbar_wait(bar_acc_empty(b), (plan.uses(b) - 1) & 1))
                    fail = kErrQmmTimeout | 2;
            }
            if (fail) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + plan.col0;
            for (uint32_t ks = 0; ks < ksteps; ++ks, ++it) {
                const uint32_t s = it % kQmmStages, use = it / kQmmStages;
                if (!q_mbar_wait(bar_full_a(s), use & 1) || !q_mbar_wait(bar_full_b(s), use & 1)) { fail = kErrQmmTimeout | 3; break; }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t stage = base + s * L::kStage;
                    const uint64_t b_desc = umma_smem_desc(stage + NMAT * L::kATile);
#pragma unroll
                    for (int m = 0; m < NMAT; ++m) {
                        const uint64_t a_desc = umma_smem_desc(stage + m * L::kATile);
#pragma unroll
                        for (int j = 0; j < kQmmK / 16; ++j)      // 16 columns = 32 bytes along K per MMA
                            tc_mma_f16(acc + m * plan.mat_stride, a_desc + (uint64_t)(j * 2), b_desc + (uint64_t)(j * 2), idesc,
                                       (ks > 0 || j > 0) ? 1u : 0u);
                    }
                    tc_commit(bar_empty(s));                      // the stage is free once these MMAs have read it
                    if (ks + 1 == ksteps) {
                        if (plan.both || plan.buf == 0) tc_commit(bar_acc_full(0));
                        if (plan.both || plan.buf == 1) tc_commit(bar_acc_full(1));
                    }
                }
                __syncwarp();
            }
            plan.done();
        }
    } else if (warp >= kQmmFirstDequantWarp && warp < kQmmFirstEpilogueWarp) {
        // ===================== dequantisers: two threads per weight row =====================
        const uint32_t idx = threadIdx.x - kQmmFirstDequantWarp * kWarp;
        const uint32_t r = idx >> 1, hf = idx & 1;               // row within the tile, half of the 64 columns
        const uint32_t row_off = (r >> 3) * 1024 + (r & 7) * 128, sw = r & 7;
        const uint32_t my_tiles = total_tiles > blockIdx.x ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
        const uint32_t total_steps = my_tiles * ksteps;
        // The packed codes come straight from global memory, so each thread keeps a few k-steps of them in
        // flight in registers (kPrefetch); the fetch cursor runs ahead of the processing loop and crosses tile boundaries.
        uint32_t f_tile = blockIdx.x, f_ks = 0;
        const uint8_t* f_w[NMAT];
        const uint16_t* f_s[NMAT];
        const uint16_t* f_b[NMAT];
        bool f_valid = false;
        auto f_resolve = [&]() {
            uint32_t gi, tt, wt;
            locate(f_tile, gi, tt, wt);
            const uint32_t wrow = wt * kQmmRows + r;
            f_valid = wrow < args.rows;
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                f_w[m] = args.groups[gi].W[m] + (size_t)wrow * row_bytes + hf * 16;
                f_s[m] = args.groups[gi].S[m] + (size_t)wrow * groups_per_row;
                f_b[m] = args.groups[gi].B[m] + (size_t)wrow * groups_per_row;
            }
        };
        uint4 codes[kQmmPrefetch][NMAT];
        uint32_t sb[kQmmPrefetch][NMAT];
        auto fetch = [&](uint4 (&c)[NMAT], uint32_t (&q)[NMAT]) {
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                if (f_valid) {
                    c[m] = __ldg(reinterpret_cast<const uint4*>(f_w[m] + f_ks * 32));
                    q[m] = (uint32_t)__ldg(f_s[m] + f_ks) | ((uint32_t)__ldg(f_b[m] + f_ks) << 16);
                } else {
                    c[m] = make_uint4(0u, 0u, 0u, 0u);
                    q[m] = 0u;
                }
            }
            if (++f_ks == ksteps) {
                f_ks = 0;
                f_tile += gridDim.x;
                if (f_tile < total_tiles) f_resolve();
            }
        };
        if (total_steps) f_resolve();
#pragma unroll
        for (int p = 0; p < kQmmPrefetch; ++p)
            if ((uint32_t)p < total_steps) fetch(codes[p], sb[p]);
        for (uint32_t it0 = 0; it0 < total_steps && !fail; it0 += kQmmPrefetch) {
#pragma unroll
            for (int p = 0; p < kQmmPrefetch; ++p) {
                const uint32_t itp = it0 + p;
                if (itp >= total_steps) break;
                const uint32_t s = itp % kQmmStages, use = itp / kQmmStages;
                if (use > 0 && !q_mbar_wait(bar_empty(s), (use - 1) & 1)) { fail = kErrQmmTimeout | 4; break; }
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                    const float sf = bf16_bits_to_float((uint16_t)(sb[p][m] & 0xFFFFu)), bf = bf16_bits_to_float((uint16_t)(sb[p][m] >> 16));
                    const bool fast = fabsf(sf) < 0.03125f;
                    const __half2 s_fast = __float2half2_rn(sf * 1048576.0f), s2 = __float2half2_rn(sf), b2 = __float2half2_rn(bf);
                    uint8_t* arow = base_ptr + s * L::kStage + m * L::kATile + row_off;
                    const uint32_t w[4] = {codes[p][m].x, codes[p][m].y, codes[p][m].z, codes[p][m].w};
#pragma unroll
                    for (int c = 0; c < 4; ++c)                   // 8 codes -> 16 bytes = one swizzle chunk
                        *reinterpret_cast<uint4*>(arow + (((hf * 4 + c) ^ sw) << 4)) = dequant8<NATURAL_K>(w[c], s_fast, s2, b2, fast);
                }
                q_fence_async_smem();                             // generic writes -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) q_mbar_arrive(bar_full_a(s));
                if (itp + kQmmPrefetch < total_steps) fetch(codes[p], sb[p]);   // refill the slot just consumed
            }
        }
    } else if (warp >= kQmmFirstEpilogueWarp) {
        // ===================== epilogue: TMEM -> registers -> global =====================
        const uint32_t q = warp & 3;                              // TMEM lane quarter this warp may read
        const uint32_t chunk_par = (warp - kQmmFirstEpilogueWarp) >> 2;   // which 16-column chunks this warp takes
        const uint32_t r = q * kWarp + lane;                      // weight row within the tile = TMEM lane
        AccPlan plan;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && !fail; tile += gridDim.x) {
            uint32_t gi, tt, wt;
            locate(tile, gi, tt, wt);
            const QmmGroup grp = args.groups[gi];
            const uint32_t wrow = wt * kQmmRows + r;
            const uint32_t out_col = (NMAT == 2 && !NATURAL_K) ? permuted_col(wrow) : wrow;   // the GeGLU output feeds the down GEMM
            const uint32_t tok0 = tt * kQmmTokMax;
            const uint32_t ntok = tile_tokens(grp.count, tt);
            plan.next<NMAT>((ntok + 15u) & ~15u);
#pragma unroll
            for (uint32_t b = 0; b < 2; ++b) {
                if (plan.takes(b) && !q_mbar_wait(bar_acc_full(b), plan.uses(b) & 1)) fail = kErrQmmTimeout | 5;
            }
            if (fail) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + ((q * kWarp) << 16) + plan.col0;
            uint16_t* out_row = args.out + (size_t)(grp.row_start + tok0) * args.out_stride + out_col;
            for (uint32_t c0 = chunk_par * 16; c0 < ntok; c0 += 32) {
                uint32_t v0[16], v1[16];
                tc_ld16(acc + c0, v0);
                if (NMAT == 2) tc_ld16(acc + plan.mat_stride + c0, v1);
                tc_wait_ld();
                if (wrow < args.rows) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const uint32_t tok = c0 + j;
                        if (tok < ntok) {
                            float y = __uint_as_float(v0[j]);
                            if (NMAT == 2) {
                                float gt = y, up = __uint_as_float(v1[j]);
                                if (args.round_gate_up) {          // Kernels/MoE/SharedExpertInt4.swift:62-93
                                    gt = __half2float(__float2half_rn(gt));
                                    up = __half2float(__float2half_rn(up));
                                }
                                y = gelu_tanh(gt) * up;            // prefill.metal:634-636
                            }
                            out_row[(size_t)tok * args.out_stride] = __half_as_ushort(__float2half_rn(y));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (plan.both || plan.buf == 0) q_mbar_arrive(bar_acc_empty(0));
                if (plan.both || plan.buf == 1) q_mbar_arrive(bar_acc_empty(1));
            }
            plan.done();
        }
    }
    if (fail && lane == 0) atomicCAS(args.error, 0u, fail);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kQmmTmemCols) : "memory");
    }
}

// ---- host side ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// fp16 matrix [rows, k] with a row stride: box = 64 columns x 64 rows, 128-byte swizzle, zero fill outside.
static tf_status make_x_map(tf_context* ctx, CUtensorMap* map, const void* x, uint64_t rows, uint32_t k, uint32_t stride_elems,
                            const char* name) {
    EncodeTiledFn fn = encode_tiled_fn();
    TF_REQUIRE(ctx, fn != nullptr, TF_ERR_UNSUPPORTED, "%s: cuTensorMapEncodeTiled is not available in this driver", name);
    const cuuint64_t dims[2] = {k, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)stride_elems * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kQmmK, (cuuint32_t)kQmmBoxRows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TF_REQUIRE(ctx, r == CUDA_SUCCESS, TF_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed (%d)", name, (int)r);
    return TF_OK;
}

template <int NMAT, bool NATURAL_K>
static tf_status launch_qmm(tf_context* ctx, void* stream, QmmArgs& a, const void* x, uint64_t x_rows, uint32_t x_stride,
                            bool dense, const char* name) {
    TF_REQUIRE(ctx, a.k % kQmmK == 0 && a.k >= (uint32_t)kQmmK, TF_ERR_INVALID_ARGUMENT, "%s: K must be a positive multiple of 64", name);
    TF_REQUIRE(ctx, aligned(x, 16) && (x_stride * 2) % 16 == 0, TF_ERR_ALIGNMENT, "%s: activation rows must be 16-byte aligned", name);
    TF_REQUIRE(ctx, ctx->qmm_groups != nullptr, TF_ERR_OUT_OF_MEMORY, "%s: context scratch missing", name);
    CUtensorMap map;
    if (tf_status s = make_x_map(ctx, &map, x, x_rows, a.k, x_stride, name)) return s;
    a.groups = static_cast<QmmGroup*>(ctx->qmm_groups);
    a.totals = ctx->qmm_totals;
    a.error = ctx->device_error;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    qmm_prepare_kernel<<<1, 32, 0, st>>>(a, NMAT, dense ? 1 : 0);
    if (tf_status s = check_launch(ctx, "qmm_prepare")) return s;
    auto kern = qmm_tcgen05_kernel<NMAT, NATURAL_K>;
    static bool configured = false;
    if (!configured) {
        TF_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)QmmSmem<NMAT>::kTotal));
        configured = true;
    }
    kern<<<ctx->sm_count, kQmmThreads, QmmSmem<NMAT>::kTotal, st>>>(map, a);
    return check_launch(ctx, name);
}

}  // namespace tf

extern "C" {

tf_status tf_grouped_moe_tensorcore(tf_context* ctx, void* stream, const void* x_sorted, uint32_t x_rows,
                                    const void* pool_layer_base, uint64_t expert_stride, const tf_expert_offsets* offsets,
                                    const tf_device_routes* routes, void* acts_scratch, void* out_rows,
                                    uint32_t d, uint32_t f) {
    const char* name = "tf_grouped_moe_tensorcore";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, x_sorted && pool_layer_base && offsets && routes && acts_scratch && out_rows, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, d % 64 == 0 && f % 64 == 0 && d > 0 && f > 0, TF_ERR_INVALID_ARGUMENT, "%s: D and F must be positive multiples of 64", name);
    const uint32_t all[9] = {offsets->gate_w_off, offsets->gate_s_off, offsets->gate_b_off, offsets->up_w_off, offsets->up_s_off,
                             offsets->up_b_off, offsets->down_w_off, offsets->down_s_off, offsets->down_b_off};
    for (uint32_t v : all) TF_REQUIRE(ctx, v % 16 == 0, TF_ERR_ALIGNMENT, "%s: blob sub-tensor offset %u is not a multiple of 16 bytes", name, v);
    TF_REQUIRE(ctx, tf::aligned(pool_layer_base, 16) && expert_stride % 16 == 0, TF_ERR_ALIGNMENT, "%s: pool must be 16-byte aligned", name);
    if (x_rows == 0) return TF_OK;
    tf::QmmArgs a{};
    a.pool_base = static_cast<const uint8_t*>(pool_layer_base); a.expert_stride = expert_stride;
    a.w_off[0] = offsets->gate_w_off; a.s_off[0] = offsets->gate_s_off; a.b_off[0] = offsets->gate_b_off;
    a.w_off[1] = offsets->up_w_off;   a.s_off[1] = offsets->up_s_off;   a.b_off[1] = offsets->up_b_off;
    a.route_groups = routes->groups; a.route_counters = routes->counters;
    a.rows = f; a.k = d; a.out = static_cast<uint16_t*>(acts_scratch); a.out_stride = f; a.round_gate_up = 0;
    if (tf_status s = tf::launch_qmm<2, false>(ctx, stream, a, x_sorted, x_rows, d, false, "tf_grouped_moe_tensorcore(gate/up)")) return s;
    tf::QmmArgs b{};
    b.pool_base = a.pool_base; b.expert_stride = expert_stride;
    b.w_off[0] = offsets->down_w_off; b.s_off[0] = offsets->down_s_off; b.b_off[0] = offsets->down_b_off;
    b.route_groups = routes->groups; b.route_counters = routes->counters;
    b.rows = d; b.k = f; b.out = static_cast<uint16_t*>(out_rows); b.out_stride = d;
    return tf::launch_qmm<1, false>(ctx, stream, b, acts_scratch, x_rows, f, false, "tf_grouped_moe_tensorcore(down)");
}

tf_status tf_int4_qmm(tf_context* ctx, void* stream, const void* weights, uint64_t weights_off, const void* scales,
                      uint64_t scales_off, const void* biases, uint64_t biases_off, const void* x, uint64_t x_off,
                      void* y, uint64_t y_off, uint32_t m, uint32_t n, uint32_t k) {
    const char* name = "tf_int4_qmm";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, weights && scales && biases && x && y, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    TF_REQUIRE(ctx, k % 64 == 0 && k > 0, TF_ERR_INVALID_ARGUMENT, "%s: K must be a positive multiple of 64", name);   // MPPPrefillInt4QMM.swift:43-55
    if (m == 0 || n == 0) return TF_OK;
    tf::QmmArgs a{};
    a.dense_W[0] = tf::byte_ptr(weights, weights_off);
    a.dense_S[0] = reinterpret_cast<const uint16_t*>(tf::byte_ptr(scales, scales_off));
    a.dense_B[0] = reinterpret_cast<const uint16_t*>(tf::byte_ptr(biases, biases_off));
    TF_REQUIRE(ctx, tf::aligned(a.dense_W[0], 16) && tf::aligned(a.dense_S[0], 2) && tf::aligned(a.dense_B[0], 2) && (k / 2) % 16 == 0,
               TF_ERR_ALIGNMENT, "%s: packed rows must be 16-byte aligned", name);
    a.dense_tokens = m; a.rows = n; a.k = k;
    a.out = reinterpret_cast<uint16_t*>(tf::byte_ptr(y, y_off)); a.out_stride = n;
    return tf::launch_qmm<1, true>(ctx, stream, a, tf::byte_ptr(x, x_off), m, k, true, name);
}

tf_status tf_shared_expert_int4_tensorcore(tf_context* ctx, void* stream, const void* x, uint32_t x_stride_elements,
                                           const tf_projection* gate, const tf_projection* up, const tf_projection* down,
                                           void* y, uint32_t y_stride_elements, void* scratch_act, uint32_t rows) {
    const char* name = "tf_shared_expert_int4_tensorcore";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, x && gate && up && down && y && scratch_act, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, gate->rows == up->rows && gate->cols == up->cols && down->rows == gate->cols && down->cols == gate->rows,
               TF_ERR_DIMENSION_MISMATCH, "SharedExpert dimension mismatch: gate=(%u,%u) up=(%u,%u) down=(%u,%u)",
               gate->rows, gate->cols, up->rows, up->cols, down->rows, down->cols);
    if (rows == 0) return TF_OK;
    const uint32_t fs = gate->rows, d = gate->cols;
    const tf_projection* ps[3] = {gate, up, down};
    const uint8_t* W[3]; const uint16_t* S[3]; const uint16_t* B[3];
    for (int i = 0; i < 3; ++i) {
        W[i] = tf::byte_ptr(ps[i]->weights, ps[i]->weights_off);
        S[i] = reinterpret_cast<const uint16_t*>(tf::byte_ptr(ps[i]->scales, ps[i]->scales_off));
        B[i] = reinterpret_cast<const uint16_t*>(tf::byte_ptr(ps[i]->biases, ps[i]->biases_off));
        TF_REQUIRE(ctx, tf::aligned(W[i], 16) && tf::aligned(S[i], 2) && tf::aligned(B[i], 2), TF_ERR_ALIGNMENT, "%s: planes must be 16-byte aligned", name);
    }
    tf::QmmArgs a{};
    a.dense_W[0] = W[0]; a.dense_S[0] = S[0]; a.dense_B[0] = B[0];
    a.dense_W[1] = W[1]; a.dense_S[1] = S[1]; a.dense_B[1] = B[1];
    a.dense_tokens = rows; a.rows = fs; a.k = d; a.out = static_cast<uint16_t*>(scratch_act); a.out_stride = fs; a.round_gate_up = 1;
    if (tf_status s = tf::launch_qmm<2, true>(ctx, stream, a, x, rows, x_stride_elements, true, "tf_shared_expert_int4_tensorcore(gate/up)")) return s;
    tf::QmmArgs b{};
    b.dense_W[0] = W[2]; b.dense_S[0] = S[2]; b.dense_B[0] = B[2];
    b.dense_tokens = rows; b.rows = d; b.k = fs; b.out = static_cast<uint16_t*>(y); b.out_stride = y_stride_elements;
    return tf::launch_qmm<1, true>(ctx, stream, b, scratch_act, rows, fs, true, "tf_shared_expert_int4_tensorcore(down)");
}

}  // extern "C"
