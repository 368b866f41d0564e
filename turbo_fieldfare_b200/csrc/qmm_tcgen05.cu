// Grouped int4 GEMM on the 5th-generation tensor cores (tcgen05 / TMEM) for batches of eight tokens and more.
//
// Replaces mpp_prefill_affine_threadgroup_f16 (Metal/TensorCore/tensorops.metal:13-105; wrapper
// Kernels/TensorCore/MPPPrefillInt4QMM.swift:34-78), the reference's "dequantise a weight tile to half,
// then matrix-unit MMA with an fp32 accumulator" kernel, and the routed prefill kernels
// prefill_grouped_routed_moe_batched_phase1 / _down (Metal/Prefill/prefill.metal:598-670), which the
// reference runs as scalar per-thread dot products.
//
//   D[128 weight rows x N tokens] += W_tile[128 x 128] . X_tile[N x 128]^T     per step of two 64-column groups, N <= 128
//
// Weights are the A operand (M = 128) and are fed to the MMA from TENSOR MEMORY; tokens are the B operand
// (N = the tile's token count rounded up to 16, carried in the instruction descriptor) in shared memory,
// K-major with the 128-byte swizzle. Data path of the weights, which carry nearly all the bytes:
//   HBM --TMA tile load--> shared memory (packed, 64 bytes per row and step)
//       --LDS.128--> registers --one HFMA2 per two codes--> w = half(q * s + b)     (tensorops.metal:60-75)
//       --tcgen05.st--> tensor memory --tcgen05.mma--> fp32 accumulators in tensor memory.
// The dequantised tile never touches shared memory: an fp16 copy of the weights is four times the packed
// bytes, and writing it to shared memory and reading it back for the MMA would cost more shared-memory
// bandwidth than the whole HBM stream.
// Roles of the 24 warps: warp 0 issues every asynchronous copy (packed codes per step, activation boxes of 16
// or 128 rows per step, the tile's scale and bias planes as 1-D bulk copies); warp 1 issues the MMAs and commits
// stages back through mbarriers; warps 4-19 dequantise (four threads per weight row); warps 20-23 read the
// accumulators with tcgen05.ld and apply GeGLU (gate and up accumulate side by side) or a plain fp16 store,
// masked to the group's real tokens. Accumulators of tiles with at most 64 tokens (one matrix: any tile)
// alternate between two buffers so that the epilogue overlaps the next tile's MMAs.
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

constexpr int kQmmTokMax = 128;        // largest N of one MMA: tokens per tile
constexpr int kQmmBoxRows = 16;        // activation rows per TMA box (2 KB per step)
constexpr int kQmmRows = 128;          // M of the MMA: weight rows per tile
constexpr int kQmmK = 128;             // columns per step: two quantisation groups, so that the per-step costs of the
                                       // single-thread roles (waits, descriptors, commits) are paid once per 128 columns
constexpr int kQmmRawStages = 4;       // ring of packed-code stages (NMAT x 8 KB each)
constexpr int kQmmBSlots = 32;         // ring of activation slots (16 rows x 64 columns, 2 KB); a step takes 2, 4, 8 or 16
constexpr int kQmmFirstDequantWarp = 4, kQmmDequantWarps = 16;      // four threads per weight row
constexpr int kQmmFirstEpilogueWarp = 20, kQmmEpilogueWarps = 4;
constexpr int kQmmThreads = (kQmmFirstEpilogueWarp + kQmmEpilogueWarps) * 32;
constexpr int kQmmTmemCols = 512;      // columns 0..255: accumulators; 256..511: ring of dequantised weight stages
constexpr int kQmmAccCols = 256;
constexpr uint32_t kQmmSpin = 1u << 22;
constexpr uint32_t kErrQmmTimeout = 0x7E000000u;
static_assert(kQmmFirstEpilogueWarp % 4 == 0 && kQmmFirstDequantWarp % 4 == 0, "warp w touches TMEM lanes 32 * (w % 4)");

struct QmmGroup {
    const uint16_t* S[2];   // scale / bias planes of the group's matrices
    const uint16_t* B[2];
    uint32_t expert;        // third coordinate of the weight tensor maps (0 for a dense matrix)
    uint32_t row_start;     // first row of the group in the (sorted) activation matrix
    uint32_t count;         // tokens of the group
    uint32_t tile_start;    // first token tile of the group in the global tile order
    uint32_t pad[4];
};
static_assert(sizeof(QmmGroup) == 64, "the context allocates 64 bytes per group-table row");

struct QmmArgs {
    QmmGroup* groups;       // device array, filled by qmm_prepare_kernel
    uint32_t* totals;       // device: [0] group count, [1] token tiles
    // routed source (prepare kernel)
    const uint8_t* pool_base;
    uint64_t expert_stride;
    uint32_t s_off[2], b_off[2];
    const tf_group* route_groups;
    const uint32_t* route_counters;
    // dense source
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
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(mbar) : "memory");
}
__device__ __forceinline__ void q_bulk_g2s(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t mbar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(mbar) : "memory");
}
// One lane of a converged warp; the address arithmetic around the elected instruction stays warp-uniform, so the
// compiler keeps descriptors in uniform registers instead of moving them over for every instruction.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile("{\n\t.reg .pred px;\n\telect.sync _|px, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, px;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void q_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 16 consecutive 32-bit columns of this thread's TMEM lane <- 16 registers (four uint4)
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint4& a, const uint4& b, const uint4& c, const uint4& d) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w),
                   "r"(c.x), "r"(c.y), "r"(c.z), "r"(c.w), "r"(d.x), "r"(d.y), "r"(d.z), "r"(d.w) : "memory");
}
// 8 consecutive 32-bit columns of this thread's TMEM lane <- 8 registers
__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint4& a, const uint4& b) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ uint4 q_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 q_lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t q_lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

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
        for (int m = 0; m < nmat; ++m) { g.S[m] = a.dense_S[m]; g.B[m] = a.dense_B[m]; }
        g.expert = 0; g.row_start = 0; g.count = a.dense_tokens; g.tile_start = 0;
        a.groups[0] = g;
        tiles = (a.dense_tokens + kQmmTokMax - 1) / kQmmTokMax;
    } else {
        ng = a.route_counters[0];
        for (uint32_t i = 0; i < ng; ++i) {
            const tf_group rg = a.route_groups[i];
            const uint8_t* blob = a.pool_base + (uint64_t)rg.expert * a.expert_stride;
            QmmGroup g{};
            for (int m = 0; m < nmat; ++m) {
                g.S[m] = reinterpret_cast<const uint16_t*>(blob + a.s_off[m]);
                g.B[m] = reinterpret_cast<const uint16_t*>(blob + a.b_off[m]);
            }
            g.expert = rg.expert; g.row_start = rg.pair_start; g.count = rg.pair_count; g.tile_start = tiles;
            a.groups[i] = g;
            tiles += (rg.pair_count + kQmmTokMax - 1) / kQmmTokMax;
        }
    }
    a.totals[0] = ng;
    a.totals[1] = tiles;
}

// Shared-memory plan (offsets from a 1024-byte aligned base).
template <int NMAT>
struct QmmSmem {
    static constexpr uint32_t kRawMat = kQmmRows * (kQmmK / 2);              // 8 KB: 128 rows x 64 packed bytes
    static constexpr uint32_t kRawStage = NMAT * kRawMat;
    static constexpr uint32_t kOffRaw = 0;
    static constexpr uint32_t kOffB = kOffRaw + kQmmRawStages * kRawStage;   // 32 slots x 2 KB
    static constexpr uint32_t kOffScales = kOffB + kQmmBSlots * kQmmBoxRows * 128;
    // scale and bias planes of a tile: 128 rows x (K / 64) bf16, two buffers, sized at launch
    __host__ __device__ static uint32_t plane_bytes(uint32_t k) { return ((kQmmRows * (k / kGroup) * 2u) + 15u) & ~15u; }
    __host__ __device__ static uint32_t scale_buf_bytes(uint32_t k) { return NMAT * 2 * plane_bytes(k); }
    __host__ __device__ static uint32_t off_bars(uint32_t k) { return kOffScales + 2 * scale_buf_bytes(k); }
    __host__ __device__ static uint32_t total(uint32_t k) { return off_bars(k) + 1024 /* barriers */ + 1024 /* alignment slack */; }
    static constexpr int kAStages = 256 / (NMAT * (kQmmK / 2));              // TMEM ring of dequantised stages: 2 or 4
};

// Eight packed codes (one 32-bit word) -> eight fp16 weights w = half(q * s + b).
// Fast form: a nibble moved to bits 4..7 of a half is the subnormal q * 2^-20, so one HFMA2 with s * 2^20
// gives fma(q, s, b) rounded once (tensorops.metal:60-75 stores half(fma(q, s, b))); s * 2^20 is exact in
// fp16 (s is a bf16) while |s| < 2^-5. Larger scales take the two-step form (1024 + q) - 1024.
// Output order: PERMUTED (k0,k4,k1,k5,k2,k6,k3,k7), otherwise natural.
template <bool NATURAL_K>
__device__ __forceinline__ uint4 order8(__half2 h0, __half2 h1, __half2 h2, __half2 h3) {
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
template <bool NATURAL_K>
__device__ __forceinline__ uint4 dequant8_fast(uint32_t w, __half2 s_fast, __half2 b) {
    uint32_t t0 = (w << 4) & 0x00F000F0u, t1 = w & 0x00F000F0u, t2 = (w >> 4) & 0x00F000F0u, t3 = (w >> 8) & 0x00F000F0u;
    return order8<NATURAL_K>(__hfma2(*reinterpret_cast<__half2*>(&t0), s_fast, b),      // (k0, k4)
                             __hfma2(*reinterpret_cast<__half2*>(&t1), s_fast, b),      // (k1, k5)
                             __hfma2(*reinterpret_cast<__half2*>(&t2), s_fast, b),      // (k2, k6)
                             __hfma2(*reinterpret_cast<__half2*>(&t3), s_fast, b));     // (k3, k7)
}
template <bool NATURAL_K>
__device__ __forceinline__ uint4 dequant8_wide(uint32_t w, __half2 s, __half2 b) {
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    uint32_t t0 = (w & 0x000F000Fu) | 0x64006400u, t1 = ((w >> 4) & 0x000F000Fu) | 0x64006400u;
    uint32_t t2 = ((w >> 8) & 0x000F000Fu) | 0x64006400u, t3 = ((w >> 12) & 0x000F000Fu) | 0x64006400u;
    return order8<NATURAL_K>(__hfma2(__hsub2(*reinterpret_cast<__half2*>(&t0), k1024), s, b),
                             __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t1), k1024), s, b),
                             __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t2), k1024), s, b),
                             __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t3), k1024), s, b));
}

// Position of column k within its eight-column block in the PERMUTED order.
__device__ __forceinline__ uint32_t permuted_col(uint32_t k) { return (k & ~7u) | ((k & 3u) << 1) | ((k >> 2) & 1u); }

// Accumulator placement in TMEM columns 0..255, two buffers of 128. A tile whose accumulators fit one buffer
// (one matrix, or two matrices of at most 64 tokens) takes the buffer used less often so far, so consecutive
// tiles alternate and the epilogue of one overlaps the MMAs of the next; a two-matrix tile of more than 64
// tokens takes both. The MMA issuer and the epilogue warps replay the same sequence, so they agree.
struct AccPlan {
    uint32_t uses0 = 0u, uses1 = 0u;
    bool both = false;
    uint32_t buf = 0, col0 = 0, mat_stride = 0;
    template <int NMAT>
    __device__ __forceinline__ void next(uint32_t n_mma) {
        both = NMAT == 2 && n_mma > 64u;
        buf = both ? 0u : (uses0 <= uses1 ? 0u : 1u);
        col0 = buf * 128u;
        mat_stride = both ? 128u : 64u;
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
qmm_tcgen05_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap x_map_big,
                   const __grid_constant__ CUtensorMap w_map0,
                   const __grid_constant__ CUtensorMap w_map1, const QmmArgs args) {
    extern __shared__ uint8_t smem_raw[];
    using L = QmmSmem<NMAT>;
    constexpr int kAStages = L::kAStages;
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                      // swizzle atoms need 1024-byte alignment
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t plane_bytes = L::plane_bytes(args.k);
    const uint32_t scale_buf = L::scale_buf_bytes(args.k);
    const uint32_t bars = base + L::off_bars(args.k);
    // barrier map (8 bytes each)
    auto bar_full_raw = [&](uint32_t s) { return bars + s * 8; };                            // 8: TMA tx
    auto bar_empty_raw = [&](uint32_t s) { return bars + (8 + s) * 8; };                     // 8: dequant warps
    auto bar_full_b = [&](uint32_t s) { return bars + (16 + s) * 8; };                       // 16: TMA tx
    auto bar_empty_b = [&](uint32_t s) { return bars + (32 + s) * 8; };                      // 16: tcgen05.commit
    auto bar_full_a = [&](uint32_t s) { return bars + (48 + s) * 8; };                       // 8: dequant warps
    auto bar_empty_a = [&](uint32_t s) { return bars + (56 + s) * 8; };                      // 8: tcgen05.commit
    auto bar_full_sc = [&](uint32_t b) { return bars + (64 + b) * 8; };                      // 2: TMA tx
    auto bar_empty_sc = [&](uint32_t b) { return bars + (66 + b) * 8; };                     // 2: dequant warps
    auto bar_acc_full = [&](uint32_t b) { return bars + (68 + b) * 8; };                     // 2: tcgen05.commit
    auto bar_acc_empty = [&](uint32_t b) { return bars + (70 + b) * 8; };                    // 2: epilogue warps
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + L::off_bars(args.k) + 72 * 8);
    volatile uint32_t* bslots_slot = tmem_slot + 1;

    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t groups_per_row = args.k / kGroup;
    const uint32_t ksteps = (groups_per_row + 1) / 2;             // an odd last group is padded with zero columns
    const uint32_t wrow_tiles = (args.rows + kQmmRows - 1) / kQmmRows;
    const uint32_t ngroups = args.totals[0];
    const uint32_t total_tiles = args.totals[1] * wrow_tiles;

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
    auto tile_tokens = [&](uint32_t count, uint32_t tt) {
        const uint32_t left = count - tt * kQmmTokMax;
        return left < (uint32_t)kQmmTokMax ? left : (uint32_t)kQmmTokMax;
    };

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < 8; ++s) {
            q_mbar_init(bar_full_raw(s), 1);
            q_mbar_init(bar_empty_raw(s), kQmmDequantWarps);
            q_mbar_init(bar_full_a(s), kQmmDequantWarps);
            q_mbar_init(bar_empty_a(s), 1);
        }
        for (uint32_t s = 0; s < 16; ++s) { q_mbar_init(bar_full_b(s), 1); q_mbar_init(bar_empty_b(s), 1); }
        for (uint32_t b = 0; b < 2; ++b) {
            q_mbar_init(bar_full_sc(b), 1);
            q_mbar_init(bar_empty_sc(b), kQmmDequantWarps);
            q_mbar_init(bar_acc_full(b), 1);
            q_mbar_init(bar_acc_empty(b), kQmmEpilogueWarps);
        }
        q_fence_async_smem();
        // Activation slots per step, fixed for this CTA: the largest tile it will meet, rounded up to 1, 2, 4 or 8
        // boxes of 16 rows, so that a step's rows are contiguous and the ring never has to be re-partitioned.
        uint32_t max_tok = 1;
        for (uint32_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            uint32_t gi, tt, wt;
            locate(tile, gi, tt, wt);
            const uint32_t n = tile_tokens(args.groups[gi].count, tt);
            max_tok = n > max_tok ? n : max_tok;
        }
        const uint32_t boxes = (max_tok + kQmmBoxRows - 1) / kQmmBoxRows;
        *bslots_slot = boxes <= 1 ? 1u : boxes <= 2 ? 2u : boxes <= 4 ? 4u : 8u;
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
    const uint32_t b_slots = *bslots_slot;                            // 16-row boxes per 64-column half of an activation stage
    const uint32_t b_stages = kQmmBSlots / (2 * b_slots);             // 16, 8, 4 or 2
    const uint32_t b_half_bytes = b_slots * kQmmBoxRows * 128;        // one 64-column half of a stage
    const uint32_t a_ring = tmem_base + kQmmAccCols;

    uint32_t fail = 0;
    uint32_t it = 0;         // running k-step index over all of this CTA's tiles (ring positions)

    if (warp == 0) {
        // ===================== copy issuer: packed codes, activation boxes, scale planes =====================
        uint32_t tile_idx = 0, sb = 0, ub = 0;                     // activation ring position and lap
        auto issue_scales = [&](uint32_t tile, uint32_t idx) -> bool {
            const uint32_t buf = idx & 1, n = idx >> 1;
            if (n > 0 && !q_mbar_wait(bar_empty_sc(buf), (n - 1) & 1)) return false;
            if (lane == 0) {
                uint32_t gi, tt, wt;
                locate(tile, gi, tt, wt);
                const uint32_t row0 = wt * kQmmRows;
                const uint32_t nrows = args.rows - row0 < (uint32_t)kQmmRows ? args.rows - row0 : (uint32_t)kQmmRows;
                const uint32_t bytes = nrows * groups_per_row * 2;        // a multiple of 16: rows are a multiple of 8
                q_mbar_expect_tx(bar_full_sc(buf), NMAT * 2 * bytes);
                for (int m = 0; m < NMAT; ++m) {
                    const uint32_t dst = base + L::kOffScales + buf * scale_buf + m * 2 * plane_bytes;
                    q_bulk_g2s(dst, args.groups[gi].S[m] + (size_t)row0 * groups_per_row, bytes, bar_full_sc(buf));
                    q_bulk_g2s(dst + plane_bytes, args.groups[gi].B[m] + (size_t)row0 * groups_per_row, bytes, bar_full_sc(buf));
                }
            }
            __syncwarp();
            return true;
        };
        if (blockIdx.x < total_tiles && !issue_scales(blockIdx.x, 0)) fail = kErrQmmTimeout | 6;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && !fail; tile += gridDim.x, ++tile_idx) {
            uint32_t gi, tt, wt;
            locate(tile, gi, tt, wt);
            const uint32_t expert = args.groups[gi].expert;
            const uint32_t row0 = args.groups[gi].row_start + tt * kQmmTokMax;
            const uint32_t boxes = (tile_tokens(args.groups[gi].count, tt) + kQmmBoxRows - 1) / kQmmBoxRows;
            // the next tile's scale planes go out once the dequantisers are certainly done with the tile before
            // this one (they have consumed this tile's first step when its ring slot comes round again)
            const uint32_t scale_step = ksteps > (uint32_t)kQmmRawStages ? (uint32_t)kQmmRawStages : ksteps - 1;
            for (uint32_t ks = 0; ks < ksteps; ++ks, ++it) {
                const uint32_t sr = it % kQmmRawStages, ur = it / kQmmRawStages;
                if (ur > 0 && !q_mbar_wait(bar_empty_raw(sr), (ur - 1) & 1)) { fail = kErrQmmTimeout | 1; break; }
                const bool leader = elect_one();
                if (leader) {
                    q_mbar_expect_tx(bar_full_raw(sr), L::kRawStage);
                    tma_load_3d(base + L::kOffRaw + sr * L::kRawStage, &w_map0, (int)(ks * (kQmmK / 2)), (int)(wt * kQmmRows), (int)expert, bar_full_raw(sr));
                    if (NMAT == 2)
                        tma_load_3d(base + L::kOffRaw + sr * L::kRawStage + L::kRawMat, &w_map1, (int)(ks * (kQmmK / 2)), (int)(wt * kQmmRows), (int)expert, bar_full_raw(sr));
                }
                if (ub > 0 && !q_mbar_wait(bar_empty_b(sb), (ub - 1) & 1)) { fail = kErrQmmTimeout | 7; break; }
                if (leader) {
                    if (boxes > 4) {                              // more than 64 tokens: one 128-row box per half
                        q_mbar_expect_tx(bar_full_b(sb), 2 * kQmmTokMax * 128);
                        for (uint32_t h = 0; h < 2; ++h)
                            tma_load_2d(base + L::kOffB + sb * 2 * b_half_bytes + h * b_half_bytes, &x_map_big,
                                        (int)(ks * kQmmK + h * 64), (int)row0, bar_full_b(sb));
                    } else {
                        q_mbar_expect_tx(bar_full_b(sb), 2 * boxes * kQmmBoxRows * 128);
                        for (uint32_t h = 0; h < 2; ++h)          // columns past K (odd group count) read as zero
                            for (uint32_t b = 0; b < boxes; ++b)
                                tma_load_2d(base + L::kOffB + sb * 2 * b_half_bytes + h * b_half_bytes + b * kQmmBoxRows * 128, &x_map,
                                            (int)(ks * kQmmK + h * 64), (int)(row0 + b * kQmmBoxRows), bar_full_b(sb));
                    }
                }
                __syncwarp();
                if (++sb == b_stages) { sb = 0; ++ub; }
                if (ks == scale_step && tile + gridDim.x < total_tiles && !issue_scales(tile + gridDim.x, tile_idx + 1)) { fail = kErrQmmTimeout | 6; break; }
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        AccPlan plan;
        uint32_t sb = 0, ub = 0;                                  // activation ring position and lap
        const uint64_t b_desc0 = umma_smem_desc(base + L::kOffB);
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
                const uint32_t sa = it % kAStages, ua = it / kAStages;
                if (!q_mbar_wait(bar_full_a(sa), ua & 1) || !q_mbar_wait(bar_full_b(sb), ub & 1)) { fail = kErrQmmTimeout | 3; break; }
                tc_fence_after();
                const bool leader = elect_one();
                const uint64_t b_desc = b_desc0 + (uint64_t)((sb * 2 * b_half_bytes) >> 4);
                const uint32_t a_stage = a_ring + sa * (NMAT * 64);
                const uint32_t nj = (2 * ks + 1 < groups_per_row) ? 8u : 4u;     // the padded half of an odd last step is skipped
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
#pragma unroll
                    for (int j = 0; j < kQmmK / 16; ++j) {        // 16 columns of K: 8 TMEM columns of A, 32 bytes of B
                        if ((uint32_t)j < nj && leader)
                            tc_mma_f16_ts(acc + m * plan.mat_stride, a_stage + m * 64 + j * 8,
                                          b_desc + (uint64_t)((j >> 2) * (b_half_bytes >> 4) + (j & 3) * 2), idesc, (ks > 0 || j > 0) ? 1u : 0u);
                    }
                }
                if (leader) {
                    tc_commit(bar_empty_a(sa));                   // both rings' stages are free once these MMAs have read them
                    tc_commit(bar_empty_b(sb));
                    if (ks + 1 == ksteps) {
                        if (plan.both || plan.buf == 0) tc_commit(bar_acc_full(0));
                        if (plan.both || plan.buf == 1) tc_commit(bar_acc_full(1));
                    }
                }
                __syncwarp();
                if (++sb == b_stages) { sb = 0; ++ub; }
            }
            plan.done();
        }
    } else if (warp >= kQmmFirstDequantWarp && warp < kQmmFirstEpilogueWarp) {
        // ===================== dequantisers: four threads per weight row =====================
        const uint32_t dw = warp - kQmmFirstDequantWarp;
        const uint32_t q = dw & 3, qc = dw >> 2;                 // TMEM lane quarter; quarter of the step's 128 columns
        const uint32_t r = q * kWarp + lane;                     // row within the tile = TMEM lane
        // packed codes of the row: 64 bytes whose 16-byte chunks sit at chunk ^ ((row / 2) % 4) (64-byte TMA swizzle)
        const uint32_t raw_off = r * 64 + ((qc ^ ((r >> 1) & 3u)) << 4);
        const uint32_t sc_off = r * groups_per_row * 2;
        const uint32_t a_lane = a_ring + ((q * kWarp) << 16) + qc * 16;
        uint32_t tile_idx = 0;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && !fail; tile += gridDim.x, ++tile_idx) {
            const uint32_t buf = tile_idx & 1;
            if (!q_mbar_wait(bar_full_sc(buf), (tile_idx >> 1) & 1)) { fail = kErrQmmTimeout | 8; break; }
            const uint32_t sc_base = base + L::kOffScales + buf * scale_buf + sc_off;
            for (uint32_t ks = 0; ks < ksteps; ++ks, ++it) {
                const uint32_t sr = it % kQmmRawStages, ur = it / kQmmRawStages;
                const uint32_t sa = it % kAStages, ua = it / kAStages;
                const uint32_t grp_idx = 2 * ks + (qc >> 1);      // this thread's 32 columns lie in one quantisation group
                const bool real = grp_idx < groups_per_row;      // the padded group of an odd last step dequantises to zero
                if (!q_mbar_wait(bar_full_raw(sr), ur & 1)) { fail = kErrQmmTimeout | 4; break; }
                uint4 codes[NMAT];
                float sf[NMAT], bf[NMAT];
                bool fast = true;
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                    codes[m] = q_lds128(base + L::kOffRaw + sr * L::kRawStage + m * L::kRawMat + raw_off);
                    sf[m] = real ? bf16_bits_to_float((uint16_t)q_lds16(sc_base + m * 2 * plane_bytes + grp_idx * 2)) : 0.0f;
                    bf[m] = real ? bf16_bits_to_float((uint16_t)q_lds16(sc_base + m * 2 * plane_bytes + plane_bytes + grp_idx * 2)) : 0.0f;
                    fast = fast && fabsf(sf[m]) < 0.03125f;
                }
                uint4 out[NMAT][4];
                if (__all_sync(kFullMask, fast)) {                // one branch per warp and step, both arms straight-line
#pragma unroll
                    for (int m = 0; m < NMAT; ++m) {
                        const __half2 s_fast = __float2half2_rn(sf[m] * 1048576.0f), b2 = __float2half2_rn(bf[m]);
                        out[m][0] = dequant8_fast<NATURAL_K>(codes[m].x, s_fast, b2);
                        out[m][1] = dequant8_fast<NATURAL_K>(codes[m].y, s_fast, b2);
                        out[m][2] = dequant8_fast<NATURAL_K>(codes[m].z, s_fast, b2);
                        out[m][3] = dequant8_fast<NATURAL_K>(codes[m].w, s_fast, b2);
                    }
                } else {
#pragma unroll
                    for (int m = 0; m < NMAT; ++m) {
                        const __half2 s2 = __float2half2_rn(sf[m]), b2 = __float2half2_rn(bf[m]);
                        out[m][0] = dequant8_wide<NATURAL_K>(codes[m].x, s2, b2);
                        out[m][1] = dequant8_wide<NATURAL_K>(codes[m].y, s2, b2);
                        out[m][2] = dequant8_wide<NATURAL_K>(codes[m].z, s2, b2);
                        out[m][3] = dequant8_wide<NATURAL_K>(codes[m].w, s2, b2);
                    }
                }
                __syncwarp();
                if (lane == 0) q_mbar_arrive(bar_empty_raw(sr));  // the codes are in registers
                if (ua > 0 && !q_mbar_wait(bar_empty_a(sa), (ua - 1) & 1)) { fail = kErrQmmTimeout | 5; break; }
                tc_fence_after();
#pragma unroll
                for (int m = 0; m < NMAT; ++m) tc_st16(a_lane + sa * (NMAT * 64) + m * 64, out[m][0], out[m][1], out[m][2], out[m][3]);
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) q_mbar_arrive(bar_full_a(sa));
            }
            __syncwarp();
            if (lane == 0) q_mbar_arrive(bar_empty_sc(buf));      // done with this tile's scale planes
        }
    } else if (warp >= kQmmFirstEpilogueWarp) {
        // ===================== epilogue: TMEM -> registers -> global =====================
        const uint32_t q = warp & 3;                              // TMEM lane quarter this warp may read
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
                if (plan.takes(b) && !q_mbar_wait(bar_acc_full(b), plan.uses(b) & 1)) fail = kErrQmmTimeout | 9;
            }
            if (fail) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + ((q * kWarp) << 16) + plan.col0;
            uint16_t* out_row = args.out + (size_t)(grp.row_start + tok0) * args.out_stride + out_col;
            for (uint32_t c0 = 0; c0 < ntok; c0 += 16) {
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

// fp16 matrix [rows, k] with a row stride: box = 64 columns x box_rows rows, 128-byte swizzle, zero fill outside.
static tf_status make_x_map(tf_context* ctx, CUtensorMap* map, const void* x, uint64_t rows, uint32_t k, uint32_t stride_elems,
                            uint32_t box_rows, const char* name) {
    EncodeTiledFn fn = encode_tiled_fn();
    TF_REQUIRE(ctx, fn != nullptr, TF_ERR_UNSUPPORTED, "%s: cuTensorMapEncodeTiled is not available in this driver", name);
    const cuuint64_t dims[2] = {k, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)stride_elems * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TF_REQUIRE(ctx, r == CUDA_SUCCESS, TF_ERR_CUDA, "%s: cuTensorMapEncodeTiled(activations) failed (%d)", name, (int)r);
    return TF_OK;
}

// Packed int4 weights as bytes [experts, rows, k / 2]: box = 64 bytes x 128 rows x 1 expert, 64-byte swizzle
// (the 16-byte chunks of a row are permuted by (row / 2) % 4, which makes the row-per-lane LDS.128 conflict
// free); rows past the matrix and bytes past the row read as zero.
static tf_status make_w_map(tf_context* ctx, CUtensorMap* map, const void* w, uint32_t rows, uint32_t k, uint64_t experts,
                            uint64_t expert_stride, const char* name) {
    EncodeTiledFn fn = encode_tiled_fn();
    TF_REQUIRE(ctx, fn != nullptr, TF_ERR_UNSUPPORTED, "%s: cuTensorMapEncodeTiled is not available in this driver", name);
    const cuuint64_t dims[3] = {k / 2, rows, experts};
    const cuuint64_t strides[2] = {(cuuint64_t)(k / 2), expert_stride};
    const cuuint32_t box[3] = {(cuuint32_t)(kQmmK / 2), (cuuint32_t)kQmmRows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(w), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TF_REQUIRE(ctx, r == CUDA_SUCCESS, TF_ERR_CUDA, "%s: cuTensorMapEncodeTiled(weights) failed (%d)", name, (int)r);
    return TF_OK;
}

// W[m]: base of matrix m's packed plane for expert 0 (dense: the matrix itself).
template <int NMAT, bool NATURAL_K>
static tf_status launch_qmm(tf_context* ctx, void* stream, QmmArgs& a, const void* x, uint64_t x_rows, uint32_t x_stride,
                            const uint8_t* const* W, uint64_t experts, uint64_t expert_stride, bool dense, const char* name) {
    TF_REQUIRE(ctx, a.k % kGroup == 0 && a.k >= (uint32_t)kGroup, TF_ERR_INVALID_ARGUMENT, "%s: K must be a positive multiple of 64", name);
    TF_REQUIRE(ctx, a.rows % 8 == 0 && a.rows > 0, TF_ERR_INVALID_ARGUMENT, "%s: the weight rows must be a positive multiple of 8", name);
    TF_REQUIRE(ctx, aligned(x, 16) && (x_stride * 2) % 16 == 0, TF_ERR_ALIGNMENT, "%s: activation rows must be 16-byte aligned", name);
    TF_REQUIRE(ctx, ctx->qmm_groups != nullptr, TF_ERR_OUT_OF_MEMORY, "%s: context scratch missing", name);
    const uint32_t smem = QmmSmem<NMAT>::total(a.k);
    TF_REQUIRE(ctx, smem <= 227u * 1024u, TF_ERR_UNSUPPORTED, "%s: K=%u needs %u bytes of shared memory for the scale planes", name, a.k, smem);
    CUtensorMap xmap, xmap_big, wmap[2];
    if (tf_status s = make_x_map(ctx, &xmap, x, x_rows, a.k, x_stride, kQmmBoxRows, name)) return s;
    if (tf_status s = make_x_map(ctx, &xmap_big, x, x_rows, a.k, x_stride, kQmmTokMax, name)) return s;
    for (int m = 0; m < 2; ++m)
        if (tf_status s = make_w_map(ctx, &wmap[m], W[m < NMAT ? m : 0], a.rows, a.k, experts, dense ? (uint64_t)a.rows * (a.k / 2) : expert_stride, name)) return s;
    a.groups = static_cast<QmmGroup*>(ctx->qmm_groups) + (dense ? TF_MAX_ROUTER_EXPERTS + 1 : 0);
    a.totals = ctx->qmm_totals + (dense ? 2 : 0);
    a.error = ctx->device_error;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    qmm_prepare_kernel<<<1, 32, 0, st>>>(a, NMAT, dense ? 1 : 0);
    if (tf_status s = check_launch(ctx, "qmm_prepare")) return s;
    auto kern = qmm_tcgen05_kernel<NMAT, NATURAL_K>;
    static DeviceSmemCache configured;
    if (tf_status s = ensure_dynamic_smem(ctx, kern, configured, smem)) return s;
    kern<<<ctx->sm_count, kQmmThreads, smem, st>>>(xmap, xmap_big, wmap[0], wmap[1], a);
    return check_launch(ctx, name);
}

tf_status launch_qmm_generic(tf_context* ctx, void* stream, const uint8_t* W, const uint16_t* S, const uint16_t* B,
                             const uint16_t* X, uint16_t* Y, uint32_t m, uint32_t n, uint32_t k, const char* name);   // qmm_generic.cu

}  // namespace tf

extern "C" {

tf_status tf_grouped_moe_tensorcore(tf_context* ctx, void* stream, const void* x_sorted, uint32_t x_rows,
                                    const void* pool_layer_base, uint64_t expert_stride, uint32_t num_experts,
                                    const tf_expert_offsets* offsets, const tf_device_routes* routes,
                                    void* acts_scratch, void* out_rows, uint32_t d, uint32_t f) {
    const char* name = "tf_grouped_moe_tensorcore";
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, x_sorted && pool_layer_base && offsets && routes && acts_scratch && out_rows, TF_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    TF_REQUIRE(ctx, d % 64 == 0 && f % 64 == 0 && d > 0 && f > 0, TF_ERR_INVALID_ARGUMENT, "%s: D and F must be positive multiples of 64", name);
    TF_REQUIRE(ctx, num_experts > 0 && num_experts <= TF_MAX_ROUTER_EXPERTS, TF_ERR_INVALID_ARGUMENT, "%s: numExperts must be in 1...256", name);
    const uint32_t all[9] = {offsets->gate_w_off, offsets->gate_s_off, offsets->gate_b_off, offsets->up_w_off, offsets->up_s_off,
                             offsets->up_b_off, offsets->down_w_off, offsets->down_s_off, offsets->down_b_off};
    for (uint32_t v : all) TF_REQUIRE(ctx, v % 16 == 0, TF_ERR_ALIGNMENT, "%s: blob sub-tensor offset %u is not a multiple of 16 bytes", name, v);
    TF_REQUIRE(ctx, tf::aligned(pool_layer_base, 16) && expert_stride % 16 == 0, TF_ERR_ALIGNMENT, "%s: pool must be 16-byte aligned", name);
    if (x_rows == 0) return TF_OK;
    const uint8_t* pool = static_cast<const uint8_t*>(pool_layer_base);
    tf::QmmArgs a{};
    a.pool_base = pool; a.expert_stride = expert_stride;
    a.s_off[0] = offsets->gate_s_off; a.b_off[0] = offsets->gate_b_off;
    a.s_off[1] = offsets->up_s_off;   a.b_off[1] = offsets->up_b_off;
    a.route_groups = routes->groups; a.route_counters = routes->counters;
    a.rows = f; a.k = d; a.out = static_cast<uint16_t*>(acts_scratch); a.out_stride = f; a.round_gate_up = 0;
    const uint8_t* w_gu[2] = {pool + offsets->gate_w_off, pool + offsets->up_w_off};
    if (tf_status s = tf::launch_qmm<2, false>(ctx, stream, a, x_sorted, x_rows, d, w_gu, num_experts, expert_stride, false,
                                                "tf_grouped_moe_tensorcore(gate/up)")) return s;
    tf::QmmArgs b{};
    b.pool_base = pool; b.expert_stride = expert_stride;
    b.s_off[0] = offsets->down_s_off; b.b_off[0] = offsets->down_b_off;
    b.route_groups = routes->groups; b.route_counters = routes->counters;
    b.rows = d; b.k = f; b.out = static_cast<uint16_t*>(out_rows); b.out_stride = d;
    const uint8_t* w_dn[2] = {pool + offsets->down_w_off, pool + offsets->down_w_off};
    return tf::launch_qmm<1, false>(ctx, stream, b, acts_scratch, x_rows, f, w_dn, num_experts, expert_stride, false,
                                    "tf_grouped_moe_tensorcore(down)");
}

tf_status tf_int4_qmm_with_path(tf_context* ctx, void* stream, const void* weights, uint64_t weights_off, const void* scales,
                                uint64_t scales_off, const void* biases, uint64_t biases_off, const void* x, uint64_t x_off,
                                void* y, uint64_t y_off, uint32_t m, uint32_t n, uint32_t k, tf_qmm_path* path_out) {
    const char* name = "tf_int4_qmm";
    if (path_out) *path_out = TF_QMM_PATH_UNAVAILABLE;
    TF_REQUIRE(ctx, ctx != nullptr, TF_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", name);
    TF_REQUIRE(ctx, weights && scales && biases && x && y, TF_ERR_INVALID_ARGUMENT, "%s: NULL buffer", name);
    const uint8_t* wp = tf::byte_ptr(weights, weights_off);
    const uint8_t* sp = tf::byte_ptr(scales, scales_off);
    const uint8_t* bp = tf::byte_ptr(biases, biases_off);
    const uint8_t* xp = tf::byte_ptr(x, x_off);
    uint8_t* yp = tf::byte_ptr(y, y_off);
    // the reference's guard (MPPPrefillInt4QMM.swift:43-55): positive sizes, K % 64 == 0, even 16-bit plane offsets
    const bool supported = m > 0 && n > 0 && k > 0 && k % 64 == 0 && tf::aligned(sp, 2) && tf::aligned(bp, 2) &&
                           tf::aligned(xp, 2) && tf::aligned(yp, 2);
    if (!supported) {
        if (path_out) return TF_OK;         // the reference reports .unavailable and the caller falls back
        TF_REQUIRE(ctx, m == 0 || n == 0 || (k % 64 == 0 && k > 0), TF_ERR_INVALID_ARGUMENT, "%s: K must be a positive multiple of 64", name);
        if (m == 0 || n == 0) return TF_OK;
        return tf::fail(ctx, TF_ERR_ALIGNMENT, "%s: scale, bias, x and y offsets must be even", name);
    }
    const bool tensor = n % 8 == 0 && tf::aligned(wp, 16) && tf::aligned(sp, 16) && tf::aligned(bp, 16) && tf::aligned(xp, 16);
    if (!tensor) {
        // odd row counts or planes off the 16-byte grid: the CUDA-core kernel takes any byte offset
        tf_status s = tf::launch_qmm_generic(ctx, stream, wp, reinterpret_cast<const uint16_t*>(sp), reinterpret_cast<const uint16_t*>(bp),
                                             reinterpret_cast<const uint16_t*>(xp), reinterpret_cast<uint16_t*>(yp), m, n, k, name);
        if (!s && path_out) *path_out = TF_QMM_PATH_CUDA_CORES;
        return s;
    }
    tf::QmmArgs a{};
    const uint8_t* w[2] = {wp, wp};
    a.dense_S[0] = reinterpret_cast<const uint16_t*>(sp);
    a.dense_B[0] = reinterpret_cast<const uint16_t*>(bp);
    a.dense_tokens = m; a.rows = n; a.k = k;
    a.out = reinterpret_cast<uint16_t*>(yp); a.out_stride = n;
    tf_status s = tf::launch_qmm<1, true>(ctx, stream, a, xp, m, k, w, 1, 0, true, name);
    if (!s && path_out) *path_out = TF_QMM_PATH_TENSORCORE;
    return s;
}

tf_status tf_int4_qmm(tf_context* ctx, void* stream, const void* weights, uint64_t weights_off, const void* scales,
                      uint64_t scales_off, const void* biases, uint64_t biases_off, const void* x, uint64_t x_off,
                      void* y, uint64_t y_off, uint32_t m, uint32_t n, uint32_t k) {
    return tf_int4_qmm_with_path(ctx, stream, weights, weights_off, scales, scales_off, biases, biases_off, x, x_off, y, y_off,
                                 m, n, k, nullptr);
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
        TF_REQUIRE(ctx, tf::aligned(W[i], 16) && tf::aligned(S[i], 16) && tf::aligned(B[i], 16), TF_ERR_ALIGNMENT, "%s: planes must be 16-byte aligned", name);
    }
    tf::QmmArgs a{};
    a.dense_S[0] = S[0]; a.dense_B[0] = B[0];
    a.dense_S[1] = S[1]; a.dense_B[1] = B[1];
    a.dense_tokens = rows; a.rows = fs; a.k = d; a.out = static_cast<uint16_t*>(scratch_act); a.out_stride = fs; a.round_gate_up = 1;
    const uint8_t* w_gu[2] = {W[0], W[1]};
    if (tf_status s = tf::launch_qmm<2, true>(ctx, stream, a, x, rows, x_stride_elements, w_gu, 1, 0, true,
                                               "tf_shared_expert_int4_tensorcore(gate/up)")) return s;
    tf::QmmArgs b{};
    b.dense_S[0] = S[2]; b.dense_B[0] = B[2];
    b.dense_tokens = rows; b.rows = d; b.k = fs; b.out = static_cast<uint16_t*>(y); b.out_stride = y_stride_elements;
    const uint8_t* w_dn[2] = {W[2], W[2]};
    return tf::launch_qmm<1, true>(ctx, stream, b, scratch_act, rows, fs, w_dn, 1, 0, true, "tf_shared_expert_int4_tensorcore(down)");
}

}  // extern "C"
