// One-token decode step of the whole layer stack in ONE launch.
//
// At one token a layer moves 37 MB of weights (5.7 us at HBM speed) through seven dependent kernels whose launch
// and drain latencies add up to several times that. Here one persistent grid (one CTA per SM, all co-resident)
// walks all layers; the phases of a layer are separated by grid barriers instead of kernel boundaries:
//
//   P0  every CTA: x = half(rmsnorm(h) * w) (the arithmetic and reduction tree of residual_rmsnorm_kernel), staged
//       in shared memory as MMA B-fragments
//   P1  router logits (canonical fp32 order of router.cuh, one expert row per CTA) and the shared expert's
//       gate/up rows, split evenly over the CTAs                                              -> barrier 1
//   P2  every CTA selects the top-k from the logits (same warp routine as the router kernels), then the routed
//       experts' gate/up rows, K * F row pairs split evenly over the CTAs                      -> barrier 2
//   P3  down projections of the K routed experts and of the shared expert for the CTA's slice of output rows,
//       the weighted combine in rank order (Metal/MoE/moe.metal:473-480) and the residual add  -> barrier 3
//
// Weights never wait for a warp: a loader warp streams the CTA's rows of P1, P2, P3, then the next layer's P1, ...
// through a ring of shared-memory stages (16 rows each, one cp.async.bulk per row, completion on an mbarrier) as
// far ahead as the ring and the router allow (the rows of P2 and P3 are known once the layer's top-k is), so HBM
// keeps streaming across the grid barriers. Sixteen compute warps consume the stages in items of 16 rows x up to 4
// column groups with the mma.sync GEMV building block of mma_gemv.cuh; partial sums meet in shared memory and are
// added in a fixed order, so results do not depend on timing. Scale and bias rows of a phase are staged by the
// compute warps while the first stage is in flight.
//
// Rounding points are those of the per-kernel path: routed act = half(gelu(g) * u) with g, u in fp32
// (moe.metal:368); shared act = half(gelu(half(g)) * half(u)), shared y = half(down . act)
// (Kernels/MoE/SharedExpertInt4.swift:62-93); y = half(shared_y + sum_r w_r * partial_r); h = half(h + y).
//
// Every wait is bounded (grid barriers, stage barriers, the router hand-over to the loader): a wait that runs out
// records a code in the context's device error word, after which nothing in the CTA waits any more and the kernel
// runs to its end with meaningless results; tf_device_status reports it.
#include <algorithm>

#include "async_copy.cuh"
#include "block.cuh"
#include "mma_gemv.cuh"
#include "router.cuh"

namespace tf {

constexpr int kDsComputeWarps = 16;
constexpr int kDsComputeThreads = kDsComputeWarps * kWarp;
constexpr int kDsThreads = kDsComputeThreads + kWarp;      // + the loader warp
constexpr uint32_t kDsStages = 6;                // ring depth
constexpr uint32_t kDsMaxItems = 128;            // items of one phase in one CTA
constexpr uint32_t kDsSpinLimit = 1u << 22;      // grid barrier polls, ~0.5 us each
constexpr uint32_t kErrGridBarrier = 0x7F000021u;
constexpr uint32_t kErrStageWait = 0x7F000022u;
constexpr uint32_t kErrLoaderWait = 0x7F000023u;
constexpr uint32_t kErrScaleWait = 0x7F000024u;
constexpr uint32_t kDsPairPad = 32;               // bytes of padding after every pair of gate/up rows in a ring stage
constexpr int kDsNormThreads = 128;              // threads that compute the sum of squares (as residual_rmsnorm_kernel)
constexpr int kDsNormSlices = 4;

struct DecodeLayer {
    const uint8_t* router_w; const uint16_t* router_s; const uint16_t* router_b;
    const uint16_t* eff; const uint16_t* pes; const float* logit_bias;
    const uint8_t* pool; uint64_t stride; tf_expert_offsets off;
    const uint8_t* sg_w; const uint16_t* sg_s; const uint16_t* sg_b;
    const uint8_t* su_w; const uint16_t* su_s; const uint16_t* su_b;
    const uint8_t* sd_w; const uint16_t* sd_s; const uint16_t* sd_b;
    const uint16_t* norm_w;
};

struct DecodeArgs {
    const DecodeLayer* layers;
    uint32_t n_layers, d, f, fs, E, K;
    float eps;
    uint16_t* hidden;        // [d] fp16, updated in place
    float* logits;           // [E]
    uint16_t* acts;          // [K * f]
    uint16_t* shared_act;    // [fs]
    uint32_t* out_idx;       // [K] router ids of the last layer (for inspection)
    uint16_t* out_w;         // [K]
    uint32_t* barrier;       // zero at launch
    uint32_t* error;
    unsigned long long* trace;   // optional: CTA 0 stamps the global timer at every phase boundary (8 per layer)
    uint32_t trace_capacity;
    uint32_t bulk_scales;        // gate/up scale rows by bulk copies (even row spaces, 16-byte aligned planes, ngd % 4 == 0)
};

// One item: 16 rows of a stage x up to 4 column groups of one matrix. Constant across layers.
struct DsItem {
    uint16_t stage_local;    // stage of the phase that holds the item's rows
    uint16_t stage_items;    // low byte: items that read that stage (the last one to finish hands the slot back); high byte: row stride / 16
    uint16_t tile;           // 16-row tile of the CTA's slice; bit 15: the stage pads every pair of rows (gate/up layout)
    uint16_t row_off;        // byte offset of the item's first group inside the stage (expert block + column)
    uint16_t group;          // first group in the B-fragment / group-sum arrays
    uint16_t scale_base;     // element offset of the source's scale rows inside the phase's scale plane
    uint16_t scale_stride;   // groups per scale row of the source
    uint16_t g0_ngr;         // first group within the source's row << 4 | groups in the item (1...4)
};

__host__ __device__ inline uint32_t ds_split(uint32_t total, uint32_t part, uint32_t parts) {
    return (uint32_t)(((uint64_t)total * part) / parts);
}
// Slices of the gate/up row spaces start on even rows (when the space is even), so that a slice's scale rows form
// 16-byte aligned runs that one bulk copy each can fetch.
__host__ __device__ inline uint32_t ds_split_rows(uint32_t total, uint32_t part, uint32_t parts) {
    return (total & 1u) ? ds_split(total, part, parts) : 2u * ds_split(total / 2u, part, parts);
}
__host__ __device__ inline uint32_t ds_max_rows(uint32_t total, uint32_t parts) {
    return (total & 1u) ? (total + parts - 1) / parts : 2u * ((total / 2u + parts - 1) / parts);
}
__host__ __device__ inline uint32_t ds_kparts(uint32_t ng) { return (ng + 3u) / 4u; }
__host__ __device__ inline uint32_t ds_ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

// Shared-memory layout (bytes from the start of dynamic shared memory).
struct DsSmem {
    uint32_t ring, row_stride, stage_bytes, sc1, sc1_plane, sc2, sc2_plane, sc3, sc3_plane, rows1, rows2, rows3,
        x16, xf, a16, frag_a, sum_a, frag_b, sum_b, wrow, partial, tabs, scores, sel_idx, sel_w, red, bars, cnt, total;
    __host__ __device__ DsSmem(uint32_t d, uint32_t f, uint32_t fs, uint32_t E, uint32_t K, uint32_t grid) {
        auto up = [](uint32_t v, uint32_t a) { return (v + a - 1) / a * a; };
        const uint32_t ngd = d / 64, ngf = f / 64, ngs = fs / 64, ngb = K * ngf + ngs;
        // A ring stage holds one of three layouts (a bulk copy has a fixed cost in the copy engine, so a stage is
        // filled with as few copies as the source layout allows):
        //   gate/up rows (P1, P2): 16 rows of d/2 bytes, two rows per copy, 32 bytes of padding per pair of rows
        //   routed down rows (P3): up to four experts x 16 rows of f/2 bytes, expert-major and dense, one copy per expert
        //   shared down rows (P3): 16 rows of fs/2 bytes, dense, one copy
        row_stride = d / 2;
        const uint32_t st_gu = 16 * (d / 2) + 8 * kDsPairPad, st_rd = (K < 4u ? K : 4u) * 16 * (f / 2), st_sd = 16 * (fs / 2);
        stage_bytes = up(st_gu > st_rd ? (st_gu > st_sd ? st_gu : st_sd) : (st_rd > st_sd ? st_rd : st_sd), 128);
        rows1 = ds_max_rows(fs, grid); rows2 = ds_max_rows(K * f, grid); rows3 = (d + grid - 1) / grid;
        // scale planes (elements): P1 / P2 hold [matrix][row][group], P3 holds [source][row][group]
        // (P3 rows are padded to a multiple of four groups so that four scales are one aligned 8-byte read)
        sc1_plane = up(2 * rows1 * ngd, 8); sc2_plane = up(2 * rows2 * ngd, 8);
        sc3_plane = up(rows3 * (K * up(ngf, 4) + up(ngs, 4)), 8);
        uint32_t o = 0;
        ring = o; o += kDsStages * stage_bytes;
        sc1 = o; o += sc1_plane * 4;                                // scale plane, then bias plane (16-bit elements)
        sc2 = o; o += sc2_plane * 4;
        sc3 = o; o += sc3_plane * 4;
        x16 = o; a16 = o; o += up(d * 2, 16);                       // a16 (P3) overlays x16 + xf (P0..P2)
        xf = o; o += up(d * 4, 16);
        if (o - a16 < up((K * f + fs) * 2, 16)) o = a16 + up((K * f + fs) * 2, 16);
        frag_a = o; o += ngd * 128;
        sum_a = o; o += up(ngd * 4, 16);
        frag_b = o; o += ngb * 128;
        sum_b = o; o += up(ngb * 4, 16);
        wrow = o; o += up(d, 16) + up(ngd * 2, 16) * 2;
        partial = o; o += kDsMaxItems * 64;
        tabs = o; o += 3 * kDsMaxItems * (uint32_t)sizeof(DsItem);
        scores = o; o += up(E * 4, 16);
        sel_idx = o; o += 32;
        sel_w = o; o += 16;
        red = o; o += 16;
        bars = o; o += (2 * kDsStages + 5) * 8 + 8;
        cnt = o; o += up(kDsStages * 4 + 4, 16);                    // per-slot item counters, then the dead flag
        total = o;
    }
};

// Per-CTA constants of the launch, kept in shared memory so that the phase functions (compiled as separate
// functions: each gets its own register allocation) read what they need instead of carrying it in registers.
struct DsCtx {
    uint32_t d, f, fs, E, K, ngd, ngf, ngs, kp_d, kp_f, kp_s, subs;
    uint32_t p1_lo, p1_hi, p2_lo, p2_hi, p3_lo, p3_hi, p1_tiles, p2_tiles, p3_tiles, p3_per_tile;
    uint32_t n_st1, n_st2, n_st3;                       // stages per phase
    uint32_t cta, grid, row_stride, stage_bytes;
    uint32_t rows1_cap, rows2_cap, rows3_cap, sc1_plane, sc2_plane, sc3_plane;   // scale rows per slice (capacity), plane sizes (elements)
    uint32_t ngf_pad, ngs_pad;                          // groups per staged P3 scale row (multiples of four)
    uint32_t bulk_scales;                               // the gate/up scale rows arrive by bulk copies of the loader warp
    uint32_t ring_addr, bars_addr, sc1_addr, sc2_addr;  // shared-window addresses
    uint8_t* ring; uint16_t* sc1; uint16_t* sc2; uint16_t* sc3; uint16_t* x16; float* xf; uint16_t* a16; uint32_t* frag_a; float* sum_a;
    uint32_t* frag_b; float* sum_b; uint8_t* wrow; float* partial; DsItem* tabs; float* scores; uint32_t* sel_idx;
    uint16_t* sel_w; float* red; uint32_t* cnt; volatile uint32_t* dead;
    uint16_t* hidden; float* logits; uint16_t* acts; uint16_t* shared_act; uint32_t* out_idx; uint16_t* out_w;
    uint32_t* error;
    unsigned long long* prof;        // optional: cycle counts of warp 0 of CTA 0 inside the item loop, 4 per phase
    float eps;
};

__device__ __forceinline__ uint32_t ds_bar_full(const DsCtx* c, uint32_t slot) { return c->bars_addr + slot * 8; }
__device__ __forceinline__ uint32_t ds_bar_empty(const DsCtx* c, uint32_t slot) { return c->bars_addr + (kDsStages + slot) * 8; }
__device__ __forceinline__ uint32_t ds_bar_routing(const DsCtx* c) { return c->bars_addr + 2 * kDsStages * 8; }
// scale rows of P1 (which = 0) and P2 (which = 1): filled by the loader, released by the compute warps
__device__ __forceinline__ uint32_t ds_bar_sc_full(const DsCtx* c, uint32_t which) { return c->bars_addr + (2 * kDsStages + 1 + which) * 8; }
__device__ __forceinline__ uint32_t ds_bar_sc_empty(const DsCtx* c, uint32_t which) { return c->bars_addr + (2 * kDsStages + 3 + which) * 8; }

// barrier of the compute warps only (the loader warp runs ahead on its own)
__device__ __forceinline__ void cta_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kDsComputeThreads) : "memory"); }

__device__ __forceinline__ void ds_fail(const DsCtx* c, uint32_t code) {
    atomicCAS(c->error, 0u, code);
    *c->dead = 1u;
}

// ---------------------------------------------------------------------------
// grid barrier (compute warps)
// ---------------------------------------------------------------------------
struct GridSync {
    uint32_t* counter; uint32_t target;
};

__device__ __forceinline__ void grid_sync(const DsCtx* c, GridSync& gs) {
    cta_sync();
    if (threadIdx.x == 0) {
        gs.target += gridDim.x;
        __threadfence();
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(gs.counter) : "memory");
        if (!*c->dead) {
            uint32_t spins = 0;
            for (;;) {
                uint32_t v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(gs.counter) : "memory");
                if ((int32_t)(v - gs.target) >= 0) break;
                if (++spins > kDsSpinLimit) { ds_fail(c, kErrGridBarrier); break; }
                if ((spins & 1023u) == 0u && *reinterpret_cast<volatile uint32_t*>(c->error) != 0u) { *c->dead = 1u; break; }
            }
        }
    }
    cta_sync();
}

// One warp brings [p, p + bytes) into L2.
__device__ __forceinline__ void prefetch_l2_warp(const void* p, uint32_t bytes, int lane) {
    const uintptr_t first = reinterpret_cast<uintptr_t>(p) & ~(uintptr_t)127;
    const uintptr_t last = reinterpret_cast<uintptr_t>(p) + bytes;
    for (uintptr_t a = first + (uintptr_t)lane * 128; a < last; a += (uintptr_t)kWarp * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
}

// ---------------------------------------------------------------------------
// loader warp
// ---------------------------------------------------------------------------
// Waits for the slot of stage q to be free and arms its barrier with the bytes about to land. Returns the slot's
// shared-window address, or 0 when the CTA has given up waiting.
__device__ __forceinline__ uint32_t ds_open_stage(const DsCtx* c, uint32_t q, uint32_t tx_bytes, int lane) {
    const uint32_t slot = q % kDsStages, use = q / kDsStages;
    if (*c->dead) return 0u;
    if (use > 0 && !mbar_wait(ds_bar_empty(c, slot), (use - 1) & 1)) {
        if (lane == 0) ds_fail(c, kErrLoaderWait);
        __syncwarp();
        return 0u;
    }
    if (lane == 0) {
        fence_proxy_async();                     // the slot was last read through the generic proxy
        mbar_arrive_expect_tx(ds_bar_full(c, slot), tx_bytes);
    }
    __syncwarp();
    return c->ring_addr + slot * c->stage_bytes;
}

// Scale and bias rows of a gate/up slice [lo, lo + rows) of a row space made of `spaces` consecutive matrices pairs
// (P1: the shared expert, one space of fs rows; P2: the K routed experts, f rows each): one bulk copy per run of rows
// inside one space, matrix and plane. Layout in shared memory: plane p at p * plane elements, matrix m at
// m * rows_cap * ngd, then [row][group].
struct ScaleSrc { const uint8_t* gate_s; const uint8_t* gate_b; const uint8_t* up_s; const uint8_t* up_b; };

template <typename SrcOf>
__device__ __forceinline__ void ds_load_scales(const DsCtx* c, uint32_t which, uint32_t layer, uint32_t lo, uint32_t rows, uint32_t space_rows,
                                               uint32_t rows_cap, uint32_t plane_elems, uint32_t dst_addr, int lane, SrcOf src_of) {
    if (rows == 0 || *c->dead) return;
    if (layer > 0 && !mbar_wait(ds_bar_sc_empty(c, which), (layer - 1) & 1)) {
        if (lane == 0) ds_fail(c, kErrLoaderWait);
        __syncwarp();
        return;
    }
    const uint32_t ngd = c->ngd;
    if (lane == 0) {
        fence_proxy_async();
        mbar_arrive_expect_tx(ds_bar_sc_full(c, which), rows * ngd * 2 * 4);
    }
    __syncwarp();
    const uint32_t first_space = lo / space_rows, last_space = (lo + rows - 1) / space_rows;
    const uint32_t n_runs = last_space - first_space + 1;
    for (uint32_t j = lane; j < n_runs * 4; j += kWarp) {
        const uint32_t run = j / 4, which_plane = j % 4;                 // gate s, gate b, up s, up b
        const uint32_t sp = first_space + run;
        const uint32_t r_lo = sp == first_space ? lo - sp * space_rows : 0u;
        const uint32_t r_hi = sp == last_space ? lo + rows - sp * space_rows : space_rows;
        const ScaleSrc src = src_of(sp);
        const uint8_t* plane = which_plane == 0 ? src.gate_s : which_plane == 1 ? src.gate_b : which_plane == 2 ? src.up_s : src.up_b;
        const uint32_t mat = which_plane / 2, pl = which_plane % 2;
        const uint32_t local_row = sp * space_rows + r_lo - lo;
        const uint32_t dst = dst_addr + (pl * plane_elems + mat * rows_cap * ngd + local_row * ngd) * 2;
        bulk_copy_g2s(dst, plane + (size_t)r_lo * ngd * 2, (r_hi - r_lo) * ngd * 2, ds_bar_sc_full(c, which));
    }
}

__device__ __noinline__ void ds_loader(const DsCtx* c, const DecodeLayer* layers, uint32_t n_layers) {
    const int lane = threadIdx.x % kWarp;
    const uint32_t d = c->d, f = c->f, fs = c->fs, K = c->K, RS = c->row_stride;
    uint32_t q = 0;
    for (uint32_t l = 0; l < n_layers; ++l) {
        const DecodeLayer* L = layers + l;
        // P1: shared gate/up rows and their scales (no dependency: runs ahead of the previous layer's barrier 3)
        if (c->bulk_scales)
            ds_load_scales(c, 0, l, c->p1_lo, c->p1_hi - c->p1_lo, fs, c->rows1_cap, c->sc1_plane, c->sc1_addr, lane, [&](uint32_t) {
                return ScaleSrc{reinterpret_cast<const uint8_t*>(L->sg_s), reinterpret_cast<const uint8_t*>(L->sg_b),
                                reinterpret_cast<const uint8_t*>(L->su_s), reinterpret_cast<const uint8_t*>(L->su_b)};
            });
        for (uint32_t s = 0; s < c->n_st1; ++s, ++q) {
            const uint32_t tile = s / 2, mat = s % 2;
            const uint32_t r0 = c->p1_lo + tile * 16;
            const uint32_t n = c->p1_hi - r0 < 16u ? c->p1_hi - r0 : 16u;
            const uint32_t dst = ds_open_stage(c, q, n * (d / 2), lane);
            if (!dst) continue;
            const uint8_t* W = mat ? L->su_w : L->sg_w;
            if ((uint32_t)lane * 2 < n) {       // rows 2 lane, 2 lane + 1 (consecutive in the matrix) as one copy
                const uint32_t nr = n - lane * 2 < 2u ? 1u : 2u;
                bulk_copy_g2s(dst + lane * (2 * RS + kDsPairPad), W + (size_t)(r0 + lane * 2) * RS, nr * RS, ds_bar_full(c, q % kDsStages));
            }
        }
        // the rows of P2 and P3 depend on the layer's top-k
        if (!*c->dead && !mbar_wait(ds_bar_routing(c), l & 1)) {
            if (lane == 0) ds_fail(c, kErrLoaderWait);
            __syncwarp();
        }
        const uint8_t* pool = L->pool;
        const uint64_t stride = L->stride;
        if (c->bulk_scales)
            ds_load_scales(c, 1, l, c->p2_lo, c->p2_hi - c->p2_lo, f, c->rows2_cap, c->sc2_plane, c->sc2_addr, lane, [&](uint32_t k) {
                const uint8_t* blob = pool + (uint64_t)c->sel_idx[k] * stride;
                return ScaleSrc{blob + L->off.gate_s_off, blob + L->off.gate_b_off, blob + L->off.up_s_off, blob + L->off.up_b_off};
            });
        for (uint32_t s = 0; s < c->n_st2; ++s, ++q) {
            const uint32_t tile = s / 2, mat = s % 2;
            const uint32_t i0 = c->p2_lo + tile * 16;
            const uint32_t n = c->p2_hi - i0 < 16u ? c->p2_hi - i0 : 16u;
            const uint32_t dst = ds_open_stage(c, q, n * (d / 2), lane);
            if (!dst) continue;
            if ((uint32_t)lane * 2 < n) {
                // slices start on even rows and f is even: a pair of rows never straddles two experts
                const uint32_t idx = i0 + lane * 2, k = idx / f, r = idx % f;
                const uint32_t nr = n - lane * 2 < 2u ? 1u : 2u;
                const uint8_t* src = pool + (uint64_t)c->sel_idx[k] * stride + (mat ? L->off.up_w_off : L->off.gate_w_off) + (size_t)r * RS;
                bulk_copy_g2s(dst + lane * (2 * RS + kDsPairPad), src, nr * RS, ds_bar_full(c, q % kDsStages));
            }
        }
        for (uint32_t s = 0; s < c->n_st3; ++s, ++q) {
            const uint32_t tile = s / (c->subs + 1), sub = s % (c->subs + 1);
            const uint32_t r0 = c->p3_lo + tile * 16;
            const uint32_t n = c->p3_hi - r0 < 16u ? c->p3_hi - r0 : 16u;
            if (sub < c->subs) {
                const uint32_t k0 = sub * 4, nk = K - k0 < 4u ? K - k0 : 4u;
                const uint32_t dst = ds_open_stage(c, q, n * nk * (f / 2), lane);
                if (!dst) continue;
                if ((uint32_t)lane < nk) {     // the rows of one expert are consecutive in its blob: one copy per expert
                    const uint8_t* src = pool + (uint64_t)c->sel_idx[k0 + lane] * stride + L->off.down_w_off + (size_t)r0 * (f / 2);
                    bulk_copy_g2s(dst + lane * 16 * (f / 2), src, n * (f / 2), ds_bar_full(c, q % kDsStages));
                }
            } else {
                const uint32_t dst = ds_open_stage(c, q, n * (fs / 2), lane);
                if (!dst) continue;
                if (lane == 0) bulk_copy_g2s(dst, L->sd_w + (size_t)r0 * (fs / 2), n * (fs / 2), ds_bar_full(c, q % kDsStages));
            }
        }
    }
    // Copies still in flight must land before the CTA's shared memory goes away: wait (bounded) for the last use of
    // every slot and of the scale buffers. On the normal path the consumers have already seen these phases complete.
    for (uint32_t back = 0; back < kDsStages && back < q; ++back) {
        const uint32_t qq = q - 1 - back;
        mbar_wait(ds_bar_full(c, qq % kDsStages), (qq / kDsStages) & 1);
    }
    if (c->bulk_scales && n_layers) {
        if (c->p1_hi > c->p1_lo) mbar_wait(ds_bar_sc_full(c, 0), (n_layers - 1) & 1);
        if (c->p2_hi > c->p2_lo) mbar_wait(ds_bar_sc_full(c, 1), (n_layers - 1) & 1);
    }
}

// ---------------------------------------------------------------------------
// compute warps
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// Runs the phase's items first, first + step, ... on this warp. Stage q0 + item.stage_local holds the item's rows;
// scale rows of the item's source start at sS[item.scale_base] as [row][item.scale_stride], biases plane_elems further
// on; partial sums of rows g and g + 8 go to partial[item][16]. VEC: scale rows are 8-byte aligned four groups at a time.
template <bool VEC>
__device__ __forceinline__ void run_items(const DsCtx* c, const DsItem* tab, uint32_t n_items, uint32_t first, uint32_t step,
                                          uint32_t q0, uint32_t rows, const uint16_t* sS, uint32_t plane_elems,
                                          const uint32_t* frag_base, const float* xsum_base, int lane, uint32_t prof_slot = 0) {
    const int g = lane >> 2, t = lane & 3;
    const uint16_t* sB = sS + plane_elems;
    float* partial = c->partial;
    const bool prof = c->prof != nullptr && c->cta == 0 && threadIdx.x == 0;
    long long t_wait = 0, t_load = 0, t_math = 0, t_tail = 0, t0 = prof ? clock64() : 0;
    for (uint32_t it = first; it < n_items; it += step) {
        const uint4 raw = *reinterpret_cast<const uint4*>(tab + it);
        // word 0: stage | items of the stage (8 bits) | row stride / 16 (8 bits); word 1: tile (15 bits) | pair padding | row offset
        const uint32_t stage_local = raw.x & 0xFFFFu, stage_items = (raw.x >> 16) & 0xFFu, rs = (raw.x >> 24) * 16u,
                       tile = raw.y & 0x7FFFu, pad = (raw.y & 0x8000u) ? kDsPairPad : 0u, row_off = raw.y >> 16,
                       group = raw.z & 0xFFFFu, scale_base = raw.z >> 16, scale_stride = raw.w & 0xFFFFu,
                       G0 = raw.w >> 20, ngr = (raw.w >> 16) & 0xFu;
        const uint32_t q = q0 + stage_local, slot = q % kDsStages;
        if (!*c->dead && !mbar_wait(ds_bar_full(c, slot), (q / kDsStages) & 1)) {
            if (lane == 0) ds_fail(c, kErrStageWait);
        }
        __syncwarp();
        if (prof) { const long long n = clock64(); t_wait += n - t0; t0 = n; }
        const uint32_t base = c->ring_addr + slot * c->stage_bytes + row_off + t * 8 + g * rs + (g >> 1) * pad;
        const uint32_t row8 = 8 * rs + 4 * pad;
        uint2 wa[4], wb[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if ((uint32_t)i < ngr) { wa[i] = lds64(base + i * 32); wb[i] = lds64(base + row8 + i * 32); }
            else { wa[i] = make_uint2(0u, 0u); wb[i] = make_uint2(0u, 0u); }
        }
        uint32_t r0 = tile * 16 + g, r1 = r0 + 8;
        r0 = r0 < rows ? r0 : rows - 1; r1 = r1 < rows ? r1 : rows - 1;
        const uint32_t i0 = scale_base + r0 * scale_stride + G0, i1 = scale_base + r1 * scale_stride + G0;
        uint16_t s0b[4], s1b[4], b0b[4], b1b[4];
        if constexpr (VEC) {
            const uint2 vs0 = *reinterpret_cast<const uint2*>(sS + i0), vs1 = *reinterpret_cast<const uint2*>(sS + i1);
            const uint2 vb0 = *reinterpret_cast<const uint2*>(sB + i0), vb1 = *reinterpret_cast<const uint2*>(sB + i1);
            s0b[0] = (uint16_t)vs0.x; s0b[1] = (uint16_t)(vs0.x >> 16); s0b[2] = (uint16_t)vs0.y; s0b[3] = (uint16_t)(vs0.y >> 16);
            s1b[0] = (uint16_t)vs1.x; s1b[1] = (uint16_t)(vs1.x >> 16); s1b[2] = (uint16_t)vs1.y; s1b[3] = (uint16_t)(vs1.y >> 16);
            b0b[0] = (uint16_t)vb0.x; b0b[1] = (uint16_t)(vb0.x >> 16); b0b[2] = (uint16_t)vb0.y; b0b[3] = (uint16_t)(vb0.y >> 16);
            b1b[0] = (uint16_t)vb1.x; b1b[1] = (uint16_t)(vb1.x >> 16); b1b[2] = (uint16_t)vb1.y; b1b[3] = (uint16_t)(vb1.y >> 16);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const bool ok = (uint32_t)i < ngr;
                s0b[i] = ok ? sS[i0 + i] : (uint16_t)0; s1b[i] = ok ? sS[i1 + i] : (uint16_t)0;
                b0b[i] = ok ? sB[i0 + i] : (uint16_t)0; b1b[i] = ok ? sB[i1 + i] : (uint16_t)0;
            }
        }
        if (prof) { const long long n = clock64(); t_load += n - t0; t0 = n; }
        float zc[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) asm volatile("mov.f32 %0, 0f00000000;" : "=f"(zc[j]));
        float cacc[4][4];
        const uint32_t* frag = frag_base + (group * 4 + t) * 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint2 bf = make_uint2(0u, 0u);
                if (g == 0 && (uint32_t)i < ngr) bf = *reinterpret_cast<const uint2*>(frag + i * 32 + j * 2);
                const uint32_t wx = (j < 2) ? wa[i].x : wa[i].y, wy = (j < 2) ? wb[i].x : wb[i].y;
                const uint32_t mask = (j & 1) ? 0x00F000F0u : 0x000F000Fu;
                const uint32_t a0 = wx & mask, a1 = wy & mask, a2 = (wx >> 8) & mask, a3 = (wy >> 8) & mask;
                if (j == 0) gm_mma(cacc[i], a0, a1, a2, a3, bf.x, bf.y, zc);
                else gm_mma(cacc[i], a0, a1, a2, a3, bf.x, bf.y, cacc[i]);
            }
        }
        float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if ((uint32_t)i < ngr) {
                // the codes entered the MMA as q * 2^-24: fold 2^24 into the scale
                const float s0 = bf16_bits_to_float(s0b[i]) * 16777216.0f, s1 = bf16_bits_to_float(s1b[i]) * 16777216.0f;
                const float xs = xsum_base[group + i];
                acc0 = fmaf(s0, cacc[i][0], fmaf(bf16_bits_to_float(b0b[i]), xs, acc0));
                acc1 = fmaf(s1, cacc[i][2], fmaf(bf16_bits_to_float(b1b[i]), xs, acc1));
            }
        }
        if (t == 0) { partial[it * 16 + g] = acc0; partial[it * 16 + g + 8] = acc1; }
        __syncwarp();
        if (prof) { const long long n = clock64(); t_math += n - t0; t0 = n; }
        if (lane == 0) {
            // the last item that read the stage hands the slot back to the loader
            if (atomicAdd(&c->cnt[slot], 1u) + 1u == stage_items) {
                c->cnt[slot] = 0u;
                mbar_arrive(ds_bar_empty(c, slot));
            }
        }
        if (prof) { const long long n = clock64(); t_tail += n - t0; t0 = n; }
    }
    if (prof) {
        c->prof[prof_slot * 4 + 0] += t_wait; c->prof[prof_slot * 4 + 1] += t_load;
        c->prof[prof_slot * 4 + 2] += t_math; c->prof[prof_slot * 4 + 3] += t_tail;
    }
}

// B fragments and group sums of an fp16 vector that sits in shared memory (16-byte aligned, n = 64 ng).
__device__ __forceinline__ void stage_frags(const uint16_t* xs, uint32_t ng, uint32_t* frag, float* xsum) {
    for (uint32_t idx = threadIdx.x; idx < ((ng * 4 + 31u) & ~31u); idx += kDsComputeThreads) {     // whole warps: shuffles below
        const bool ok = idx < ng * 4;
        uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
        if (ok) {
            const uint4* p = reinterpret_cast<const uint4*>(xs + idx * 16);
            lo = p[0]; hi = p[1];
        }
        const uint32_t r[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float sum = 0.0f;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&r[q]));
            sum += v.x + v.y;
        }
        sum += __shfl_xor_sync(kFullMask, sum, 1);
        sum += __shfl_xor_sync(kFullMask, sum, 2);
        if (!ok) continue;
        if ((idx & 3u) == 0u) xsum[idx >> 2] = sum;
        gm_make_frag(r, frag + idx * 8);
    }
}

// A warp copies n consecutive 16-bit values from global memory into shared memory, eight loads in flight per lane.
__device__ __forceinline__ void warp_copy_u16(const uint16_t* __restrict__ src, uint16_t* dst, uint32_t n, int lane) {
    for (uint32_t base = lane; base < n; base += kWarp * 8) {
        uint16_t v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t i = base + j * kWarp;
            v[j] = i < n ? __ldg(src + i) : (uint16_t)0;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t i = base + j * kWarp;
            if (i < n) dst[i] = v[j];
        }
    }
}

// Optional fine-grained timing: CTA 0, thread 0 adds the time since the previous mark to prof[12 + slot].
struct DsMark {
    unsigned long long* acc; unsigned long long last;
    __device__ __forceinline__ DsMark(const DsCtx* c) : acc(nullptr), last(0) {
        if (c->prof && c->cta == 0 && threadIdx.x == 0) { acc = c->prof + 12; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(last)); }
    }
    __device__ __forceinline__ void mark(int slot) {
        if (acc) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); acc[slot] += t - last; last = t; }
    }
};

// A warp copies rows x ng consecutive 16-bit values from global memory into rows of ng_pad values in shared memory.
__device__ __forceinline__ void warp_copy_rows_u16(const uint16_t* __restrict__ src, uint16_t* dst, uint32_t rows, uint32_t ng,
                                                   uint32_t ng_pad, int lane) {
    const uint32_t n = rows * ng;
    const uint32_t rcp = 0xFFFFFFFFu / ng + 1u;             // e / ng = umulhi(e, rcp) for the small e of a slice
    for (uint32_t base = lane; base < n; base += kWarp * 8) {
        uint16_t v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t i = base + j * kWarp;
            v[j] = i < n ? __ldg(src + i) : (uint16_t)0;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t i = base + j * kWarp;
            if (i < n) {
                const uint32_t r = __umulhi(i, rcp);
                dst[r * ng_pad + (i - r * ng)] = v[j];
            }
        }
    }
}

// P0: x = half(rmsnorm(h) * w) into shared memory (bits of residual_rmsnorm_kernel: same thread striding and
// reduction tree), its B fragments, and the router's fp32 operand x * effective_scale.
__device__ __noinline__ void ds_phase0(const DsCtx* c, const DecodeLayer* L) {
    const uint32_t d = c->d, vecs = d / 8;
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    float v[kDsNormSlices][8];
    uint4 wv[kDsNormSlices];
    float acc = 0.0f;
    const uint16_t* nw = L->norm_w;
    // the effective scale of the router for this thread's eight columns: issued with the other loads
    uint4 ev = make_uint4(0u, 0u, 0u, 0u);
    const bool eff16 = (reinterpret_cast<uintptr_t>(L->eff) & 15) == 0;
    if (eff16 && threadIdx.x < vecs) ev = __ldg(reinterpret_cast<const uint4*>(L->eff) + threadIdx.x);
    if (threadIdx.x < kDsNormThreads) {
        uint4 hv[kDsNormSlices];
#pragma unroll
        for (int s = 0; s < kDsNormSlices; ++s) {
            const uint32_t i = threadIdx.x + s * kDsNormThreads;
            hv[s] = make_uint4(0u, 0u, 0u, 0u); wv[s] = hv[s];
            if (i < vecs) { hv[s] = __ldcg(reinterpret_cast<const uint4*>(c->hidden) + i); wv[s] = __ldg(reinterpret_cast<const uint4*>(nw) + i); }
        }
#pragma unroll
        for (int s = 0; s < kDsNormSlices; ++s) {
            const uint32_t i = threadIdx.x + s * kDsNormThreads;
            if (i < vecs) {
                const uint32_t hw[4] = {hv[s].x, hv[s].y, hv[s].z, hv[s].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&hw[j]));
                    v[s][2 * j] = a.x; v[s][2 * j + 1] = a.y;
                    acc = fmaf(a.x, a.x, acc); acc = fmaf(a.y, a.y, acc);
                }
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) c->red[warp] = acc;
    }
    cta_sync();
    if (threadIdx.x < kDsNormThreads) {
        float tot = lane < kDsNormThreads / kWarp ? c->red[lane] : 0.0f;
        tot = warp_sum(tot);
        const float inv = rsqrtf(tot / (float)d + c->eps);
#pragma unroll
        for (int s = 0; s < kDsNormSlices; ++s) {
            const uint32_t i = threadIdx.x + s * kDsNormThreads;
            if (i < vecs) {
                const uint32_t ww[4] = {wv[s].x, wv[s].y, wv[s].z, wv[s].w};
                uint32_t ow[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half2 r = __floats2half2_rn(v[s][2 * j] * inv * bf16_bits_to_float((uint16_t)(ww[j] & 0xFFFFu)),
                                                        v[s][2 * j + 1] * inv * bf16_bits_to_float((uint16_t)(ww[j] >> 16)));
                    ow[j] = *reinterpret_cast<const uint32_t*>(&r);
                }
                reinterpret_cast<uint4*>(c->x16)[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
        }
    }
    cta_sync();
    stage_frags(c->x16, c->ngd, c->frag_a, c->sum_a);
    if (eff16) {
        if (threadIdx.x < vecs) {
            const uint4 xv = reinterpret_cast<const uint4*>(c->x16)[threadIdx.x];
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, ew[4] = {ev.x, ev.y, ev.z, ev.w};
            float* out = c->xf + threadIdx.x * 8;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                out[2 * j] = __fmul_rn(f16_bits_to_float((uint16_t)(xw[j] & 0xFFFFu)), bf16_bits_to_float((uint16_t)(ew[j] & 0xFFFFu)));
                out[2 * j + 1] = __fmul_rn(f16_bits_to_float((uint16_t)(xw[j] >> 16)), bf16_bits_to_float((uint16_t)(ew[j] >> 16)));
            }
        }
    } else {
        const uint16_t* eff = L->eff;
        for (uint32_t i = threadIdx.x; i < d; i += kDsComputeThreads)
            c->xf[i] = __fmul_rn(f16_bits_to_float(c->x16[i]), bf16_bits_to_float(eff[i]));
    }
    cta_sync();
}

// Scale rows of a gate/up slice by the compute warps (the fallback when the loader cannot bulk-copy them): one warp
// per (run, matrix, plane), same shared-memory layout as ds_load_scales.
template <typename SrcOf>
__device__ __forceinline__ void ds_stage_scales_plain(const DsCtx* c, uint32_t lo, uint32_t rows, uint32_t space_rows, uint32_t rows_cap,
                                                      uint32_t plane_elems, uint16_t* dst, SrcOf src_of) {
    if (rows == 0) return;
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t ngd = c->ngd;
    const uint32_t first_space = lo / space_rows, last_space = (lo + rows - 1) / space_rows;
    const uint32_t n_jobs = (last_space - first_space + 1) * 4;
    for (uint32_t j = warp; j < n_jobs; j += kDsComputeWarps) {
        const uint32_t run = j / 4, which_plane = j % 4;
        const uint32_t sp = first_space + run;
        const uint32_t r_lo = sp == first_space ? lo - sp * space_rows : 0u;
        const uint32_t r_hi = sp == last_space ? lo + rows - sp * space_rows : space_rows;
        const ScaleSrc src = src_of(sp);
        const uint8_t* plane = which_plane == 0 ? src.gate_s : which_plane == 1 ? src.gate_b : which_plane == 2 ? src.up_s : src.up_b;
        const uint32_t mat = which_plane / 2, pl = which_plane % 2;
        const uint32_t local_row = sp * space_rows + r_lo - lo;
        warp_copy_u16(reinterpret_cast<const uint16_t*>(plane) + (size_t)r_lo * ngd,
                      dst + pl * plane_elems + mat * rows_cap * ngd + local_row * ngd, (r_hi - r_lo) * ngd, lane);
    }
}

// Waits (bounded) until the loader's scale rows of P1 / P2 have landed.
__device__ __forceinline__ void ds_wait_scales(const DsCtx* c, uint32_t which, uint32_t layer, uint32_t rows) {
    if (!c->bulk_scales || rows == 0 || *c->dead) return;
    if (!mbar_wait(ds_bar_sc_full(c, which), layer & 1)) {
        if ((threadIdx.x % kWarp) == 0) ds_fail(c, kErrScaleWait);
    }
}

// P1: this CTA's router rows (canonical logit, last compute warp) beside its slice of the shared expert's gate/up rows.
__device__ __noinline__ void ds_phase1(const DsCtx* c, const DecodeLayer* L, uint32_t q0, uint32_t layer) {
    const uint32_t d = c->d, ngd = c->ngd, kp_d = c->kp_d;
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t lo = c->p1_lo, rows = c->p1_hi - c->p1_lo;
    const uint32_t n_items = c->p1_tiles * 2 * kp_d;
    if (!c->bulk_scales) {
        ds_stage_scales_plain(c, lo, rows, c->fs, c->rows1_cap, c->sc1_plane, c->sc1, [&](uint32_t) {
            return ScaleSrc{reinterpret_cast<const uint8_t*>(L->sg_s), reinterpret_cast<const uint8_t*>(L->sg_b),
                            reinterpret_cast<const uint8_t*>(L->su_s), reinterpret_cast<const uint8_t*>(L->su_b)};
        });
        cta_sync();
    }
    const bool has_router_row = c->cta < c->E;
    if (warp == kDsComputeWarps - 1 && has_router_row) {
        // the router rows of this CTA: the whole row lands in registers before the first store
        uint16_t* srow = reinterpret_cast<uint16_t*>(c->wrow + ((d + 15u) & ~15u));
        uint16_t* brow = srow + ((ngd * 2 + 15u) & ~15u) / 2;
        for (uint32_t e = c->cta; e < c->E; e += c->grid) {
            const uint8_t* wsrc = L->router_w + (size_t)e * d;
            if ((reinterpret_cast<uintptr_t>(wsrc) & 15) == 0 && d <= 16u * kWarp * 8u) {
                uint4 rv[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t i = lane + j * kWarp;
                    rv[j] = i < d / 16 ? ldg_nc_u4(wsrc + (size_t)i * 16) : make_uint4(0u, 0u, 0u, 0u);
                }
                uint16_t sv[2] = {0, 0}, bv[2] = {0, 0};
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint32_t i = lane + j * kWarp;
                    if (i < ngd) { sv[j] = L->router_s[(size_t)e * ngd + i]; bv[j] = L->router_b[(size_t)e * ngd + i]; }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t i = lane + j * kWarp;
                    if (i < d / 16) reinterpret_cast<uint4*>(c->wrow)[i] = rv[j];
                }
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint32_t i = lane + j * kWarp;
                    if (i < ngd) { srow[i] = sv[j]; brow[i] = bv[j]; }
                }
                for (uint32_t i = lane + 2 * kWarp; i < ngd; i += kWarp) {
                    srow[i] = L->router_s[(size_t)e * ngd + i];
                    brow[i] = L->router_b[(size_t)e * ngd + i];
                }
            } else {
                for (uint32_t i = lane; i < d; i += kWarp) c->wrow[i] = wsrc[i];
                for (uint32_t i = lane; i < ngd; i += kWarp) {
                    srow[i] = L->router_s[(size_t)e * ngd + i];
                    brow[i] = L->router_b[(size_t)e * ngd + i];
                }
            }
            __syncwarp();
            float logit = router_row_logit_smem(c->wrow, srow, brow, c->xf, ngd, lane);
            if (L->logit_bias) logit = __fadd_rn(logit, L->logit_bias[e]);
            if (lane == 0) c->logits[e] = logit;
            __syncwarp();
        }
    } else {
        // the other warps (all of them where the CTA has no router row) share the items
        const uint32_t workers = has_router_row ? kDsComputeWarps - 1 : kDsComputeWarps;
        ds_wait_scales(c, 0, layer, rows);
        if (ngd % 4 == 0) run_items<true>(c, c->tabs, n_items, warp, workers, q0, rows, c->sc1, c->sc1_plane, c->frag_a, c->sum_a, lane, 0);
        else run_items<false>(c, c->tabs, n_items, warp, workers, q0, rows, c->sc1, c->sc1_plane, c->frag_a, c->sum_a, lane, 0);
    }
    cta_sync();
    if (threadIdx.x == 0 && c->bulk_scales && rows) mbar_arrive(ds_bar_sc_empty(c, 0));
    const float* partial = c->partial;
    for (uint32_t j = threadIdx.x; j < rows; j += kDsComputeThreads) {
        const uint32_t tile = j / 16, r = j % 16;
        float gt = 0.0f, up = 0.0f;
        for (uint32_t kp = 0; kp < kp_d; ++kp) {
            gt += partial[((tile * 2 + 0) * kp_d + kp) * 16 + r];
            up += partial[((tile * 2 + 1) * kp_d + kp) * 16 + r];
        }
        // the shared expert stores gate and up as fp16 before the activation
        gt = __half2float(__float2half_rn(gt));
        up = __half2float(__float2half_rn(up));
        c->shared_act[lo + j] = __half_as_ushort(__float2half_rn(gelu_tanh(gt) * up));
    }
}

// P2: top-k of the logits (every CTA, identically), then this CTA's slice of the routed experts' gate/up rows.
__device__ __noinline__ void ds_phase2(const DsCtx* c, const DecodeLayer* L, const DecodeLayer* N, uint32_t q0, uint32_t layer) {
    const uint32_t d = c->d, f = c->f, E = c->E, K = c->K, ngd = c->ngd, ngf = c->ngf, ngs = c->ngs, kp_d = c->kp_d;
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    DsMark mk(c);
    for (uint32_t i = threadIdx.x; i < E; i += kDsComputeThreads) c->scores[i] = __ldcg(c->logits + i);
    cta_sync();
    mk.mark(0);
    if (warp == 0) {
        warp_select_topk(c->scores, E, K, L->pes, c->sel_idx, c->sel_w, lane);
        __syncwarp();
        if ((uint32_t)lane < K) {
            uint32_t e = c->sel_idx[lane];
            if (c->cta == 0) { c->out_idx[lane] = e; c->out_w[lane] = c->sel_w[lane]; }
            if (e >= E) e = E - 1;                        // min(id, E-1): Runtime/Inference/RealForwardRunner.swift:1486
            c->sel_idx[lane] = e;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_bar_routing(c));    // the loader may now address the routed experts
    }
    cta_sync();
    mk.mark(1);
    const uint32_t lo = c->p2_lo, rows = c->p2_hi - c->p2_lo;
    const uint32_t n_items = c->p2_tiles * 2 * kp_d;
    const uint8_t* pool = L->pool;
    const uint64_t stride = L->stride;
    const tf_expert_offsets off = L->off;
    const uint32_t* sel = c->sel_idx;
    if (!c->bulk_scales) {
        ds_stage_scales_plain(c, lo, rows, f, c->rows2_cap, c->sc2_plane, c->sc2, [&](uint32_t k) {
            const uint8_t* blob = pool + (uint64_t)sel[k] * stride;
            return ScaleSrc{blob + off.gate_s_off, blob + off.gate_b_off, blob + off.up_s_off, blob + off.up_b_off};
        });
    }
    // Scale and bias rows of P3 depend only on the routing: one warp asks for them in L2 now, P3 copies them from there.
    if (warp == kDsComputeWarps - 2) {
        const uint32_t lo3 = c->p3_lo, n3 = c->p3_hi - c->p3_lo;
        if (n3) {
            for (uint32_t src = 0; src < K; ++src) {
                const uint8_t* blob = pool + (uint64_t)sel[src] * stride;
                prefetch_l2_warp(blob + off.down_s_off + (size_t)lo3 * ngf * 2, n3 * ngf * 2, lane);
                prefetch_l2_warp(blob + off.down_b_off + (size_t)lo3 * ngf * 2, n3 * ngf * 2, lane);
            }
            prefetch_l2_warp(L->sd_s + (size_t)lo3 * ngs, n3 * ngs * 2, lane);
            prefetch_l2_warp(L->sd_b + (size_t)lo3 * ngs, n3 * ngs * 2, lane);
        }
    }
    // the last warp brings the next layer's small operands into L2 ahead of use
    if (warp == kDsComputeWarps - 1 && N) {
        for (uint32_t e = c->cta; e < E; e += c->grid) {
            prefetch_l2_warp(N->router_w + (size_t)e * d, d, lane);
            prefetch_l2_warp(N->router_s + (size_t)e * ngd, ngd * 2, lane);
            prefetch_l2_warp(N->router_b + (size_t)e * ngd, ngd * 2, lane);
        }
        if (c->cta < 8) {
            prefetch_l2_warp(N->norm_w, d * 2, lane);
            prefetch_l2_warp(N->eff, d * 2, lane);
        }
    }
    if (!c->bulk_scales) cta_sync();
    mk.mark(2);
    ds_wait_scales(c, 1, layer, rows);
    mk.mark(3);
    if (ngd % 4 == 0) run_items<true>(c, c->tabs + kDsMaxItems, n_items, warp, kDsComputeWarps, q0, rows, c->sc2, c->sc2_plane, c->frag_a, c->sum_a, lane, 1);
    else run_items<false>(c, c->tabs + kDsMaxItems, n_items, warp, kDsComputeWarps, q0, rows, c->sc2, c->sc2_plane, c->frag_a, c->sum_a, lane, 1);
    mk.mark(4);
    cta_sync();
    mk.mark(5);
    if (threadIdx.x == 0 && c->bulk_scales && rows) mbar_arrive(ds_bar_sc_empty(c, 1));
    const float* partial = c->partial;
    for (uint32_t j = threadIdx.x; j < rows; j += kDsComputeThreads) {
        const uint32_t tile = j / 16, r = j % 16;
        float gt = 0.0f, up = 0.0f;
        for (uint32_t kp = 0; kp < kp_d; ++kp) {
            gt += partial[((tile * 2 + 0) * kp_d + kp) * 16 + r];
            up += partial[((tile * 2 + 1) * kp_d + kp) * 16 + r];
        }
        c->acts[lo + j] = __half_as_ushort(__float2half_rn(gelu_tanh(gt) * up));     // moe.metal:368
    }
    mk.mark(6);
}

// Scale and bias rows of P3 from global memory (L2 after the prefetch of P2) into shared memory, all threads at once and
// every thread's loads issued before its first store. Layout: plane p at p * sc3_plane, source s (K routed experts, then
// the shared one) at s * rows3_cap * ngf_pad, then [row][groups padded to a multiple of four]. A job is up to
// kDsScaleChunk consecutive groups of one row of one source and plane.
constexpr uint32_t kDsScaleChunk = 12;
__device__ __forceinline__ void ds_stage_down_scales(const DsCtx* c, const DecodeLayer* L) {
    const uint32_t K = c->K, ngf = c->ngf, ngs = c->ngs;
    const uint32_t lo3 = c->p3_lo, n3 = c->p3_hi - c->p3_lo;
    const uint32_t cf = (ngf + kDsScaleChunk - 1) / kDsScaleChunk, cs = (ngs + kDsScaleChunk - 1) / kDsScaleChunk;
    const uint32_t per_row = K * cf + cs;                    // chunks of one (row, plane)
    const uint32_t jobs = n3 * 2 * per_row;
    const uint32_t rcp_row = 0xFFFFFFFFu / per_row + 1u;          // per_row >= 2
    const uint32_t rcp_cf = cf > 1 ? 0xFFFFFFFFu / cf + 1u : 0u;
    const uint8_t* pool = L->pool;
    const uint64_t stride = L->stride;
    for (uint32_t j = threadIdx.x; j < jobs; j += kDsComputeThreads) {
        const uint32_t rp = __umulhi(j, rcp_row), slot = j - rp * per_row;       // rp = row * 2 + plane
        const uint32_t r = rp >> 1, pl = rp & 1;
        const uint16_t* src;
        uint16_t* dst;
        uint32_t n;
        if (slot < K * cf) {
            const uint32_t k = cf > 1 ? __umulhi(slot, rcp_cf) : slot, ch = slot - k * cf;
            const uint8_t* blob = pool + (uint64_t)c->sel_idx[k] * stride;
            const uint32_t g0 = ch * kDsScaleChunk;
            src = reinterpret_cast<const uint16_t*>(blob + (pl ? L->off.down_b_off : L->off.down_s_off)) + (size_t)(lo3 + r) * ngf + g0;
            dst = c->sc3 + pl * c->sc3_plane + k * c->rows3_cap * c->ngf_pad + r * c->ngf_pad + g0;
            n = ngf - g0 < kDsScaleChunk ? ngf - g0 : kDsScaleChunk;
        } else {
            const uint32_t g0 = (slot - K * cf) * kDsScaleChunk;
            src = (pl ? L->sd_b : L->sd_s) + (size_t)(lo3 + r) * ngs + g0;
            dst = c->sc3 + pl * c->sc3_plane + K * c->rows3_cap * c->ngf_pad + r * c->ngs_pad + g0;
            n = ngs - g0 < kDsScaleChunk ? ngs - g0 : kDsScaleChunk;
        }
        uint16_t v[kDsScaleChunk];
#pragma unroll
        for (uint32_t i = 0; i < kDsScaleChunk; ++i) v[i] = i < n ? __ldg(src + i) : (uint16_t)0;
#pragma unroll
        for (uint32_t i = 0; i < kDsScaleChunk; ++i)
            if (i < n) dst[i] = v[i];
    }
}

// P3: down projections of the K routed experts and of the shared expert for this CTA's output rows, combine in rank
// order, residual add.
__device__ __noinline__ void ds_phase3(const DsCtx* c, const DecodeLayer* L, uint32_t q0) {
    const uint32_t f = c->f, fs = c->fs, K = c->K, ngf = c->ngf, ngs = c->ngs, kp_f = c->kp_f, kp_s = c->kp_s;
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t lo = c->p3_lo, rows = c->p3_hi - c->p3_lo, per_tile = c->p3_per_tile;
    const uint32_t n_act = K * f + fs;
    DsMark mk(c);
    for (uint32_t i = threadIdx.x; i < n_act / 8; i += kDsComputeThreads) {
        const uint32_t e8 = i * 8;
        const uint16_t* src = e8 < K * f ? c->acts + e8 : c->shared_act + (e8 - K * f);
        reinterpret_cast<uint4*>(c->a16)[i] = __ldcg(reinterpret_cast<const uint4*>(src));
    }
    ds_stage_down_scales(c, L);
    cta_sync();
    mk.mark(8);
    stage_frags(c->a16, K * ngf + ngs, c->frag_b, c->sum_b);      // K routed vectors of ngf groups, then the shared one
    // the residual row of this CTA's finalize lanes (half-warp per output row, below): read ahead of the item loop
    const uint32_t fin_row = threadIdx.x / 16, fin_lane = threadIdx.x % 16;
    float h_in = 0.0f;
    if (fin_lane == 0 && fin_row < rows) h_in = f16_bits_to_float(__ldcg(c->hidden + lo + fin_row));
    cta_sync();
    mk.mark(9);
    const uint32_t n_items = c->p3_tiles * per_tile;
    run_items<true>(c, c->tabs + 2 * kDsMaxItems, n_items, warp, kDsComputeWarps, q0, rows, c->sc3, c->sc3_plane, c->frag_b, c->sum_b, lane, 2);
    mk.mark(10);
    cta_sync();
    mk.mark(11);
    // Finalize: a half-warp per output row. Lane s < K sums the K-parts of routed expert s, lane K those of the shared
    // expert (each in ascending part order, as a single thread would); lane 0 then folds them in rank order.
    const float* partial = c->partial;
    for (uint32_t j0 = 0; j0 < rows; j0 += kDsComputeThreads / 16) {
        const uint32_t j = j0 + fin_row;
        const bool live = j < rows;
        float pk = 0.0f;
        if (live && fin_lane <= K) {
            const uint32_t tile = j / 16, r = j % 16;
            const float* pt = partial + (size_t)tile * per_tile * 16 + r;
            if (fin_lane < K) { for (uint32_t kp = 0; kp < kp_f; ++kp) pk += pt[(fin_lane * kp_f + kp) * 16]; }
            else              { for (uint32_t kp = 0; kp < kp_s; ++kp) pk += pt[(K * kp_f + kp) * 16]; }
        }
        const int base = (lane / 16) * 16;
        float acc = __half2float(__float2half_rn(__shfl_sync(kFullMask, pk, base + (int)K)));        // shared y is stored as fp16
        for (uint32_t k = 0; k < K; ++k) {
            const float p = __shfl_sync(kFullMask, pk, base + (int)k);
            acc = __fadd_rn(acc, __fmul_rn(f16_bits_to_float(c->sel_w[k]), p));                          // rank order 0..K-1
        }
        if (live && fin_lane == 0) {
            const float y = __half2float(__float2half_rn(acc));
            const float h = j0 == 0 ? h_in : f16_bits_to_float(__ldcg(c->hidden + lo + j));
            c->hidden[lo + j] = __half_as_ushort(__float2half_rn(h + y));
        }
    }
    mk.mark(12);
}

// Item tables of the three phases (constant across layers), built once per launch.
__device__ void ds_build_tables(const DsCtx* c) {
    const uint32_t kp_d = c->kp_d, kp_f = c->kp_f, kp_s = c->kp_s, K = c->K, ngd = c->ngd, ngf = c->ngf, ngs = c->ngs, f = c->f;
    for (uint32_t ph = 0; ph < 2; ++ph) {
        const uint32_t n = (ph ? c->p2_tiles : c->p1_tiles) * 2 * kp_d;
        const uint32_t rows_cap = ph ? c->rows2_cap : c->rows1_cap;
        for (uint32_t it = threadIdx.x; it < n; it += kDsComputeThreads) {
            const uint32_t st = it / kp_d, kp = it % kp_d, G0 = kp * 4;
            DsItem e;
            e.stage_local = (uint16_t)st; e.stage_items = (uint16_t)(kp_d | ((c->d / 32) << 8)); e.tile = (uint16_t)((st / 2) | 0x8000u);
            e.row_off = (uint16_t)(G0 * 32); e.group = (uint16_t)G0; e.scale_base = (uint16_t)((st % 2) * rows_cap * ngd);
            e.scale_stride = (uint16_t)ngd;
            e.g0_ngr = (uint16_t)((G0 << 4) | (ngd - G0 < 4u ? ngd - G0 : 4u));
            c->tabs[ph * kDsMaxItems + it] = e;
        }
    }
    const uint32_t per_tile = c->p3_per_tile, n3 = c->p3_tiles * per_tile;
    for (uint32_t it = threadIdx.x; it < n3; it += kDsComputeThreads) {
        const uint32_t tile = it / per_tile, rem = it % per_tile;
        DsItem e;
        e.tile = (uint16_t)tile;
        if (rem < K * kp_f) {
            const uint32_t k = rem / kp_f, G0 = (rem % kp_f) * 4, sub = k / 4;
            const uint32_t nk = K - sub * 4 < 4u ? K - sub * 4 : 4u;
            e.stage_local = (uint16_t)(tile * (c->subs + 1) + sub); e.stage_items = (uint16_t)((nk * kp_f) | ((f / 32) << 8));
            e.row_off = (uint16_t)((k % 4) * 16 * (f / 2) + G0 * 32); e.group = (uint16_t)(k * ngf + G0);
            e.scale_base = (uint16_t)(k * c->rows3_cap * c->ngf_pad); e.scale_stride = (uint16_t)c->ngf_pad;
            e.g0_ngr = (uint16_t)((G0 << 4) | (ngf - G0 < 4u ? ngf - G0 : 4u));
        } else {
            const uint32_t G0 = (rem - K * kp_f) * 4;
            e.stage_local = (uint16_t)(tile * (c->subs + 1) + c->subs); e.stage_items = (uint16_t)(kp_s | ((c->fs / 32) << 8));
            e.row_off = (uint16_t)(G0 * 32); e.group = (uint16_t)(K * ngf + G0);
            e.scale_base = (uint16_t)(K * c->rows3_cap * c->ngf_pad); e.scale_stride = (uint16_t)c->ngs_pad;
            e.g0_ngr = (uint16_t)((G0 << 4) | (ngs - G0 < 4u ? ngs - G0 : 4u));
        }
        c->tabs[2 * kDsMaxItems + it] = e;
    }
}

__global__ void __launch_bounds__(kDsThreads, 1)
decode_step_kernel(const DecodeArgs args) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ DsCtx ctx;
    if (threadIdx.x == 0) {
        const uint32_t d = args.d, f = args.f, fs = args.fs, E = args.E, K = args.K;
        const DsSmem lay(d, f, fs, E, K, gridDim.x);
        DsCtx& c = ctx;
        c.d = d; c.f = f; c.fs = fs; c.E = E; c.K = K;
        c.ngd = d / kGroup; c.ngf = f / kGroup; c.ngs = fs / kGroup;
        c.kp_d = ds_kparts(c.ngd); c.kp_f = ds_kparts(c.ngf); c.kp_s = ds_kparts(c.ngs);
        c.subs = (K + 3) / 4;
        c.cta = blockIdx.x; c.grid = gridDim.x;
        c.p1_lo = ds_split_rows(fs, c.cta, c.grid); c.p1_hi = ds_split_rows(fs, c.cta + 1, c.grid);
        c.p2_lo = ds_split_rows(K * f, c.cta, c.grid); c.p2_hi = ds_split_rows(K * f, c.cta + 1, c.grid);
        c.p3_lo = ds_split(d, c.cta, c.grid); c.p3_hi = ds_split(d, c.cta + 1, c.grid);
        c.p1_tiles = (c.p1_hi - c.p1_lo + 15) / 16; c.p2_tiles = (c.p2_hi - c.p2_lo + 15) / 16; c.p3_tiles = (c.p3_hi - c.p3_lo + 15) / 16;
        c.p3_per_tile = K * c.kp_f + c.kp_s;
        c.n_st1 = c.p1_tiles * 2; c.n_st2 = c.p2_tiles * 2; c.n_st3 = c.p3_tiles * (c.subs + 1);
        c.row_stride = lay.row_stride; c.stage_bytes = lay.stage_bytes;
        c.rows1_cap = lay.rows1; c.rows2_cap = lay.rows2; c.rows3_cap = lay.rows3;
        c.sc1_plane = lay.sc1_plane; c.sc2_plane = lay.sc2_plane; c.sc3_plane = lay.sc3_plane;
        c.ngf_pad = (c.ngf + 3u) & ~3u; c.ngs_pad = (c.ngs + 3u) & ~3u;
        c.bulk_scales = args.bulk_scales;
        c.ring = smem + lay.ring; c.ring_addr = smem_addr_u32(c.ring);
        c.bars_addr = smem_addr_u32(smem + lay.bars);
        c.sc1 = reinterpret_cast<uint16_t*>(smem + lay.sc1); c.sc1_addr = smem_addr_u32(c.sc1);
        c.sc2 = reinterpret_cast<uint16_t*>(smem + lay.sc2); c.sc2_addr = smem_addr_u32(c.sc2);
        c.sc3 = reinterpret_cast<uint16_t*>(smem + lay.sc3);
        c.x16 = reinterpret_cast<uint16_t*>(smem + lay.x16);
        c.xf = reinterpret_cast<float*>(smem + lay.xf);
        c.a16 = reinterpret_cast<uint16_t*>(smem + lay.a16);
        c.frag_a = reinterpret_cast<uint32_t*>(smem + lay.frag_a);
        c.sum_a = reinterpret_cast<float*>(smem + lay.sum_a);
        c.frag_b = reinterpret_cast<uint32_t*>(smem + lay.frag_b);
        c.sum_b = reinterpret_cast<float*>(smem + lay.sum_b);
        c.wrow = smem + lay.wrow;
        c.partial = reinterpret_cast<float*>(smem + lay.partial);
        c.tabs = reinterpret_cast<DsItem*>(smem + lay.tabs);
        c.scores = reinterpret_cast<float*>(smem + lay.scores);
        c.sel_idx = reinterpret_cast<uint32_t*>(smem + lay.sel_idx);
        c.sel_w = reinterpret_cast<uint16_t*>(smem + lay.sel_w);
        c.red = reinterpret_cast<float*>(smem + lay.red);
        c.cnt = reinterpret_cast<uint32_t*>(smem + lay.cnt);
        c.dead = c.cnt + kDsStages;
        c.hidden = args.hidden; c.logits = args.logits; c.acts = args.acts; c.shared_act = args.shared_act;
        c.out_idx = args.out_idx; c.out_w = args.out_w; c.error = args.error; c.eps = args.eps;
        // a trace buffer with room beyond the phase stamps also receives the item-loop cycle counts (12 words)
        c.prof = (args.trace && args.trace_capacity >= 8 * args.n_layers + 28) ? args.trace + 8 * args.n_layers : nullptr;
        if (c.prof && blockIdx.x == 0) for (int i = 0; i < 28; ++i) c.prof[i] = 0ull;
        for (uint32_t s = 0; s < kDsStages; ++s) {
            mbar_init(c.bars_addr + s * 8, 1);
            mbar_init(c.bars_addr + (kDsStages + s) * 8, 1);
            c.cnt[s] = 0u;
        }
        for (uint32_t s = 0; s < 5; ++s) mbar_init(c.bars_addr + (2 * kDsStages + s) * 8, 1);     // routing, scales full x 2, empty x 2
        *c.dead = 0u;
        fence_proxy_async();
    }
    __syncthreads();
    if (threadIdx.x >= kDsComputeThreads) {
        ds_loader(&ctx, args.layers, args.n_layers);
        return;
    }
    ds_build_tables(&ctx);
    cta_sync();
    GridSync gs{args.barrier, 0u};
    uint32_t stamp_at = 0;
    auto stamp = [&]() {
        if (args.trace && blockIdx.x == 0 && threadIdx.x == 0 && stamp_at < args.trace_capacity) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            args.trace[stamp_at++] = t;
        }
    };
    const uint32_t per_layer = ctx.n_st1 + ctx.n_st2 + ctx.n_st3;
    for (uint32_t l = 0; l < args.n_layers; ++l) {
        const DecodeLayer* L = args.layers + l;
        const uint32_t q0 = l * per_layer;
        stamp();
        ds_phase0(&ctx, L);
        stamp();
        ds_phase1(&ctx, L, q0, l);
        stamp();
        grid_sync(&ctx, gs);
        stamp();
        ds_phase2(&ctx, L, l + 1 < args.n_layers ? L + 1 : nullptr, q0 + ctx.n_st1, l);
        stamp();
        grid_sync(&ctx, gs);
        stamp();
        ds_phase3(&ctx, L, q0 + ctx.n_st1 + ctx.n_st2);
        stamp();
        grid_sync(&ctx, gs);
        stamp();
    }
}

}  // namespace tf

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
namespace tf {

static uint32_t ds_max_items(uint32_t d, uint32_t f, uint32_t fs, uint32_t K, uint32_t grid) {
    uint32_t worst = 0;
    const uint32_t kp_d = ds_kparts(d / 64), kp_f = ds_kparts(f / 64), kp_s = ds_kparts(fs / 64);
    for (uint32_t c = 0; c < grid; ++c) {
        const uint32_t t1 = (ds_split_rows(fs, c + 1, grid) - ds_split_rows(fs, c, grid) + 15) / 16;
        const uint32_t t2 = (ds_split_rows(K * f, c + 1, grid) - ds_split_rows(K * f, c, grid) + 15) / 16;
        const uint32_t t3 = (ds_split(d, c + 1, grid) - ds_split(d, c, grid) + 15) / 16;
        const uint32_t m = std::max(std::max(t1 * 2 * kp_d, t2 * 2 * kp_d), t3 * (K * kp_f + kp_s));
        worst = std::max(worst, m);
    }
    return worst;
}

// Whether the stack's layers can take the single-launch step (same dimensions everywhere, aligned planes).
bool decode_step_eligible(const tf_stack* st, const tf_workspace* ws) {
    if (!st->device_layers || st->layers.empty()) return false;
    const tf_moe_layer& a = st->layers[0];
    const uint32_t d = a.d, f = a.f, fs = a.fs, E = a.num_experts, K = a.top_k;
    if (d % 64 || f % 64 || fs % 64 || d == 0 || f == 0 || fs == 0) return false;
    if (d > 8u * kDsNormThreads * kDsNormSlices || E > TF_MAX_ROUTER_EXPERTS || K == 0 || K > TF_MAX_TOP_K || E < K) return false;
    if (ws->d != d || ws->f != f || ws->fs != fs || ws->top_k != K || ws->num_experts != E) return false;
    const uint32_t grid = (uint32_t)st->ctx->sm_count;
    if (ds_max_items(d, f, fs, K, grid) > kDsMaxItems) return false;
    const DsSmem lay(d, f, fs, E, K, grid);
    if (lay.total > 227u * 1024u) return false;
    // 8-bit fields of the item table: row strides in 16-byte units, items per stage; 16-bit row offsets inside a stage
    if (d / 32 > 0xFFu || f / 32 > 0xFFu || fs / 32 > 0xFFu || 4u * ((f / 64 + 3) / 4) > 0xFFu || (d / 64 + 3) / 4 > 0xFFu ||
        (fs / 64 + 3) / 4 > 0xFFu || lay.stage_bytes > 0xFFFFu) return false;
    // 16-bit fields of the item table
    if ((uint64_t)K * (f / 64) + fs / 64 > 0xFFFu || d / 64 > 0xFFFu) return false;
    if ((uint64_t)2 * lay.rows2 * (d / 64) > 0xFFFFu || (uint64_t)2 * lay.rows1 * (d / 64) > 0xFFFFu ||
        (uint64_t)lay.rows3 * (K * ((f / 64 + 3) & ~3u) + ((fs / 64 + 3) & ~3u)) > 0xFFFFu) return false;
    return st->decode_step_ok;
}

tf_status decode_step_prepare(tf_context* ctx, tf_stack* st) {
    // one device copy of the per-layer pointers; alignment rules of the stage copies (16-byte rows) and 2-byte planes
    std::vector<DecodeLayer> host(st->layers.size());
    bool ok = true;
    for (size_t l = 0; l < st->layers.size(); ++l) {
        const tf_moe_layer& m = st->layers[l];
        const tf_moe_layer& a = st->layers[0];
        ok = ok && m.d == a.d && m.f == a.f && m.fs == a.fs && m.num_experts == a.num_experts && m.top_k == a.top_k;
        DecodeLayer& o = host[l];
        auto w = [](const tf_projection& p) { return byte_ptr(p.weights, p.weights_off); };
        auto s = [](const tf_projection& p) { return reinterpret_cast<const uint16_t*>(byte_ptr(p.scales, p.scales_off)); };
        auto b = [](const tf_projection& p) { return reinterpret_cast<const uint16_t*>(byte_ptr(p.biases, p.biases_off)); };
        o.router_w = w(m.router); o.router_s = s(m.router); o.router_b = b(m.router);
        o.eff = static_cast<const uint16_t*>(m.effective_scale); o.pes = static_cast<const uint16_t*>(m.per_expert_scale);
        o.logit_bias = m.logit_bias;
        o.pool = static_cast<const uint8_t*>(m.pool_layer_base); o.stride = m.expert_stride; o.off = m.offsets;
        o.sg_w = w(m.shared_gate); o.sg_s = s(m.shared_gate); o.sg_b = b(m.shared_gate);
        o.su_w = w(m.shared_up); o.su_s = s(m.shared_up); o.su_b = b(m.shared_up);
        o.sd_w = w(m.shared_down); o.sd_s = s(m.shared_down); o.sd_b = b(m.shared_down);
        o.norm_w = static_cast<const uint16_t*>(st->norm_weights[l]);
        ok = ok && m.router.rows == m.num_experts && m.router.cols == m.d && m.shared_bits != 8;
        ok = ok && m.shared_gate.rows == m.fs && m.shared_gate.cols == m.d && m.shared_up.rows == m.fs && m.shared_up.cols == m.d &&
             m.shared_down.rows == m.d && m.shared_down.cols == m.fs;
        ok = ok && aligned(o.pool, 16) && o.stride % 16 == 0 && o.off.gate_w_off % 16 == 0 && o.off.up_w_off % 16 == 0 && o.off.down_w_off % 16 == 0;
        ok = ok && aligned(o.sg_w, 16) && aligned(o.su_w, 16) && aligned(o.sd_w, 16) && aligned(o.norm_w, 16);
        const uint32_t sb[6] = {o.off.gate_s_off, o.off.gate_b_off, o.off.up_s_off, o.off.up_b_off, o.off.down_s_off, o.off.down_b_off};
        for (uint32_t v : sb) ok = ok && v % 2 == 0;
        ok = ok && aligned(o.sg_s, 2) && aligned(o.sg_b, 2) && aligned(o.su_s, 2) && aligned(o.su_b, 2) && aligned(o.sd_s, 2) &&
             aligned(o.sd_b, 2) && aligned(o.router_s, 2) && aligned(o.router_b, 2) && aligned(o.eff, 2) && aligned(o.pes, 2);
    }
    st->decode_step_ok = ok;
    if (!ok) return TF_OK;
    // The loader can fetch the gate/up scale rows with bulk copies when every run of rows starts and ends on a
    // 16-byte boundary: even row spaces (slices then start on even rows), two scale rows a multiple of 16 bytes, and
    // 16-byte aligned planes.
    {
        const tf_moe_layer& a = st->layers[0];
        bool bulk = (a.d / 64) % 4 == 0 && a.fs % 2 == 0 && a.f % 2 == 0;
        for (const DecodeLayer& o : host) {
            bulk = bulk && aligned(o.sg_s, 16) && aligned(o.sg_b, 16) && aligned(o.su_s, 16) && aligned(o.su_b, 16) &&
                   o.off.gate_s_off % 16 == 0 && o.off.gate_b_off % 16 == 0 && o.off.up_s_off % 16 == 0 && o.off.up_b_off % 16 == 0;
        }
        st->decode_step_bulk_scales = bulk;
    }
    TF_CUDA(ctx, cudaMalloc(&st->device_layers, host.size() * sizeof(DecodeLayer)));
    TF_CUDA(ctx, cudaMemcpy(st->device_layers, host.data(), host.size() * sizeof(DecodeLayer), cudaMemcpyHostToDevice));
    return TF_OK;
}

tf_status launch_decode_step(tf_context* ctx, void* stream, tf_stack* st, void* hidden, tf_workspace* ws) {
    const char* name = "tf_stack_forward(one-token step)";
    const tf_moe_layer& a = st->layers[0];
    DecodeArgs args{};
    args.layers = static_cast<const DecodeLayer*>(st->device_layers);
    args.n_layers = (uint32_t)st->layers.size();
    args.d = a.d; args.f = a.f; args.fs = a.fs; args.E = a.num_experts; args.K = a.top_k; args.eps = st->eps;
    args.hidden = static_cast<uint16_t*>(hidden);
    args.logits = ctx->router_logits;
    args.acts = ws->acts; args.shared_act = ws->shared_act;
    args.out_idx = ws->indices; args.out_w = ws->weights;
    args.barrier = ctx->grid_barrier; args.error = ctx->device_error;
    args.trace = ctx->step_trace; args.trace_capacity = ctx->step_trace_capacity;
    args.bulk_scales = st->decode_step_bulk_scales ? 1u : 0u;
    const uint32_t smem = DsSmem(args.d, args.f, args.fs, args.E, args.K, (uint32_t)ctx->sm_count).total;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    static DeviceSmemCache configured;
    if (tf_status s = ensure_dynamic_smem(ctx, decode_step_kernel, configured, smem)) return s;
    TF_CUDA(ctx, cudaMemsetAsync(ctx->grid_barrier, 0, sizeof(uint32_t), cs));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctx->sm_count); cfg.blockDim = dim3(kDsThreads); cfg.dynamicSmemBytes = smem; cfg.stream = cs;
    // All CTAs must be resident at once. Outside a stream capture the launch is cooperative, which makes the
    // runtime check that; a captured launch relies on the grid being one CTA per SM, and every wait is bounded.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    TF_CUDA(ctx, cudaStreamIsCapturing(cs, &cap));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = cap == cudaStreamCaptureStatusNone ? 1 : 0;
    TF_CUDA(ctx, cudaLaunchKernelEx(&cfg, decode_step_kernel, args));
    return check_launch(ctx, name);
}

}  // namespace tf
