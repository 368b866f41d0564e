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
//   P2  every CTA selects the top-k from the 128 logits (same warp routine as the router kernels), then the
//       routed experts' gate/up rows, K * F row pairs split evenly over the CTAs               -> barrier 2
//   P3  down projections of the K routed experts and of the shared expert for the CTA's slice of output rows,
//       the weighted combine in rank order (Metal/MoE/moe.metal:473-480) and the residual add  -> barrier 3
//
// Weight rows are consumed straight from global memory by warps that own 16 rows x up to 4 column groups (the
// mma.sync GEMV building block of mma_gemv.cuh); a CTA's rows of a phase are cut into such items, partial sums meet
// in shared memory and are added in a fixed order, so the result does not depend on timing. Everything that does
// not depend on the router (next phase's rows, the next layer's router row and shared rows) is prefetched into L2
// while the current phase streams, so only the routed gate/up rows are waited for at DRAM latency.
//
// Rounding points are those of the per-kernel path: routed act = half(gelu(g) * u) with g, u in fp32
// (moe.metal:368); shared act = half(gelu(half(g)) * half(u)), shared y = half(down . act)
// (Kernels/MoE/SharedExpertInt4.swift:62-93); y = half(shared_y + sum_r w_r * partial_r); h = half(h + y).
//
// Grid barriers are bounded: a CTA that waits longer than kDsSpinLimit polls records kErrGridBarrier in the
// context's device error word, after which no barrier waits any more and the kernel runs to its end (with
// meaningless results); tf_device_status reports it.
#include <algorithm>

#include "block.cuh"
#include "mma_gemv.cuh"
#include "router.cuh"

namespace tf {

constexpr int kDsThreads = 512;
constexpr int kDsWarps = kDsThreads / kWarp;
constexpr uint32_t kDsMaxItems = 192;            // items of one phase in one CTA
constexpr uint32_t kDsSpinLimit = 1u << 22;      // x ~0.5 us per poll
constexpr uint32_t kErrGridBarrier = 0x7F000021u;
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
};

// ---------------------------------------------------------------------------
// grid barrier
// ---------------------------------------------------------------------------
struct GridSync {
    uint32_t* counter; uint32_t* error; uint32_t target; bool dead;
};

__device__ __forceinline__ void grid_sync(GridSync& gs) {
    __syncthreads();
    if (threadIdx.x == 0) {
        gs.target += gridDim.x;
        __threadfence();
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(gs.counter) : "memory");
        if (!gs.dead) {
            uint32_t spins = 0;
            for (;;) {
                uint32_t v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(gs.counter) : "memory");
                if ((int32_t)(v - gs.target) >= 0) break;
                if (++spins > kDsSpinLimit) { atomicCAS(gs.error, 0u, kErrGridBarrier); gs.dead = true; break; }
                if ((spins & 1023u) == 0u && *reinterpret_cast<volatile uint32_t*>(gs.error) != 0u) { gs.dead = true; break; }
            }
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
    const uint8_t* b = static_cast<const uint8_t*>(p);
    const uintptr_t first = reinterpret_cast<uintptr_t>(b) & ~(uintptr_t)127;
    const uintptr_t last = reinterpret_cast<uintptr_t>(b) + bytes;
    for (uintptr_t a = first + (uintptr_t)threadIdx.x * 128; a < last; a += (uintptr_t)kDsThreads * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
}

// ---------------------------------------------------------------------------
// items: 16 rows (two independent 8-row halves) x up to 4 column groups of one matrix
// ---------------------------------------------------------------------------
struct ItemSrc {                                // where an item's operands come from (needed only to issue its loads)
    const uint8_t* w0; const uint8_t* w1;       // this lane's rows g and g + 8, at the item's first group, + 8 t
    const uint16_t* s0; const uint16_t* s1; const uint16_t* b0; const uint16_t* b1;   // at the item's first group
};
struct ItemUse {                                // what the arithmetic needs besides the loaded registers
    uint32_t frag_word;                         // word offset of the B fragments of the item's first group for this lane's t
    uint32_t group;                             // index of the first group in the group-sum array
    uint32_t ngr;                               // groups in the item (1...4)
};

template <bool VEC>
struct ItemRegs {
    uint2 wa[4], wb[4];
    uint2 vs0, vs1, vb0, vb1;                   // VEC: scale / bias of four groups per row
    uint16_t ss0[4], ss1[4], sb0[4], sb1[4];    // !VEC
};

template <bool VEC>
__device__ __forceinline__ void item_load(const ItemSrc& it, uint32_t ngr, ItemRegs<VEC>& r) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if ((uint32_t)i < ngr) { r.wa[i] = gm_ldg64(it.w0 + i * 32); r.wb[i] = gm_ldg64(it.w1 + i * 32); }
        else { r.wa[i] = make_uint2(0u, 0u); r.wb[i] = make_uint2(0u, 0u); }
    }
    if constexpr (VEC) {
        r.vs0 = __ldg(reinterpret_cast<const uint2*>(it.s0)); r.vs1 = __ldg(reinterpret_cast<const uint2*>(it.s1));
        r.vb0 = __ldg(reinterpret_cast<const uint2*>(it.b0)); r.vb1 = __ldg(reinterpret_cast<const uint2*>(it.b1));
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const bool ok = (uint32_t)i < ngr;
            r.ss0[i] = ok ? __ldg(it.s0 + i) : (uint16_t)0; r.ss1[i] = ok ? __ldg(it.s1 + i) : (uint16_t)0;
            r.sb0[i] = ok ? __ldg(it.b0 + i) : (uint16_t)0; r.sb1[i] = ok ? __ldg(it.b1 + i) : (uint16_t)0;
        }
    }
}

// Returns the item's partial sums of rows g (x) and g + 8 (y); valid in the lanes with t == 0.
template <bool VEC>
__device__ __forceinline__ float2 item_compute(const ItemUse& it, const ItemRegs<VEC>& r, const uint32_t* frag_base,
                                               const float* xsum_base, int g) {
    float zc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) asm volatile("mov.f32 %0, 0f00000000;" : "=f"(zc[j]));
    float c[4][4];
    const uint32_t* frag = frag_base + it.frag_word;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint2 bf = make_uint2(0u, 0u);
            if (g == 0 && (uint32_t)i < it.ngr) bf = *reinterpret_cast<const uint2*>(frag + i * 32 + j * 2);
            const uint32_t wx = (j < 2) ? r.wa[i].x : r.wa[i].y, wy = (j < 2) ? r.wb[i].x : r.wb[i].y;
            const uint32_t mask = (j & 1) ? 0x00F000F0u : 0x000F000Fu;
            const uint32_t a0 = wx & mask, a1 = wy & mask, a2 = (wx >> 8) & mask, a3 = (wy >> 8) & mask;
            if (j == 0) gm_mma(c[i], a0, a1, a2, a3, bf.x, bf.y, zc);
            else gm_mma(c[i], a0, a1, a2, a3, bf.x, bf.y, c[i]);
        }
    }
    float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if ((uint32_t)i < it.ngr) {
            uint16_t s0b, s1b, b0b, b1b;
            if constexpr (VEC) {
                const uint32_t sv0 = i < 2 ? r.vs0.x : r.vs0.y, sv1 = i < 2 ? r.vs1.x : r.vs1.y;
                const uint32_t bv0 = i < 2 ? r.vb0.x : r.vb0.y, bv1 = i < 2 ? r.vb1.x : r.vb1.y;
                s0b = (uint16_t)((i & 1) ? sv0 >> 16 : sv0 & 0xFFFFu); s1b = (uint16_t)((i & 1) ? sv1 >> 16 : sv1 & 0xFFFFu);
                b0b = (uint16_t)((i & 1) ? bv0 >> 16 : bv0 & 0xFFFFu); b1b = (uint16_t)((i & 1) ? bv1 >> 16 : bv1 & 0xFFFFu);
            } else {
                s0b = r.ss0[i]; s1b = r.ss1[i]; b0b = r.sb0[i]; b1b = r.sb1[i];
            }
            // the codes entered the MMA as q * 2^-24: fold 2^24 into the scale
            const float s0 = bf16_bits_to_float(s0b) * 16777216.0f, s1 = bf16_bits_to_float(s1b) * 16777216.0f;
            const float xs = xsum_base[it.group + i];
            acc0 = fmaf(s0, c[i][0], fmaf(bf16_bits_to_float(b0b), xs, acc0));
            acc1 = fmaf(s1, c[i][2], fmaf(bf16_bits_to_float(b1b), xs, acc1));
        }
    }
    return make_float2(acc0, acc1);
}

// Runs items first, first + step, ... < n_items on this warp; `make` fills the source and use records of an item for
// this lane. The next item's loads are issued before the current item is computed.
template <bool VEC, typename Make>
__device__ __forceinline__ void run_items(uint32_t first, uint32_t step, uint32_t n_items, float* partial,
                                          const uint32_t* frag_base, const float* xsum_base, int lane, Make make) {
    const int g = lane >> 2, t = lane & 3;
    if (first >= n_items) return;
    ItemUse cur_u, nxt_u;
    ItemRegs<VEC> cur_r, nxt_r;
    {
        ItemSrc src;
        make(first, g, t, src, cur_u);
        item_load<VEC>(src, cur_u.ngr, cur_r);
    }
    for (uint32_t it = first; it < n_items; it += step) {
        const bool more = it + step < n_items;
        if (more) {
            ItemSrc src;
            make(it + step, g, t, src, nxt_u);
            item_load<VEC>(src, nxt_u.ngr, nxt_r);
        }
        const float2 v = item_compute<VEC>(cur_u, cur_r, frag_base, xsum_base, g);
        if (t == 0) { partial[it * 16 + g] = v.x; partial[it * 16 + g + 8] = v.y; }
        if (more) { cur_u = nxt_u; cur_r = nxt_r; }
    }
}

// B fragments and group sums of an fp16 vector that sits in shared memory (16-byte aligned, n = 64 ng).
__device__ __forceinline__ void stage_frags(const uint16_t* xs, uint32_t ng, uint32_t* frag, float* xsum) {
    for (uint32_t idx = threadIdx.x; idx < ((ng * 4 + 31u) & ~31u); idx += kDsThreads) {     // whole warps: shuffles below
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

__host__ __device__ inline uint32_t ds_split(uint32_t total, uint32_t part, uint32_t parts) {
    return (uint32_t)(((uint64_t)total * part) / parts);
}
__host__ __device__ inline uint32_t ds_kparts(uint32_t ng) { return (ng + 3u) / 4u; }

struct DsSmem {
    uint32_t x16, xf, frag_a, sum_a, a16, frag_b, sum_b, wrow, partial, scores, sel_idx, sel_w, red, total;
    __host__ __device__ DsSmem(uint32_t d, uint32_t f, uint32_t fs, uint32_t E, uint32_t K) {
        auto up = [](uint32_t v) { return (v + 15u) & ~15u; };
        const uint32_t ngd = d / 64, ngb = K * (f / 64) + fs / 64;
        uint32_t o = 0;
        x16 = o; o += up(d * 2);
        xf = o; o += up(d * 4);
        frag_a = o; o += ngd * 128;
        sum_a = o; o += up(ngd * 4);
        a16 = o; o += up((K * f + fs) * 2);
        frag_b = o; o += ngb * 128;
        sum_b = o; o += up(ngb * 4);
        wrow = o; o += up(d) + up(ngd * 2) * 2;
        partial = o; o += kDsMaxItems * 64;
        scores = o; o += up(E * 4);
        sel_idx = o; o += 32;
        sel_w = o; o += 16;
        red = o; o += 16;
        total = o;
    }
};

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
// Per-CTA constants of the launch, kept in shared memory so that the phase functions (compiled as separate
// functions: each gets its own register allocation) read what they need instead of carrying it in registers.
struct DsCtx {
    uint32_t d, f, fs, E, K, ngd, ngf, ngs, kp_d, kp_f, kp_s;
    uint32_t p1_lo, p1_hi, p2_lo, p2_hi, p3_lo, p3_hi, p1_tiles, p2_tiles, p3_tiles, p3_per_tile;
    uint32_t cta, grid;
    uint16_t* x16; float* xf; uint32_t* frag_a; float* sum_a; uint16_t* a16; uint32_t* frag_b; float* sum_b;
    uint8_t* wrow; uint16_t* srow; uint16_t* brow; float* partial; float* scores; uint32_t* sel_idx; uint16_t* sel_w; float* red;
    uint16_t* hidden; float* logits; uint16_t* acts; uint16_t* shared_act; uint32_t* out_idx; uint16_t* out_w;
    float eps;
};

// P0: x = half(rmsnorm(h) * w) into shared memory (bits of residual_rmsnorm_kernel: same thread striding and
// reduction tree), its B fragments, and the router's fp32 operand x * effective_scale.
__device__ __noinline__ void ds_phase0(const DsCtx* c, const DecodeLayer* L) {
    const uint32_t d = c->d, vecs = d / 8;
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    float v[kDsNormSlices][8];
    float acc = 0.0f;
    if (threadIdx.x < kDsNormThreads) {
#pragma unroll
        for (int s = 0; s < kDsNormSlices; ++s) {
            const uint32_t i = threadIdx.x + s * kDsNormThreads;
            if (i < vecs) {
                const uint4 hv = __ldcg(reinterpret_cast<const uint4*>(c->hidden) + i);
                const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
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
    __syncthreads();
    if (threadIdx.x < kDsNormThreads) {
        float tot = lane < kDsNormThreads / kWarp ? c->red[lane] : 0.0f;
        tot = warp_sum(tot);
        const float inv = rsqrtf(tot / (float)d + c->eps);
        const uint16_t* nw = L->norm_w;
#pragma unroll
        for (int s = 0; s < kDsNormSlices; ++s) {
            const uint32_t i = threadIdx.x + s * kDsNormThreads;
            if (i < vecs) {
                const uint4 wv = __ldg(reinterpret_cast<const uint4*>(nw) + i);
                const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
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
    __syncthreads();
    stage_frags(c->x16, c->ngd, c->frag_a, c->sum_a);
    const uint16_t* eff = L->eff;
    for (uint32_t i = threadIdx.x; i < d; i += kDsThreads)
        c->xf[i] = __fmul_rn(f16_bits_to_float(c->x16[i]), bf16_bits_to_float(eff[i]));
    __syncthreads();
}

// P1: this CTA's router rows (canonical logit) and its slice of the shared expert's gate/up rows.
__device__ __noinline__ void ds_phase1(const DsCtx* c, const DecodeLayer* L) {
    const uint32_t d = c->d, ngd = c->ngd, kp_d = c->kp_d;
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    for (uint32_t e = c->cta; e < c->E; e += c->grid) {
        const uint8_t* wsrc = L->router_w + (size_t)e * d;
        if ((reinterpret_cast<uintptr_t>(wsrc) & 15) == 0) {
            for (uint32_t i = threadIdx.x; i < d / 16; i += kDsThreads) reinterpret_cast<uint4*>(c->wrow)[i] = ldg_nc_u4(wsrc + (size_t)i * 16);
        } else {
            for (uint32_t i = threadIdx.x; i < d; i += kDsThreads) c->wrow[i] = wsrc[i];
        }
        for (uint32_t i = threadIdx.x; i < ngd; i += kDsThreads) {
            c->srow[i] = L->router_s[(size_t)e * ngd + i];
            c->brow[i] = L->router_b[(size_t)e * ngd + i];
        }
        __syncthreads();
        if (warp == 0) {
            float logit = router_row_logit_smem(c->wrow, c->srow, c->brow, c->xf, ngd, lane);
            if (L->logit_bias) logit = __fadd_rn(logit, L->logit_bias[e]);
            if (lane == 0) c->logits[e] = logit;
        }
        __syncthreads();
    }
    const uint32_t lo = c->p1_lo, hi = c->p1_hi;
    const uint32_t n_items = c->p1_tiles * 2 * kp_d;
    const uint8_t* Wg = L->sg_w; const uint8_t* Wu = L->su_w;
    const uint16_t* Sg = L->sg_s; const uint16_t* Su = L->su_s; const uint16_t* Bg = L->sg_b; const uint16_t* Bu = L->su_b;
    const bool vec = (ngd % 4 == 0) && ((reinterpret_cast<uintptr_t>(Sg) | reinterpret_cast<uintptr_t>(Bg) |
                                           reinterpret_cast<uintptr_t>(Su) | reinterpret_cast<uintptr_t>(Bu)) & 7) == 0;
    auto make = [&](uint32_t it, int g, int t, ItemSrc& o, ItemUse& u) {
        const uint32_t tile = it / (2 * kp_d), rem = it % (2 * kp_d), mat = rem / kp_d, kp = rem % kp_d;
        const uint32_t G0 = kp * 4;
        uint32_t r0 = lo + tile * 16 + g, r1 = r0 + 8;
        r0 = r0 < hi ? r0 : hi - 1; r1 = r1 < hi ? r1 : hi - 1;
        const uint8_t* W = mat ? Wu : Wg;
        const uint16_t* S = mat ? Su : Sg;
        const uint16_t* B = mat ? Bu : Bg;
        o.w0 = W + (size_t)r0 * (d / 2) + G0 * 32 + t * 8; o.w1 = W + (size_t)r1 * (d / 2) + G0 * 32 + t * 8;
        o.s0 = S + (size_t)r0 * ngd + G0; o.s1 = S + (size_t)r1 * ngd + G0;
        o.b0 = B + (size_t)r0 * ngd + G0; o.b1 = B + (size_t)r1 * ngd + G0;
        u.frag_word = (G0 * 4 + t) * 8; u.group = G0;
        u.ngr = ngd - G0 < 4u ? ngd - G0 : 4u;
    };
    if (vec) run_items<true>(warp, kDsWarps, n_items, c->partial, c->frag_a, c->sum_a, lane, make);
    else run_items<false>(warp, kDsWarps, n_items, c->partial, c->frag_a, c->sum_a, lane, make);
    __syncthreads();
    const float* partial = c->partial;
    for (uint32_t j = threadIdx.x; j < hi - lo; j += kDsThreads) {
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
__device__ __noinline__ void ds_phase2(const DsCtx* c, const DecodeLayer* L, const DecodeLayer* N) {
    const uint32_t d = c->d, f = c->f, fs = c->fs, E = c->E, K = c->K, ngd = c->ngd, ngf = c->ngf, ngs = c->ngs, kp_d = c->kp_d;
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    for (uint32_t i = threadIdx.x; i < E; i += kDsThreads) c->scores[i] = __ldcg(c->logits + i);
    __syncthreads();
    if (warp == 0) warp_select_topk(c->scores, E, K, L->pes, c->sel_idx, c->sel_w, lane);
    __syncthreads();
    if (threadIdx.x < K) {
        uint32_t e = c->sel_idx[threadIdx.x];
        if (c->cta == 0) { c->out_idx[threadIdx.x] = e; c->out_w[threadIdx.x] = c->sel_w[threadIdx.x]; }
        if (e >= E) e = E - 1;                        // min(id, E-1): Runtime/Inference/RealForwardRunner.swift:1486
        c->sel_idx[threadIdx.x] = e;
    }
    __syncthreads();
    const uint32_t lo = c->p2_lo, hi = c->p2_hi;
    const uint32_t n_items = c->p2_tiles * 2 * kp_d;
    const uint8_t* pool = L->pool;
    const uint64_t stride = L->stride;
    const tf_expert_offsets off = L->off;
    const uint32_t* sel = c->sel_idx;
    const bool vec = (ngd % 4 == 0) && ((reinterpret_cast<uintptr_t>(pool) | stride | off.gate_s_off | off.gate_b_off |
                                           off.up_s_off | off.up_b_off) & 7) == 0;
    auto make = [&](uint32_t it, int g, int t, ItemSrc& o, ItemUse& u) {
        const uint32_t tile = it / (2 * kp_d), rem = it % (2 * kp_d), mat = rem / kp_d, kp = rem % kp_d;
        const uint32_t G0 = kp * 4;
        uint32_t i0 = lo + tile * 16 + g, i1 = i0 + 8;
        i0 = i0 < hi ? i0 : hi - 1; i1 = i1 < hi ? i1 : hi - 1;
        const uint8_t* blob0 = pool + (uint64_t)sel[i0 / f] * stride;
        const uint8_t* blob1 = pool + (uint64_t)sel[i1 / f] * stride;
        const uint32_t r0 = i0 % f, r1 = i1 % f;
        const uint32_t wo = mat ? off.up_w_off : off.gate_w_off, so = mat ? off.up_s_off : off.gate_s_off,
                       bo = mat ? off.up_b_off : off.gate_b_off;
        o.w0 = blob0 + wo + (size_t)r0 * (d / 2) + G0 * 32 + t * 8; o.w1 = blob1 + wo + (size_t)r1 * (d / 2) + G0 * 32 + t * 8;
        o.s0 = reinterpret_cast<const uint16_t*>(blob0 + so) + (size_t)r0 * ngd + G0;
        o.s1 = reinterpret_cast<const uint16_t*>(blob1 + so) + (size_t)r1 * ngd + G0;
        o.b0 = reinterpret_cast<const uint16_t*>(blob0 + bo) + (size_t)r0 * ngd + G0;
        o.b1 = reinterpret_cast<const uint16_t*>(blob1 + bo) + (size_t)r1 * ngd + G0;
        u.frag_word = (G0 * 4 + t) * 8; u.group = G0;
        u.ngr = ngd - G0 < 4u ? ngd - G0 : 4u;
    };
    if (vec) run_items<true>(warp, kDsWarps, n_items, c->partial, c->frag_a, c->sum_a, lane, make);
    else run_items<false>(warp, kDsWarps, n_items, c->partial, c->frag_a, c->sum_a, lane, make);
    // while the routed rows stream: bring this CTA's rows of P3 and of the next layer's P1 into L2
    const uint32_t lo3 = c->p3_lo, n3 = c->p3_hi - c->p3_lo;
    if (n3) {
        for (uint32_t k = 0; k < K; ++k) {
            const uint8_t* blob = pool + (uint64_t)sel[k] * stride;
            prefetch_l2(blob + off.down_w_off + (size_t)lo3 * (f / 2), n3 * (f / 2));
            prefetch_l2(blob + off.down_s_off + (size_t)lo3 * ngf * 2, n3 * ngf * 2);
            prefetch_l2(blob + off.down_b_off + (size_t)lo3 * ngf * 2, n3 * ngf * 2);
        }
        prefetch_l2(L->sd_w + (size_t)lo3 * (fs / 2), n3 * (fs / 2));
        prefetch_l2(L->sd_s + (size_t)lo3 * ngs, n3 * ngs * 2);
        prefetch_l2(L->sd_b + (size_t)lo3 * ngs, n3 * ngs * 2);
    }
    if (N) {
        for (uint32_t e = c->cta; e < E; e += c->grid) prefetch_l2(N->router_w + (size_t)e * d, d);
        const uint32_t lo1 = c->p1_lo, n1 = c->p1_hi - c->p1_lo;
        if (n1) {
            prefetch_l2(N->sg_w + (size_t)lo1 * (d / 2), n1 * (d / 2));
            prefetch_l2(N->su_w + (size_t)lo1 * (d / 2), n1 * (d / 2));
            prefetch_l2(N->sg_s + (size_t)lo1 * ngd, n1 * ngd * 2);
            prefetch_l2(N->sg_b + (size_t)lo1 * ngd, n1 * ngd * 2);
            prefetch_l2(N->su_s + (size_t)lo1 * ngd, n1 * ngd * 2);
            prefetch_l2(N->su_b + (size_t)lo1 * ngd, n1 * ngd * 2);
        }
    }
    __syncthreads();
    const float* partial = c->partial;
    for (uint32_t j = threadIdx.x; j < hi - lo; j += kDsThreads) {
        const uint32_t tile = j / 16, r = j % 16;
        float gt = 0.0f, up = 0.0f;
        for (uint32_t kp = 0; kp < kp_d; ++kp) {
            gt += partial[((tile * 2 + 0) * kp_d + kp) * 16 + r];
            up += partial[((tile * 2 + 1) * kp_d + kp) * 16 + r];
        }
        c->acts[lo + j] = __half_as_ushort(__float2half_rn(gelu_tanh(gt) * up));     // moe.metal:368
    }
}

// P3: down projections of the K routed experts and of the shared expert for this CTA's output rows, combine in rank
// order, residual add.
__device__ __noinline__ void ds_phase3(const DsCtx* c, const DecodeLayer* L) {
    const uint32_t f = c->f, fs = c->fs, K = c->K, ngf = c->ngf, ngs = c->ngs, kp_f = c->kp_f, kp_s = c->kp_s;
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t n_act = K * f + fs;
    for (uint32_t i = threadIdx.x; i < n_act / 8; i += kDsThreads) {
        const uint32_t e8 = i * 8;
        const uint16_t* src = e8 < K * f ? c->acts + e8 : c->shared_act + (e8 - K * f);
        reinterpret_cast<uint4*>(c->a16)[i] = __ldcg(reinterpret_cast<const uint4*>(src));
    }
    __syncthreads();
    stage_frags(c->a16, K * ngf + ngs, c->frag_b, c->sum_b);      // K routed vectors of ngf groups, then the shared one
    __syncthreads();
    const uint32_t lo = c->p3_lo, hi = c->p3_hi, per_tile = c->p3_per_tile;
    const uint32_t n_items = c->p3_tiles * per_tile;
    const uint8_t* pool = L->pool;
    const uint64_t stride = L->stride;
    const uint32_t dw = L->off.down_w_off, dso = L->off.down_s_off, dbo = L->off.down_b_off;
    const uint8_t* sdw = L->sd_w; const uint16_t* sds = L->sd_s; const uint16_t* sdb = L->sd_b;
    const uint32_t* sel = c->sel_idx;
    auto make = [&](uint32_t it, int g, int t, ItemSrc& o, ItemUse& u) {
        const uint32_t tile = it / per_tile, rem = it % per_tile;
        uint32_t r0 = lo + tile * 16 + g, r1 = r0 + 8;
        r0 = r0 < hi ? r0 : hi - 1; r1 = r1 < hi ? r1 : hi - 1;
        if (rem < K * kp_f) {
            const uint32_t k = rem / kp_f, G0 = (rem % kp_f) * 4;
            const uint8_t* blob = pool + (uint64_t)sel[k] * stride;
            const uint16_t* S = reinterpret_cast<const uint16_t*>(blob + dso);
            const uint16_t* B = reinterpret_cast<const uint16_t*>(blob + dbo);
            o.w0 = blob + dw + (size_t)r0 * (f / 2) + G0 * 32 + t * 8;
            o.w1 = blob + dw + (size_t)r1 * (f / 2) + G0 * 32 + t * 8;
            o.s0 = S + (size_t)r0 * ngf + G0; o.s1 = S + (size_t)r1 * ngf + G0;
            o.b0 = B + (size_t)r0 * ngf + G0; o.b1 = B + (size_t)r1 * ngf + G0;
            u.frag_word = ((k * ngf + G0) * 4 + t) * 8; u.group = k * ngf + G0;
            u.ngr = ngf - G0 < 4u ? ngf - G0 : 4u;
        } else {
            const uint32_t G0 = (rem - K * kp_f) * 4;
            o.w0 = sdw + (size_t)r0 * (fs / 2) + G0 * 32 + t * 8; o.w1 = sdw + (size_t)r1 * (fs / 2) + G0 * 32 + t * 8;
            o.s0 = sds + (size_t)r0 * ngs + G0; o.s1 = sds + (size_t)r1 * ngs + G0;
            o.b0 = sdb + (size_t)r0 * ngs + G0; o.b1 = sdb + (size_t)r1 * ngs + G0;
            u.frag_word = ((K * ngf + G0) * 4 + t) * 8; u.group = K * ngf + G0;
            u.ngr = ngs - G0 < 4u ? ngs - G0 : 4u;
        }
    };
    run_items<false>(warp, kDsWarps, n_items, c->partial, c->frag_b, c->sum_b, lane, make);
    __syncthreads();
    const float* partial = c->partial;
    for (uint32_t j = threadIdx.x; j < hi - lo; j += kDsThreads) {
        const uint32_t tile = j / 16, r = j % 16;
        const float* pt = partial + (size_t)tile * per_tile * 16 + r;
        float sh = 0.0f;
        for (uint32_t kp = 0; kp < kp_s; ++kp) sh += pt[(K * kp_f + kp) * 16];
        float acc = __half2float(__float2half_rn(sh));                 // shared y is stored as fp16
        for (uint32_t k = 0; k < K; ++k) {
            float pk = 0.0f;
            for (uint32_t kp = 0; kp < kp_f; ++kp) pk += pt[(k * kp_f + kp) * 16];
            acc = __fadd_rn(acc, __fmul_rn(f16_bits_to_float(c->sel_w[k]), pk));      // rank order 0..K-1
        }
        const float y = __half2float(__float2half_rn(acc));
        const float h = f16_bits_to_float(__ldcg(c->hidden + lo + j));
        c->hidden[lo + j] = __half_as_ushort(__float2half_rn(h + y));
    }
}

__global__ void __launch_bounds__(kDsThreads, 1)
decode_step_kernel(const DecodeArgs args) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ DsCtx ctx;
    if (threadIdx.x == 0) {
        const uint32_t d = args.d, f = args.f, fs = args.fs, E = args.E, K = args.K;
        const DsSmem lay(d, f, fs, E, K);
        DsCtx& c = ctx;
        c.d = d; c.f = f; c.fs = fs; c.E = E; c.K = K;
        c.ngd = d / kGroup; c.ngf = f / kGroup; c.ngs = fs / kGroup;
        c.kp_d = ds_kparts(c.ngd); c.kp_f = ds_kparts(c.ngf); c.kp_s = ds_kparts(c.ngs);
        c.cta = blockIdx.x; c.grid = gridDim.x;
        c.p1_lo = ds_split(fs, c.cta, c.grid); c.p1_hi = ds_split(fs, c.cta + 1, c.grid);
        c.p2_lo = ds_split(K * f, c.cta, c.grid); c.p2_hi = ds_split(K * f, c.cta + 1, c.grid);
        c.p3_lo = ds_split(d, c.cta, c.grid); c.p3_hi = ds_split(d, c.cta + 1, c.grid);
        c.p1_tiles = (c.p1_hi - c.p1_lo + 15) / 16; c.p2_tiles = (c.p2_hi - c.p2_lo + 15) / 16; c.p3_tiles = (c.p3_hi - c.p3_lo + 15) / 16;
        c.p3_per_tile = K * c.kp_f + c.kp_s;
        c.x16 = reinterpret_cast<uint16_t*>(smem + lay.x16);
        c.xf = reinterpret_cast<float*>(smem + lay.xf);
        c.frag_a = reinterpret_cast<uint32_t*>(smem + lay.frag_a);
        c.sum_a = reinterpret_cast<float*>(smem + lay.sum_a);
        c.a16 = reinterpret_cast<uint16_t*>(smem + lay.a16);
        c.frag_b = reinterpret_cast<uint32_t*>(smem + lay.frag_b);
        c.sum_b = reinterpret_cast<float*>(smem + lay.sum_b);
        c.wrow = smem + lay.wrow;
        c.srow = reinterpret_cast<uint16_t*>(c.wrow + ((d + 15u) & ~15u));
        c.brow = c.srow + ((c.ngd * 2 + 15u) & ~15u) / 2;
        c.partial = reinterpret_cast<float*>(smem + lay.partial);
        c.scores = reinterpret_cast<float*>(smem + lay.scores);
        c.sel_idx = reinterpret_cast<uint32_t*>(smem + lay.sel_idx);
        c.sel_w = reinterpret_cast<uint16_t*>(smem + lay.sel_w);
        c.red = reinterpret_cast<float*>(smem + lay.red);
        c.hidden = args.hidden; c.logits = args.logits; c.acts = args.acts; c.shared_act = args.shared_act;
        c.out_idx = args.out_idx; c.out_w = args.out_w; c.eps = args.eps;
    }
    __syncthreads();
    GridSync gs{args.barrier, args.error, 0u, false};
    uint32_t stamp_at = 0;
    auto stamp = [&]() {
        if (args.trace && blockIdx.x == 0 && threadIdx.x == 0 && stamp_at < args.trace_capacity) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            args.trace[stamp_at++] = t;
        }
    };
    for (uint32_t l = 0; l < args.n_layers; ++l) {
        const DecodeLayer* L = args.layers + l;
        stamp();
        ds_phase0(&ctx, L);
        stamp();
        ds_phase1(&ctx, L);
        stamp();
        grid_sync(gs);
        stamp();
        ds_phase2(&ctx, L, l + 1 < args.n_layers ? L + 1 : nullptr);
        stamp();
        grid_sync(gs);
        stamp();
        ds_phase3(&ctx, L);
        stamp();
        grid_sync(gs);
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
        const uint32_t t1 = (ds_split(fs, c + 1, grid) - ds_split(fs, c, grid) + 15) / 16;
        const uint32_t t2 = (ds_split(K * f, c + 1, grid) - ds_split(K * f, c, grid) + 15) / 16;
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
    if (DsSmem(d, f, fs, E, K).total > 200u * 1024u) return false;
    return st->decode_step_ok;
}

tf_status decode_step_prepare(tf_context* ctx, tf_stack* st) {
    // one device copy of the per-layer pointers; alignment rules of the item loads (8-byte code loads, 2-byte planes)
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
        ok = ok && m.router.rows == m.num_experts && m.router.cols == m.d;
        ok = ok && m.shared_gate.rows == m.fs && m.shared_gate.cols == m.d && m.shared_up.rows == m.fs && m.shared_up.cols == m.d &&
             m.shared_down.rows == m.d && m.shared_down.cols == m.fs;
        ok = ok && aligned(o.pool, 8) && o.stride % 8 == 0 && o.off.gate_w_off % 8 == 0 && o.off.up_w_off % 8 == 0 && o.off.down_w_off % 8 == 0;
        ok = ok && aligned(o.sg_w, 8) && aligned(o.su_w, 8) && aligned(o.sd_w, 8) && aligned(o.norm_w, 16);
        const uint32_t sb[6] = {o.off.gate_s_off, o.off.gate_b_off, o.off.up_s_off, o.off.up_b_off, o.off.down_s_off, o.off.down_b_off};
        for (uint32_t v : sb) ok = ok && v % 2 == 0;
        ok = ok && aligned(o.sg_s, 2) && aligned(o.sg_b, 2) && aligned(o.su_s, 2) && aligned(o.su_b, 2) && aligned(o.sd_s, 2) &&
             aligned(o.sd_b, 2) && aligned(o.router_s, 2) && aligned(o.router_b, 2) && aligned(o.eff, 2) && aligned(o.pes, 2);
    }
    st->decode_step_ok = ok;
    if (!ok) return TF_OK;
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
    const uint32_t smem = DsSmem(args.d, args.f, args.fs, args.E, args.K).total;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    {
        static std::mutex mu;
        static uint32_t configured[64] = {0};
        std::lock_guard<std::mutex> lock(mu);
        const int dev = ctx->device < 64 ? ctx->device : 63;
        if (smem > configured[dev] || ctx->device >= 64) {
            TF_CUDA(ctx, cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            int per_sm = 0;
            TF_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, kDsThreads, smem));
            TF_REQUIRE(ctx, per_sm >= 1, TF_ERR_UNSUPPORTED, "%s: the kernel does not fit an SM with %u bytes of shared memory", name, smem);
            configured[dev] = smem;
        }
    }
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
