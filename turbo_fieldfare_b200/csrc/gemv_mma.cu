// Streaming int4 GEMV for large matrices: y[m] = deq4(W[m,n]) . x[n] at HBM speed.
// Second implementation of dequant_int4_gemv_simd (Metal/Quant/dequant_int4.metal:93-191) for the sizes where
// the warp-per-row kernel of gemv.cu is bound by its instruction count (about three CUDA-core instructions per
// weight: extract, convert, multiply-add), e.g. the LM-head-sized instance 262144 x 2816.
//
// Here a weight costs half an instruction. Each warp owns 16 rows and walks the columns in 64-column groups;
// per group it loads 8 bytes of packed codes per lane for rows g and g + 8 straight from global memory (every
// 32-byte sector fully used), masks them into fp16 subnormals (q * 2^-24, or q * 2^-20 against activations
// pre-scaled by 1/16: one AND per two codes) and feeds them as the A operand of mma.sync.m16n8k16. The vector x
// is column 0 of the B operand (the other seven columns are zero), pre-arranged once per block in shared
// memory in fragment order. Scale and bias are applied per group to the fp32 accumulator, acc += s * (q . x)
// + b * sum(x), the reference's algebra (dequant_int4.metal:132-170). Four groups are in flight as
// independent MMA chains, and the next four groups' codes are loaded before the current ones are consumed.
#include "mma_gemv.cuh"

namespace tf {

constexpr int kGmWarps = 8;                 // 16 rows each: 128 rows per block (one large matrix)
constexpr int kGmBatchWarps = 4;            // 64 rows per block for batches of expert-sized matrices (704 = 11 x 64)
constexpr int kGmBlockGroups = 4;           // groups per inner step (independent MMA chains)

// Shared memory: B fragments of x [ng][4 lanes t][8 words], group sums [ng], scale and bias planes of the block's
// 128 rows [128][ng] each.
// A batch (blockIdx.y) walks matrices that share one layout: matrix b has its three planes `plane_stride` bytes
// after those of matrix b - 1 (e.g. the same tensor of consecutive expert blobs), its activations x_stride and its
// results y_stride elements further on (x_stride 0: one vector for all).
struct GemvBatch {
    uint64_t plane_stride;
    uint32_t x_stride, y_stride;
};

template <bool SB_FP16, bool OUT_F32, int WARPS>
__global__ void __launch_bounds__(WARPS * kWarp)
gemv_mma_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ S, const uint16_t* __restrict__ B,
                const uint16_t* __restrict__ x, void* __restrict__ y, uint32_t m, uint32_t n, const GemvBatch bt) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int kGmRows = WARPS * 16, kGmThreads = WARPS * kWarp;
    {
        const size_t b = blockIdx.y;
        W += b * bt.plane_stride;
        S = reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(S) + b * bt.plane_stride);
        B = reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(B) + b * bt.plane_stride);
        x += b * bt.x_stride;
        y = static_cast<uint8_t*>(y) + b * bt.y_stride * (OUT_F32 ? 4 : 2);
    }
    const uint32_t ng = n / kGroup;
    uint32_t* xfrag = reinterpret_cast<uint32_t*>(smem);                       // ng * 32 words
    float* xsum = reinterpret_cast<float*>(smem + (size_t)ng * 128);           // ng floats
    uint16_t* sS = reinterpret_cast<uint16_t*>(smem + (size_t)ng * 132);       // 128 * ng
    uint16_t* sB = sS + (size_t)kGmRows * ng;
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t row_base = blockIdx.x * kGmRows;

    // ---- stage x in MMA operand order: the 16 values x0..x15 at columns 64 G + 16 t feed four MMAs,
    //   j = 0: (x0,x4),(x2,x6)   j = 1: (x1,x5)/16,(x3,x7)/16   j = 2, 3: the same for x8..x15
    // (odd columns are pre-scaled by 1/16 because their codes sit four mantissa bits higher) ----
    for (uint32_t idx = threadIdx.x; idx < ((ng * 4 + 31u) & ~31u); idx += kGmThreads) {   // whole warps: the sums use shuffles
        const bool ok = idx < ng * 4;
        const uint32_t G = idx >> 2, tt = idx & 3;
        const uint4* p = reinterpret_cast<const uint4*>(x + G * kGroup + tt * 16);
        uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
        if (ok) { lo = __ldg(p); hi = __ldg(p + 1); }
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
        if (tt == 0) xsum[G] = sum;
        uint32_t* f = xfrag + idx * 8;
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const int o = 4 * h2;
            f[4 * h2 + 0] = gm_prmt(r[o], r[o + 2], 0x5410);
            f[4 * h2 + 1] = gm_prmt(r[o + 1], r[o + 3], 0x5410);
            f[4 * h2 + 2] = gm_sixteenth(gm_prmt(r[o], r[o + 2], 0x7632));
            f[4 * h2 + 3] = gm_sixteenth(gm_prmt(r[o + 1], r[o + 3], 0x7632));
        }
    }
    // ---- scale and bias planes of the block's rows (contiguous in global memory) ----
    {
        const uint32_t rows_here = m - row_base < (uint32_t)kGmRows ? m - row_base : (uint32_t)kGmRows;
        const uint32_t words = rows_here * ng / 2;                             // rows * ng is even (ng % 4 == 0)
        const uint32_t* gs = reinterpret_cast<const uint32_t*>(S + (size_t)row_base * ng);
        const uint32_t* gb = reinterpret_cast<const uint32_t*>(B + (size_t)row_base * ng);
        uint32_t* ds = reinterpret_cast<uint32_t*>(sS);
        uint32_t* db = reinterpret_cast<uint32_t*>(sB);
        for (uint32_t i = threadIdx.x; i < words; i += kGmThreads) { ds[i] = __ldg(gs + i); db[i] = __ldg(gb + i); }
    }
    __syncthreads();

    const uint32_t r0 = row_base + warp * 16 + g, r1 = r0 + 8;
    const uint32_t row_bytes = n / 2;
    // rows past the matrix read the last row (their results are not stored)
    const uint8_t* W0 = W + (size_t)(r0 < m ? r0 : m - 1) * row_bytes + t * 8;
    const uint8_t* W1 = W + (size_t)(r1 < m ? r1 : m - 1) * row_bytes + t * 8;
    const uint16_t* s0p = sS + (size_t)(warp * 16 + g) * ng;
    const uint16_t* s1p = s0p + 8 * ng;
    const uint16_t* b0p = sB + (size_t)(warp * 16 + g) * ng;
    const uint16_t* b1p = b0p + 8 * ng;
    float zc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) asm volatile("mov.f32 %0, 0f00000000;" : "=f"(zc[j]));

    float acc0 = 0.0f, acc1 = 0.0f;
    uint2 wa[kGmBlockGroups], wb[kGmBlockGroups];
#pragma unroll
    for (int i = 0; i < kGmBlockGroups; ++i) { wa[i] = gm_ldg64(W0 + i * 32); wb[i] = gm_ldg64(W1 + i * 32); }
    for (uint32_t G0 = 0; G0 < ng; G0 += kGmBlockGroups) {
        uint2 ca[kGmBlockGroups], cb[kGmBlockGroups];
#pragma unroll
        for (int i = 0; i < kGmBlockGroups; ++i) { ca[i] = wa[i]; cb[i] = wb[i]; }
        if (G0 + kGmBlockGroups < ng) {
#pragma unroll
            for (int i = 0; i < kGmBlockGroups; ++i) {
                wa[i] = gm_ldg64(W0 + (G0 + kGmBlockGroups + i) * 32);
                wb[i] = gm_ldg64(W1 + (G0 + kGmBlockGroups + i) * 32);
            }
        }
        float c[kGmBlockGroups][4];
        const uint32_t* fr = xfrag + (G0 * 4 + t) * 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int i = 0; i < kGmBlockGroups; ++i) {
                // B fragment of MMA j of group G0 + i: x lives in column 0 only (lanes with g == 0)
                uint2 bf = make_uint2(0u, 0u);
                if (g == 0) bf = *reinterpret_cast<const uint2*>(fr + i * 32 + j * 2);
                const uint32_t wx = (j < 2) ? ca[i].x : ca[i].y, wy = (j < 2) ? cb[i].x : cb[i].y;
                const uint32_t mask = (j & 1) ? 0x00F000F0u : 0x000F000Fu;
                const uint32_t a0 = wx & mask, a1 = wy & mask, a2 = (wx >> 8) & mask, a3 = (wy >> 8) & mask;
                if (j == 0) gm_mma(c[i], a0, a1, a2, a3, bf.x, bf.y, zc);
                else gm_mma(c[i], a0, a1, a2, a3, bf.x, bf.y, c[i]);
            }
        }
        // scale and bias of the four groups for rows g and g + 8 (8-byte aligned: ng % 4 == 0)
        const uint2 vs0 = *reinterpret_cast<const uint2*>(s0p + G0), vs1 = *reinterpret_cast<const uint2*>(s1p + G0);
        const uint2 vb0 = *reinterpret_cast<const uint2*>(b0p + G0), vb1 = *reinterpret_cast<const uint2*>(b1p + G0);
        const float4 xs = *reinterpret_cast<const float4*>(xsum + G0);
        const float xsv[4] = {xs.x, xs.y, xs.z, xs.w};
#pragma unroll
        for (int i = 0; i < kGmBlockGroups; ++i) {
            const uint32_t sv0 = i < 2 ? vs0.x : vs0.y, sv1 = i < 2 ? vs1.x : vs1.y;
            const uint32_t bv0 = i < 2 ? vb0.x : vb0.y, bv1 = i < 2 ? vb1.x : vb1.y;
            const uint16_t s0b = (uint16_t)((i & 1) ? sv0 >> 16 : sv0 & 0xFFFFu), s1b = (uint16_t)((i & 1) ? sv1 >> 16 : sv1 & 0xFFFFu);
            const uint16_t b0b = (uint16_t)((i & 1) ? bv0 >> 16 : bv0 & 0xFFFFu), b1b = (uint16_t)((i & 1) ? bv1 >> 16 : bv1 & 0xFFFFu);
            // the codes entered the MMA as q * 2^-24: fold 2^24 into the scale
            const float s0 = sb_to_float<SB_FP16>(s0b) * 16777216.0f, s1 = sb_to_float<SB_FP16>(s1b) * 16777216.0f;
            const float b0 = sb_to_float<SB_FP16>(b0b), b1 = sb_to_float<SB_FP16>(b1b);
            // c[i][0]: row g, column 0 (x); c[i][2]: row g + 8 — valid in the lanes with t == 0
            acc0 = fmaf(s0, c[i][0], fmaf(b0, xsv[i], acc0));
            acc1 = fmaf(s1, c[i][2], fmaf(b1, xsv[i], acc1));
        }
    }
    if (t == 0) {
        if constexpr (OUT_F32) {       // unrounded row sums (the greedy LM head compares them as fp32)
            if (r0 < m) static_cast<float*>(y)[r0] = acc0;
            if (r1 < m) static_cast<float*>(y)[r1] = acc1;
        } else {
            if (r0 < m) static_cast<uint16_t*>(y)[r0] = __half_as_ushort(__float2half_rn(acc0));
            if (r1 < m) static_cast<uint16_t*>(y)[r1] = __half_as_ushort(__float2half_rn(acc1));
        }
    }
}

static size_t gemv_mma_smem_bytes_for(uint32_t n, int warps) {
    const size_t ng = n / kGroup;
    return ng * 132 + (size_t)2 * warps * 16 * ng * 2;
}
size_t gemv_mma_smem_bytes(uint32_t n) { return gemv_mma_smem_bytes_for(n, kGmWarps); }

// Eligible: large, 16-byte aligned planes, a multiple of 256 columns (scale rows are read four groups at a time).
bool gemv_mma_eligible(const void* W, const void* S, const void* B, const void* x, uint32_t m, uint32_t n) {
    return m >= 4096 && n % 256 == 0 && aligned(W, 16) && aligned(S, 16) && aligned(B, 16) && aligned(x, 16) &&
           gemv_mma_smem_bytes(n) <= 100 * 1024;
}

tf_status launch_gemv_mma(tf_context* ctx, void* stream, const uint8_t* W, const uint16_t* S, const uint16_t* B,
                          const uint16_t* x, void* y, bool out_f32, uint32_t m, uint32_t n, bool sb_fp16, const char* name) {
    const size_t smem = gemv_mma_smem_bytes(n);
    const int which = (sb_fp16 ? 1 : 0) + (out_f32 ? 2 : 0);
    auto k = which == 0 ? gemv_mma_kernel<false, false, kGmWarps> : which == 1 ? gemv_mma_kernel<true, false, kGmWarps>
             : which == 2 ? gemv_mma_kernel<false, true, kGmWarps> : gemv_mma_kernel<true, true, kGmWarps>;
    static DeviceSmemCache configured[4];
    if (tf_status st = ensure_dynamic_smem(ctx, k, configured[which], smem)) return st;
    k<<<(m + kGmWarps * 16 - 1) / (kGmWarps * 16), kGmWarps * kWarp, smem, static_cast<cudaStream_t>(stream)>>>(W, S, B, x, y, m, n, GemvBatch{0, 0, 0});
    return check_launch(ctx, name);
}

// `count` GEMVs over matrices of one shape whose planes repeat every plane_stride bytes, in one launch.
tf_status launch_gemv_mma_batched(tf_context* ctx, void* stream, const uint8_t* W, const uint16_t* S, const uint16_t* B,
                                  uint64_t plane_stride, const uint16_t* x, uint32_t x_stride, uint16_t* y, uint32_t y_stride,
                                  uint32_t m, uint32_t n, uint32_t count, bool sb_fp16, const char* name) {
    const size_t smem = gemv_mma_smem_bytes_for(n, kGmBatchWarps);
    auto k = sb_fp16 ? gemv_mma_kernel<true, false, kGmBatchWarps> : gemv_mma_kernel<false, false, kGmBatchWarps>;
    static DeviceSmemCache configured[2];
    if (tf_status st = ensure_dynamic_smem(ctx, k, configured[sb_fp16 ? 1 : 0], smem)) return st;
    const uint32_t rows_per_block = kGmBatchWarps * 16;
    for (uint32_t first = 0; first < count; first += 65535u) {        // gridDim.y limit
        const uint32_t nb = count - first < 65535u ? count - first : 65535u;
        dim3 grid((m + rows_per_block - 1) / rows_per_block, nb);
        k<<<grid, kGmBatchWarps * kWarp, smem, static_cast<cudaStream_t>(stream)>>>(
            W + (size_t)first * plane_stride,
            reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(S) + (size_t)first * plane_stride),
            reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(B) + (size_t)first * plane_stride),
            x + (size_t)first * x_stride, y + (size_t)first * y_stride, m, n, GemvBatch{plane_stride, x_stride, y_stride});
        if (tf_status st = check_launch(ctx, name)) return st;
    }
    return TF_OK;
}

}  // namespace tf
