/*
 * tf_oracle.c — CPU restatement of the reference's routed-expert arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker for the CUDA path and the
 * timed CPU baseline of the benchmark. Nothing in the product library links,
 * imports or calls it; the CUDA library fails loudly when it cannot run.
 *
 * Parity status: the reference (drumih/turbo-fieldfare) stores no numeric
 * golden outputs for this path. Its tests regenerate inputs from a seeded PRNG
 * and compare the GPU kernel with a CPU function in the same run. What the
 * reference pins literally, and what this oracle is checked against, is:
 *   - the grouping known-answer arrays
 *     (Tests/TurboFieldfare/Core/Kernels/Prefill/PrefillMoEGroupingTests.swift:5-115),
 *   - the PRNG, quantiser and reference formulas restated below,
 *   - the struct layouts (16-byte pair, 9 x u32 offsets),
 *   - the tolerance relations between "dequantise then dot" and the kernels'
 *     group-factored order on the reference's own seeds and shapes.
 * Floating-point outputs are therefore "parity pinned by relation, not by
 * golden bytes".
 *
 * Every function cites the reference file:line it follows (paths relative to
 * the reference repository root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define TFO_GROUP 64

/* ------------------------------------------------------------------------- */
/* 16-bit float conversions                                                   */
/* ------------------------------------------------------------------------- */

static inline uint32_t f32_bits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float bits_f32(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

/* Sources/TurboFieldfare/Infrastructure/ModelIO/Quantization.swift:17-23:
 * round-half-to-even truncation to the top 16 bits, no NaN special case. */
uint16_t tfo_bf16_bits(float x) {
    uint32_t bits = f32_bits(x);
    uint32_t lsb = (bits >> 16) & 1u;
    uint32_t rounded = (bits + 0x7FFFu + lsb) >> 16;
    return (uint16_t)rounded;
}

/* Quantization.swift:26-28 */
float tfo_bf16_to_float(uint16_t b) { return bits_f32((uint32_t)b << 16); }

/* IEEE binary16 with round-to-nearest-even, the semantics of Swift's
 * Float16(Float) and Metal's half(float) used at every fp16 store in the
 * reference kernels (e.g. Metal/MoE/moe.metal:368). */
uint16_t tfo_f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mant = x & 0x007FFFFFu;
    int32_t exp = (int32_t)((x >> 23) & 0xFF);
    if (exp == 0xFF) {                       /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | (mant ? 0x0200u | (mant >> 13) : 0));
    }
    int32_t e = exp - 127 + 15;
    if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);      /* overflow -> inf */
    if (e <= 0) {                            /* subnormal or zero */
        if (e < -10) return (uint16_t)sign;
        mant |= 0x00800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half_m = mant >> shift;
        uint32_t rem = mant & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_m & 1u))) half_m++;
        return (uint16_t)(sign | half_m);
    }
    uint32_t half_m = mant >> 13;
    uint32_t rem = mant & 0x1FFFu;
    uint32_t out = sign | ((uint32_t)e << 10) | half_m;
    if (rem > 0x1000u || (rem == 0x1000u && (half_m & 1u))) out++;   /* may carry into exp: correct */
    return (uint16_t)out;
}

float tfo_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t mant = h & 0x3FFu;
    if (exp == 0) {
        if (mant == 0) return bits_f32(sign);
        /* subnormal: normalise */
        int e = -1;
        do { mant <<= 1; e++; } while (!(mant & 0x400u));
        mant &= 0x3FFu;
        return bits_f32(sign | ((uint32_t)(127 - 15 - e) << 23) | (mant << 13));
    }
    if (exp == 0x1F) return bits_f32(sign | 0x7F800000u | (mant << 13));
    return bits_f32(sign | ((exp + 127 - 15) << 23) | (mant << 13));
}

/* scale / bias plane element -> float; dtype 0 = bf16 (the .gturbo format,
 * Sources/TurboFieldfareFormat/GTurboManifestV1.swift:68-73), 1 = fp16. */
static inline float sb_to_float(uint16_t v, int sb_dtype) {
    return sb_dtype == 0 ? tfo_bf16_to_float(v) : tfo_f16_to_f32(v);
}

void tfo_f32_to_f16_array(const float* in, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = tfo_f32_to_f16(in[i]);
}
void tfo_f16_to_f32_array(const uint16_t* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = tfo_f16_to_f32(in[i]);
}
void tfo_f32_to_bf16_array(const float* in, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = tfo_bf16_bits(in[i]);
}
void tfo_bf16_to_f32_array(const uint16_t* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = tfo_bf16_to_float(in[i]);
}

/* ------------------------------------------------------------------------- */
/* PRNG                                                                       */
/* ------------------------------------------------------------------------- */

/* Sources/TurboFieldfareValidation/Support/PRNG/SplitMix64.swift:11-17 */
uint64_t tfo_splitmix64_next(uint64_t* state) {
    *state += 0x9E3779B97F4A7C15ull;
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* SplitMix64.swift:20-23: 24-bit uniform in [lo, hi) */
float tfo_uniform(uint64_t* state, float lo, float hi) {
    float u = (float)(tfo_splitmix64_next(state) >> 40) / (float)(1 << 24);
    return lo + (hi - lo) * u;
}

void tfo_uniform_fill(uint64_t* state, float lo, float hi, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = tfo_uniform(state, lo, hi);
}

/* Sources/TurboFieldfareValidation/Support/PRNG/SeedTree.swift:12-19:
 * FNV-1a of the label xor the root gives the child stream's seed. */
uint64_t tfo_seedtree_key(uint64_t root, const char* label) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (const unsigned char* p = (const unsigned char*)label; *p; ++p) {
        h ^= (uint64_t)(*p);
        h *= 0x100000001B3ull;
    }
    return root ^ h;
}

/* ------------------------------------------------------------------------- */
/* Quantisers                                                                 */
/* ------------------------------------------------------------------------- */

/* Swift's Float.rounded() = round half away from zero = C roundf. */

/* Quantization.swift:50-102 */
void tfo_quantize_int4_affine(const float* row, int n, uint8_t* packed,
                              uint16_t* scales, uint16_t* biases) {
    int n_groups = n / TFO_GROUP;
    memset(packed, 0, (size_t)n / 2);
    for (int g = 0; g < n_groups; ++g) {
        float wmin = INFINITY, wmax = -INFINITY;
        for (int k = 0; k < TFO_GROUP; ++k) {
            float w = row[g * TFO_GROUP + k];
            if (w < wmin) wmin = w;
            if (w > wmax) wmax = w;
        }
        float scale_f, bias_f;
        if (wmax == wmin) { scale_f = 1.0f; bias_f = wmin; }
        else { scale_f = (wmax - wmin) / 15.0f; bias_f = wmin; }
        uint16_t sb = tfo_bf16_bits(scale_f), bb = tfo_bf16_bits(bias_f);
        scales[g] = sb; biases[g] = bb;
        float scale = tfo_bf16_to_float(sb), bias = tfo_bf16_to_float(bb);
        float inv = scale == 0.0f ? 0.0f : 1.0f / scale;
        for (int k = 0; k < TFO_GROUP; ++k) {
            float w = row[g * TFO_GROUP + k];
            int q = (int)roundf((w - bias) * inv);
            if (q < 0) q = 0;
            if (q > 15) q = 15;
            int byte_idx = g * (TFO_GROUP / 2) + (k / 2);
            if ((k & 1) == 0) packed[byte_idx] = (uint8_t)((packed[byte_idx] & 0xF0) | q);
            else packed[byte_idx] = (uint8_t)((packed[byte_idx] & 0x0F) | (q << 4));
        }
    }
}

/* Quantization.swift:104-119 (sb_dtype 0 reproduces it exactly) */
void tfo_dequantize_int4_affine(const uint8_t* packed, const uint16_t* scales,
                                const uint16_t* biases, int sb_dtype, int n, float* out) {
    int n_groups = n / TFO_GROUP;
    for (int g = 0; g < n_groups; ++g) {
        float scale = sb_to_float(scales[g], sb_dtype);
        float bias = sb_to_float(biases[g], sb_dtype);
        for (int k = 0; k < TFO_GROUP; ++k) {
            uint8_t b = packed[g * (TFO_GROUP / 2) + (k / 2)];
            int nib = (k & 1) == 0 ? (b & 0x0F) : (b >> 4);
            out[g * TFO_GROUP + k] = (float)nib * scale + bias;
        }
    }
}

/* Quantization.swift:135-176 */
void tfo_quantize_int8_affine(const float* row, int n, uint8_t* packed,
                              uint16_t* scales, uint16_t* biases) {
    int n_groups = n / TFO_GROUP;
    for (int g = 0; g < n_groups; ++g) {
        float wmin = INFINITY, wmax = -INFINITY;
        for (int k = 0; k < TFO_GROUP; ++k) {
            float w = row[g * TFO_GROUP + k];
            if (w < wmin) wmin = w;
            if (w > wmax) wmax = w;
        }
        float scale_f, bias_f;
        if (wmax == wmin) { scale_f = 1.0f; bias_f = wmin; }
        else { scale_f = (wmax - wmin) / 255.0f; bias_f = wmin; }
        uint16_t sb = tfo_bf16_bits(scale_f), bb = tfo_bf16_bits(bias_f);
        scales[g] = sb; biases[g] = bb;
        float scale = tfo_bf16_to_float(sb), bias = tfo_bf16_to_float(bb);
        float inv = scale == 0.0f ? 0.0f : 1.0f / scale;
        for (int k = 0; k < TFO_GROUP; ++k) {
            float w = row[g * TFO_GROUP + k];
            int q = (int)roundf((w - bias) * inv);
            if (q < 0) q = 0;
            if (q > 255) q = 255;
            packed[g * TFO_GROUP + k] = (uint8_t)q;
        }
    }
}

/* Quantization.swift:178-191 */
void tfo_dequantize_int8_affine(const uint8_t* packed, const uint16_t* scales,
                                const uint16_t* biases, int sb_dtype, int n, float* out) {
    int n_groups = n / TFO_GROUP;
    for (int g = 0; g < n_groups; ++g) {
        float scale = sb_to_float(scales[g], sb_dtype);
        float bias = sb_to_float(biases[g], sb_dtype);
        for (int k = 0; k < TFO_GROUP; ++k)
            out[g * TFO_GROUP + k] = (float)packed[g * TFO_GROUP + k] * scale + bias;
    }
}

/* ------------------------------------------------------------------------- */
/* GEMV references                                                            */
/* ------------------------------------------------------------------------- */

/* Sources/TurboFieldfareValidation/Support/Reference/Quant/DequantInt4Gemv.swift:13-42
 * (and DequantInt8Gemv.swift:13-40): dequantise each row to fp32, then dot.
 * vDSP_dotpr's summation order is not specified, so two variants are given:
 * acc_mode 0 = double accumulation (the "truth" the tolerance tests use),
 * acc_mode 1 = sequential fp32. bits = 4 or 8. x and y are fp32. */
void tfo_affine_gemv_ref(const uint8_t* W, const uint16_t* S, const uint16_t* B, int sb_dtype,
                         const float* x, float* y, int m, int n, int bits, int acc_mode) {
    int n_groups = n / TFO_GROUP;
    int64_t row_bytes = bits == 4 ? n / 2 : n;
#pragma omp parallel
    {
        float* wrow = (float*)malloc(sizeof(float) * (size_t)n);
#pragma omp for schedule(static)
        for (int r = 0; r < m; ++r) {
            if (bits == 4)
                tfo_dequantize_int4_affine(W + (int64_t)r * row_bytes, S + (int64_t)r * n_groups,
                                           B + (int64_t)r * n_groups, sb_dtype, n, wrow);
            else
                tfo_dequantize_int8_affine(W + (int64_t)r * row_bytes, S + (int64_t)r * n_groups,
                                           B + (int64_t)r * n_groups, sb_dtype, n, wrow);
            if (acc_mode == 0) {
                double acc = 0.0;
                for (int i = 0; i < n; ++i) acc += (double)wrow[i] * (double)x[i];
                y[r] = (float)acc;
            } else {
                float acc = 0.0f;
                for (int i = 0; i < n; ++i) acc += wrow[i] * x[i];
                y[r] = acc;
            }
        }
        free(wrow);
    }
}

static inline float butterfly32(float* lane) {
    /* fixed xor-butterfly (offsets 16,8,4,2,1); every lane ends with the same
     * value because fp addition is commutative. This is the canonical order of
     * the CUDA kernels' warp reductions. */
    for (int off = 16; off >= 1; off >>= 1) {
        float t[32];
        for (int l = 0; l < 32; ++l) t[l] = lane[l] + lane[l ^ off];
        memcpy(lane, t, sizeof(t));
    }
    return lane[0];
}

/* One row of the int4 kernel's group-factored order
 * (Metal/Quant/dequant_int4.metal:93-191; Metal/MoE/moe.metal:187-244):
 * 4-group blocks, lane handles 8 contiguous elements, per-lane
 * acc = fma(s, dot, acc); acc = fma(b, sum, acc); then a 32-lane sum.
 * x is fp32 (already widened from fp16 by the caller). */
static float int4_row_kernel_order(const uint8_t* Wrow, const uint16_t* s_row,
                                   const uint16_t* b_row, int sb_dtype,
                                   const float* x, int n) {
    int n_groups = n / TFO_GROUP;
    int full_blocks = n_groups / 4;
    float lane_acc[32];
    for (int lane = 0; lane < 32; ++lane) {
        float acc = 0.0f;
        for (int blk = 0; blk < full_blocks; ++blk) {
            int byte_base = blk * 128 + lane * 4;
            int g = blk * 4 + (lane >> 3);
            float s = sb_to_float(s_row[g], sb_dtype);
            float b = sb_to_float(b_row[g], sb_dtype);
            int elem = byte_base * 2;
            float dot = 0.0f, sum = 0.0f;
            float e[8];
            for (int j = 0; j < 8; ++j) e[j] = x[elem + j];
            for (int j = 0; j < 4; ++j) {
                uint8_t by = Wrow[byte_base + j];
                dot = fmaf((float)(by & 0x0F), e[2 * j], dot);
                dot = fmaf((float)(by >> 4), e[2 * j + 1], dot);
            }
            sum = e[0] + e[1] + e[2] + e[3] + e[4] + e[5] + e[6] + e[7];
            acc = fmaf(s, dot, acc);
            acc = fmaf(b, sum, acc);
        }
        for (int g = full_blocks * 4; g < n_groups; ++g) {
            float s = sb_to_float(s_row[g], sb_dtype);
            float b = sb_to_float(b_row[g], sb_dtype);
            uint8_t by = Wrow[g * 32 + lane];
            float x0 = x[g * 64 + lane * 2], x1 = x[g * 64 + lane * 2 + 1];
            float dot = fmaf((float)(by & 0x0F), x0, 0.0f);
            dot = fmaf((float)(by >> 4), x1, dot);
            acc = fmaf(s, dot, acc);
            acc = fmaf(b, x0 + x1, acc);
        }
        lane_acc[lane] = acc;
    }
    return butterfly32(lane_acc);
}

/* Whole GEMV in the kernel's order; x fp16 bits in, y fp16 bits out
 * (dequant_int4.metal:187-190: lane 0 stores half(acc)). Also returns the
 * fp32 accumulators when y_f32 is non-null. */
void tfo_int4_gemv_kernel_order(const uint8_t* W, const uint16_t* S, const uint16_t* B, int sb_dtype,
                                const uint16_t* x_f16, uint16_t* y_f16, float* y_f32, int m, int n) {
    int n_groups = n / TFO_GROUP;
    float* x = (float*)malloc(sizeof(float) * (size_t)n);
    for (int i = 0; i < n; ++i) x[i] = tfo_f16_to_f32(x_f16[i]);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < m; ++r) {
        float acc = int4_row_kernel_order(W + (int64_t)r * (n / 2), S + (int64_t)r * n_groups,
                                          B + (int64_t)r * n_groups, sb_dtype, x, n);
        if (y_f32) y_f32[r] = acc;
        if (y_f16) y_f16[r] = tfo_f32_to_f16(acc);
    }
    free(x);
}

/* One row of the int8 kernels' order (Metal/Quant/dequant_int8.metal:57-97 and
 * Metal/MoE/moe.metal:78-116): lane handles elements g*64 + 2*lane, +1.
 * Canonical form used by the CUDA kernels and emulated here bit for bit:
 *   p   = fmaf(q1, x1, q0 * x0)
 *   acc = fmaf(s, p, acc); acc = fmaf(b, x0 + x1, acc)
 * then the xor-butterfly. x is fp32 (for the router: float(hidden) *
 * float(effective_scale), one fp32 multiply). Compile this file with
 * -ffp-contract=off so that no other contraction happens. */
static float int8_row_kernel_order(const uint8_t* Wrow, const uint16_t* s_row,
                                   const uint16_t* b_row, int sb_dtype,
                                   const float* x, int n) {
    int n_groups = n / TFO_GROUP;
    float lane_acc[32];
    for (int lane = 0; lane < 32; ++lane) {
        float acc = 0.0f;
        for (int g = 0; g < n_groups; ++g) {
            float s = sb_to_float(s_row[g], sb_dtype);
            float b = sb_to_float(b_row[g], sb_dtype);
            int i0 = g * 64 + lane * 2;
            float q0 = (float)Wrow[i0], q1 = (float)Wrow[i0 + 1];
            float x0 = x[i0], x1 = x[i0 + 1];
            float p = fmaf(q1, x1, q0 * x0);
            acc = fmaf(s, p, acc);
            acc = fmaf(b, x0 + x1, acc);
        }
        lane_acc[lane] = acc;
    }
    return butterfly32(lane_acc);
}

void tfo_int8_gemv_kernel_order(const uint8_t* W, const uint16_t* S, const uint16_t* B, int sb_dtype,
                                const uint16_t* x_f16, uint16_t* y_f16, float* y_f32, int m, int n) {
    int n_groups = n / TFO_GROUP;
    float* x = (float*)malloc(sizeof(float) * (size_t)n);
    for (int i = 0; i < n; ++i) x[i] = tfo_f16_to_f32(x_f16[i]);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < m; ++r) {
        float acc = int8_row_kernel_order(W + (int64_t)r * n, S + (int64_t)r * n_groups,
                                          B + (int64_t)r * n_groups, sb_dtype, x, n);
        if (y_f32) y_f32[r] = acc;
        if (y_f16) y_f16[r] = tfo_f32_to_f16(acc);
    }
    free(x);
}

/* ------------------------------------------------------------------------- */
/* Router                                                                     */
/* ------------------------------------------------------------------------- */

/* Router logits in the canonical kernel order (moe.metal:78-116,
 * Metal/Prefill/prefill.metal:478-520). hidden: fp16 bits [T, stride];
 * effective_scale: bf16 bits [D]; logits: fp32 [T, E]. */
void tfo_router_logits(const uint8_t* W, const uint16_t* S, const uint16_t* B,
                       const uint16_t* hidden_f16, int64_t hidden_stride,
                       const uint16_t* eff_scale_bf16, float* logits, int T, int E, int D) {
    int n_groups = D / TFO_GROUP;
#pragma omp parallel
    {
        float* x = (float*)malloc(sizeof(float) * (size_t)D);
#pragma omp for schedule(static)
        for (int t = 0; t < T; ++t) {
            for (int i = 0; i < D; ++i)
                x[i] = tfo_f16_to_f32(hidden_f16[(int64_t)t * hidden_stride + i]) *
                       tfo_bf16_to_float(eff_scale_bf16[i]);
            for (int e = 0; e < E; ++e)
                logits[(int64_t)t * E + e] = int8_row_kernel_order(
                    W + (int64_t)e * D, S + (int64_t)e * n_groups, B + (int64_t)e * n_groups, 0, x, D);
        }
        free(x);
    }
}

/* Double-precision logits: the order-free truth used to count near ties. */
void tfo_router_logits_f64(const uint8_t* W, const uint16_t* S, const uint16_t* B,
                           const uint16_t* hidden_f16, int64_t hidden_stride,
                           const uint16_t* eff_scale_bf16, double* logits, int T, int E, int D) {
    int n_groups = D / TFO_GROUP;
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; ++t) {
        for (int e = 0; e < E; ++e) {
            double acc = 0.0;
            for (int i = 0; i < D; ++i) {
                double w = (double)W[(int64_t)e * D + i] *
                               (double)tfo_bf16_to_float(S[(int64_t)e * n_groups + i / TFO_GROUP]) +
                           (double)tfo_bf16_to_float(B[(int64_t)e * n_groups + i / TFO_GROUP]);
                double xv = (double)tfo_f16_to_f32(hidden_f16[(int64_t)t * hidden_stride + i]) *
                            (double)tfo_bf16_to_float(eff_scale_bf16[i]);
                acc += w * xv;
            }
            logits[(int64_t)t * E + e] = acc;
        }
    }
}

/* Top-k by insertion, ties to the lower index (moe.metal:135-166;
 * prefill.metal:531-556), then softmax over the selected logits times the
 * per-expert gain, rounded to fp16 (moe.metal:168-184). expf stands in for
 * Metal's fast::exp; the weights are tolerance-checked, the indices bit-exact.
 * logits fp32 [T,E] -> idx u32 [T,K], w fp16 bits [T,K]. */
void tfo_router_select(const float* logits, const uint16_t* per_expert_scale_bf16,
                       uint32_t* out_idx, uint16_t* out_w_f16, float* out_w_f32, int T, int E, int K) {
    for (int t = 0; t < T; ++t) {
        const float* lg = logits + (int64_t)t * E;
        uint32_t top_idx[64];
        float top_score[64];
        for (int i = 0; i < K; ++i) { top_idx[i] = 0; top_score[i] = -INFINITY; }
        for (int e = 0; e < E; ++e) {
            float s = lg[e];
            if (s <= top_score[K - 1]) continue;
            int pos = K;
            for (int i = 0; i < K; ++i) {
                if (s > top_score[i] || (s == top_score[i] && (uint32_t)e < top_idx[i])) { pos = i; break; }
            }
            if (pos >= K) continue;
            for (int i = K - 1; i > pos; --i) { top_idx[i] = top_idx[i - 1]; top_score[i] = top_score[i - 1]; }
            top_idx[pos] = (uint32_t)e;
            top_score[pos] = s;
        }
        float max_s = top_score[0], sum_exp = 0.0f, exps[64];
        for (int i = 0; i < K; ++i) { exps[i] = expf(top_score[i] - max_s); sum_exp += exps[i]; }
        for (int i = 0; i < K; ++i) {
            float w = exps[i] / sum_exp * tfo_bf16_to_float(per_expert_scale_bf16[top_idx[i]]);
            out_idx[(int64_t)t * K + i] = top_idx[i];
            if (out_w_f16) out_w_f16[(int64_t)t * K + i] = tfo_f32_to_f16(w);
            if (out_w_f32) out_w_f32[(int64_t)t * K + i] = w;
        }
    }
}

/* The router reference the reference's own test uses
 * (Tests/TurboFieldfare/Core/Kernels/MoE/RouterTopKTests.swift:72-97): a full
 * stable sort by (logit desc, index asc), take K, softmax, times gain. Used to
 * check tfo_router_select against an independent formulation. */
void tfo_router_select_sorted(const float* logits, const float* expert_scale_f32,
                              uint32_t* out_idx, float* out_w, int E, int K) {
    uint32_t* order = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)E);
    for (int e = 0; e < E; ++e) order[e] = (uint32_t)e;
    for (int i = 1; i < E; ++i) {            /* insertion sort: stable, E <= 256 */
        uint32_t v = order[i];
        int j = i - 1;
        while (j >= 0 && (logits[order[j]] < logits[v] ||
                          (logits[order[j]] == logits[v] && order[j] > v))) {
            order[j + 1] = order[j];
            --j;
        }
        order[j + 1] = v;
    }
    float maximum = logits[order[0]], sum = 0.0f, ex[64];
    for (int i = 0; i < K; ++i) { ex[i] = expf(logits[order[i]] - maximum); sum += ex[i]; }
    for (int i = 0; i < K; ++i) {
        out_idx[i] = order[i];
        out_w[i] = ex[i] / sum * expert_scale_f32[order[i]];
    }
    free(order);
}

/* ------------------------------------------------------------------------- */
/* GeGLU expert FFN                                                           */
/* ------------------------------------------------------------------------- */

/* moe.metal:53-60: tanh GELU with the inner argument clamped to +-20.
 * (Reference/MoE/Moe.swift:24-32 is the same without the clamp; the clamp is a
 * no-op at fp32 precision because tanh(20) == 1.0f.) */
float tfo_gelu_tanh(float x) {
    float x3 = x * x * x;
    float inner = 0.7978845608028654f * (x + 0.044715f * x3);
    if (inner > 20.0f) inner = 20.0f;
    if (inner < -20.0f) inner = -20.0f;
    return 0.5f * x * (1.0f + tanhf(inner));
}

typedef struct {
    uint32_t gate_w, gate_s, gate_b, up_w, up_s, up_b, down_w, down_s, down_b;
} tfo_expert_offsets;   /* Kernels/MoE/MoE.swift:4-29 */

/* Decode routed experts with the kernels' rounding points:
 *   acts[k,f] = half(gelu(gate_k[f,:].x) * (up_k[f,:].x))            moe.metal:368
 *   y[d] = half(float(residual[d]) + sum_k float(w_k) * (down_k[d,:].acts_k))   moe.metal:473-480
 * blobs: K pointers to expert blobs. x, residual, w: fp16 bits. acts_out
 * (fp16 bits, K*F) is optional. order = 1 uses the kernel's lane order for
 * every dot product, order = 0 uses dequantise-then-double-dot (the truth). */
void tfo_moe_routed_decode(const uint8_t* const* blobs, const tfo_expert_offsets* off,
                           const uint16_t* x_f16, const uint16_t* w_f16, const uint16_t* residual_f16,
                           uint16_t* y_f16, float* y_f32, uint16_t* acts_out,
                           int D, int F, int K, int order) {
    int gD = D / TFO_GROUP, gF = F / TFO_GROUP;
    float* x = (float*)malloc(sizeof(float) * (size_t)D);
    uint16_t* acts = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)K * F);
    float* actf = (float*)malloc(sizeof(float) * (size_t)K * F);
    for (int i = 0; i < D; ++i) x[i] = tfo_f16_to_f32(x_f16[i]);
#pragma omp parallel for schedule(static) collapse(2)
    for (int k = 0; k < K; ++k) {
        for (int f = 0; f < F; ++f) {
            const uint8_t* base = blobs[k];
            const uint8_t* gW = base + off->gate_w + (int64_t)f * (D / 2);
            const uint8_t* uW = base + off->up_w + (int64_t)f * (D / 2);
            const uint16_t* gS = (const uint16_t*)(base + off->gate_s) + (int64_t)f * gD;
            const uint16_t* gB = (const uint16_t*)(base + off->gate_b) + (int64_t)f * gD;
            const uint16_t* uS = (const uint16_t*)(base + off->up_s) + (int64_t)f * gD;
            const uint16_t* uB = (const uint16_t*)(base + off->up_b) + (int64_t)f * gD;
            float g, u;
            if (order == 1) {
                g = int4_row_kernel_order(gW, gS, gB, 0, x, D);
                u = int4_row_kernel_order(uW, uS, uB, 0, x, D);
            } else {
                float wrow[8192];
                double a = 0.0, b2 = 0.0;
                tfo_dequantize_int4_affine(gW, gS, gB, 0, D, wrow);
                for (int i = 0; i < D; ++i) a += (double)wrow[i] * x[i];
                tfo_dequantize_int4_affine(uW, uS, uB, 0, D, wrow);
                for (int i = 0; i < D; ++i) b2 += (double)wrow[i] * x[i];
                g = (float)a; u = (float)b2;
            }
            uint16_t h = tfo_f32_to_f16(tfo_gelu_tanh(g) * u);
            acts[(int64_t)k * F + f] = h;
            actf[(int64_t)k * F + f] = tfo_f16_to_f32(h);
        }
    }
#pragma omp parallel for schedule(static)
    for (int d = 0; d < D; ++d) {
        float acc = residual_f16 ? tfo_f16_to_f32(residual_f16[d]) : 0.0f;
        for (int k = 0; k < K; ++k) {
            const uint8_t* base = blobs[k];
            const uint8_t* dW = base + off->down_w + (int64_t)d * (F / 2);
            const uint16_t* dS = (const uint16_t*)(base + off->down_s) + (int64_t)d * gF;
            const uint16_t* dB = (const uint16_t*)(base + off->down_b) + (int64_t)d * gF;
            float v;
            if (order == 1) {
                v = int4_row_kernel_order(dW, dS, dB, 0, actf + (int64_t)k * F, F);
            } else {
                float wrow[8192];
                double a = 0.0;
                tfo_dequantize_int4_affine(dW, dS, dB, 0, F, wrow);
                for (int i = 0; i < F; ++i) a += (double)wrow[i] * actf[(int64_t)k * F + i];
                v = (float)a;
            }
            acc += tfo_f16_to_f32(w_f16[k]) * v;
        }
        if (y_f32) y_f32[d] = acc;
        if (y_f16) y_f16[d] = tfo_f32_to_f16(acc);
    }
    if (acts_out) memcpy(acts_out, acts, sizeof(uint16_t) * (size_t)K * F);
    free(x); free(acts); free(actf);
}

/* Shared expert (Kernels/MoE/SharedExpertInt4.swift:60-93 with
 * Metal/Primitives/utility.metal:7-18): gate and up are stored as fp16 before
 * the activation; act fp16; down fp16. Planes are separate pointers because a
 * SharedExpertProjection carries three (buffer, offset) pairs. */
void tfo_shared_expert_int4(const uint8_t* gW, const uint16_t* gS, const uint16_t* gB,
                            const uint8_t* uW, const uint16_t* uS, const uint16_t* uB,
                            const uint8_t* dW, const uint16_t* dS, const uint16_t* dB,
                            const uint16_t* x_f16, uint16_t* y_f16, float* y_f32,
                            int D, int Fs, int order) {
    int gD = D / TFO_GROUP, gF = Fs / TFO_GROUP;
    float* x = (float*)malloc(sizeof(float) * (size_t)D);
    float* act = (float*)malloc(sizeof(float) * (size_t)Fs);
    for (int i = 0; i < D; ++i) x[i] = tfo_f16_to_f32(x_f16[i]);
#pragma omp parallel for schedule(static)
    for (int f = 0; f < Fs; ++f) {
        float g, u;
        if (order == 1) {
            g = int4_row_kernel_order(gW + (int64_t)f * (D / 2), gS + (int64_t)f * gD, gB + (int64_t)f * gD, 0, x, D);
            u = int4_row_kernel_order(uW + (int64_t)f * (D / 2), uS + (int64_t)f * gD, uB + (int64_t)f * gD, 0, x, D);
        } else {
            float wrow[8192];
            double a = 0.0, b2 = 0.0;
            tfo_dequantize_int4_affine(gW + (int64_t)f * (D / 2), gS + (int64_t)f * gD, gB + (int64_t)f * gD, 0, D, wrow);
            for (int i = 0; i < D; ++i) a += (double)wrow[i] * x[i];
            tfo_dequantize_int4_affine(uW + (int64_t)f * (D / 2), uS + (int64_t)f * gD, uB + (int64_t)f * gD, 0, D, wrow);
            for (int i = 0; i < D; ++i) b2 += (double)wrow[i] * x[i];
            g = (float)a; u = (float)b2;
        }
        float gh = tfo_f16_to_f32(tfo_f32_to_f16(g));
        float uh = tfo_f16_to_f32(tfo_f32_to_f16(u));
        act[f] = tfo_f16_to_f32(tfo_f32_to_f16(tfo_gelu_tanh(gh) * uh));
    }
#pragma omp parallel for schedule(static)
    for (int d = 0; d < D; ++d) {
        float v;
        if (order == 1) {
            v = int4_row_kernel_order(dW + (int64_t)d * (Fs / 2), dS + (int64_t)d * gF, dB + (int64_t)d * gF, 0, act, Fs);
        } else {
            float wrow[8192];
            double a = 0.0;
            tfo_dequantize_int4_affine(dW + (int64_t)d * (Fs / 2), dS + (int64_t)d * gF, dB + (int64_t)d * gF, 0, Fs, wrow);
            for (int i = 0; i < Fs; ++i) a += (double)wrow[i] * act[i];
            v = (float)a;
        }
        if (y_f32) y_f32[d] = v;
        if (y_f16) y_f16[d] = tfo_f32_to_f16(v);
    }
    free(x); free(act);
}

/* Token-major reduce (prefill.metal:575-596;
 * Tests/.../Kernels/Prefill/PrefillMoETests.swift:46-64):
 * h2[t,d] = half(sum_r fma(float(w[t,r]), float(partial[t,r,d]), acc)), rank order. */
void tfo_moe_reduce_token_major(const uint16_t* partials_f16, const uint16_t* weights_f16,
                                uint16_t* h2_f16, int T, int K, int D) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; ++t)
        for (int d = 0; d < D; ++d) {
            float acc = 0.0f;
            for (int r = 0; r < K; ++r)
                acc = fmaf(tfo_f16_to_f32(weights_f16[(int64_t)t * K + r]),
                           tfo_f16_to_f32(partials_f16[((int64_t)t * K + r) * D + d]), acc);
            h2_f16[(int64_t)t * D + d] = tfo_f32_to_f16(acc);
        }
}

/* ------------------------------------------------------------------------- */
/* Pair grouping                                                              */
/* ------------------------------------------------------------------------- */

typedef struct { uint32_t token, expert, rank, weight_bits_and_reserved; } tfo_pair;   /* PrefillRouter.swift:5-28 */
typedef struct { uint32_t expert, pair_start, pair_count; } tfo_group;                 /* PrefillMoEGrouping.swift:4-15 */
typedef struct { uint32_t group_start, group_count, pair_start, pair_count; } tfo_tile; /* PrefillMoEGrouping.swift:18-31 */

/* PrefillRouter.swift:91-111 */
void tfo_make_token_expert_pairs(const uint32_t* indices, const uint16_t* weights_f16,
                                 int query_count, int top_k, tfo_pair* out) {
    for (int t = 0; t < query_count; ++t)
        for (int r = 0; r < top_k; ++r) {
            int i = t * top_k + r;
            out[i].token = (uint32_t)t;
            out[i].expert = indices[i];
            out[i].rank = (uint32_t)r;
            out[i].weight_bits_and_reserved = weights_f16[i];
        }
}

static const uint64_t* g_sort_keys;
static int pair_cmp(const void* a, const void* b) {
    const tfo_pair* l = (const tfo_pair*)a;
    const tfo_pair* r = (const tfo_pair*)b;
    if (g_sort_keys) {
        uint64_t lk = g_sort_keys[l->expert], rk = g_sort_keys[r->expert];
        if (lk != rk) return lk < rk ? -1 : 1;
    }
    if (l->expert != r->expert) return l->expert < r->expert ? -1 : 1;
    if (l->token != r->token) return l->token < r->token ? -1 : 1;
    if (l->rank != r->rank) return l->rank < r->rank ? -1 : 1;
    return 0;
}

/* PrefillMoEGrouping.swift:91-193. Error codes follow the order of
 * PrefillMoEGroupingError's cases (:52-62), starting at 1. Returns 0 on
 * success. (token, rank) keys are unique once validated, so the comparison
 * sort is a total order and qsort's instability cannot show. Not re-entrant. */
int tfo_group_pairs(const tfo_pair* pairs, int pair_count, int query_count, int top_k,
                    int num_experts, int tile_expert_count,
                    const uint64_t* expert_sort_keys, int sort_key_count,
                    tfo_pair* sorted_out, uint32_t* per_expert_offsets, uint32_t* per_expert_counts,
                    tfo_group* groups_out, int* group_count_out,
                    tfo_tile* tiles_out, int* tile_count_out) {
    if (query_count < 0) return 1;
    if (top_k <= 0) return 2;
    if (num_experts <= 0) return 3;
    if (tile_expert_count < 1 || tile_expert_count > 16) return 4;
    if (expert_sort_keys && sort_key_count != num_experts) return 10;
    if (pair_count != query_count * top_k) return 5;
    uint8_t* seen = (uint8_t*)calloc((size_t)(pair_count > 0 ? pair_count : 1), 1);
    for (int i = 0; i < pair_count; ++i) {
        if (pairs[i].token >= (uint32_t)query_count) { free(seen); return 6; }
        if (pairs[i].rank >= (uint32_t)top_k) { free(seen); return 7; }
        if (pairs[i].expert >= (uint32_t)num_experts) { free(seen); return 8; }
        size_t key = (size_t)pairs[i].token * (size_t)top_k + pairs[i].rank;
        if (seen[key]) { free(seen); return 9; }
        seen[key] = 1;
    }
    free(seen);
    memcpy(sorted_out, pairs, sizeof(tfo_pair) * (size_t)pair_count);
    g_sort_keys = expert_sort_keys;
    qsort(sorted_out, (size_t)pair_count, sizeof(tfo_pair), pair_cmp);
    g_sort_keys = NULL;
    for (int e = 0; e < num_experts; ++e) { per_expert_offsets[e] = 0xFFFFFFFFu; per_expert_counts[e] = 0; }
    int ng = 0, i = 0;
    while (i < pair_count) {
        uint32_t expert = sorted_out[i].expert;
        int start = i;
        while (i < pair_count && sorted_out[i].expert == expert) ++i;
        per_expert_offsets[expert] = (uint32_t)start;
        per_expert_counts[expert] = (uint32_t)(i - start);
        groups_out[ng].expert = expert;
        groups_out[ng].pair_start = (uint32_t)start;
        groups_out[ng].pair_count = (uint32_t)(i - start);
        ++ng;
    }
    int nt = 0, gs = 0;
    while (gs < ng) {
        int ge = gs + tile_expert_count < ng ? gs + tile_expert_count : ng;
        tiles_out[nt].group_start = (uint32_t)gs;
        tiles_out[nt].group_count = (uint32_t)(ge - gs);
        tiles_out[nt].pair_start = groups_out[gs].pair_start;
        tiles_out[nt].pair_count = groups_out[ge - 1].pair_start + groups_out[ge - 1].pair_count - groups_out[gs].pair_start;
        ++nt;
        gs = ge;
    }
    *group_count_out = ng;
    *tile_count_out = nt;
    return 0;
}

/* ------------------------------------------------------------------------- */
/* Batched (per-pair) routed experts and the QMM                              */
/* ------------------------------------------------------------------------- */

/* Per-pair prefill reference with the kernels' rounding points
 * (prefill.metal:598-670; Tests/.../Prefill/PrefillGroupedRoutedMoETests.swift:229-303):
 *   act = half(gelu(gate) * up) with gate, up in fp32; down -> fp16 partial at
 *   route_partials[(token*K + rank)*D + d].
 * act_dtype: 0 = fp16 activations/partials (the reference), 1 = bf16 (the
 * bf16 prefill configuration). hidden rows are [T, stride] in the same dtype.
 * pool_base + expert*stride gives each blob. Double accumulation. */
void tfo_grouped_moe_pairs(const uint8_t* pool_base, int64_t expert_stride, const tfo_expert_offsets* off,
                           const uint16_t* hidden, int64_t hidden_stride, int act_dtype,
                           const tfo_pair* pairs, int pair_count,
                           uint16_t* route_partials, int D, int F, int K) {
    int gD = D / TFO_GROUP, gF = F / TFO_GROUP;
#pragma omp parallel
    {
        float* x = (float*)malloc(sizeof(float) * (size_t)D);
        float* act = (float*)malloc(sizeof(float) * (size_t)F);
        float* wrow = (float*)malloc(sizeof(float) * (size_t)(D > F ? D : F));
#pragma omp for schedule(dynamic, 4)
        for (int p = 0; p < pair_count; ++p) {
            const tfo_pair pr = pairs[p];
            const uint8_t* base = pool_base + (int64_t)pr.expert * expert_stride;
            const uint16_t* xr = hidden + (int64_t)pr.token * hidden_stride;
            for (int i = 0; i < D; ++i) x[i] = act_dtype ? tfo_bf16_to_float(xr[i]) : tfo_f16_to_f32(xr[i]);
            for (int f = 0; f < F; ++f) {
                double g = 0.0, u = 0.0;
                tfo_dequantize_int4_affine(base + off->gate_w + (int64_t)f * (D / 2),
                                           (const uint16_t*)(base + off->gate_s) + (int64_t)f * gD,
                                           (const uint16_t*)(base + off->gate_b) + (int64_t)f * gD, 0, D, wrow);
                for (int i = 0; i < D; ++i) g += (double)wrow[i] * x[i];
                tfo_dequantize_int4_affine(base + off->up_w + (int64_t)f * (D / 2),
                                           (const uint16_t*)(base + off->up_s) + (int64_t)f * gD,
                                           (const uint16_t*)(base + off->up_b) + (int64_t)f * gD, 0, D, wrow);
                for (int i = 0; i < D; ++i) u += (double)wrow[i] * x[i];
                float a = tfo_gelu_tanh((float)g) * (float)u;
                act[f] = act_dtype ? tfo_bf16_to_float(tfo_bf16_bits(a)) : tfo_f16_to_f32(tfo_f32_to_f16(a));
            }
            uint16_t* out = route_partials + ((int64_t)pr.token * K + pr.rank) * D;
            for (int d = 0; d < D; ++d) {
                double v = 0.0;
                tfo_dequantize_int4_affine(base + off->down_w + (int64_t)d * (F / 2),
                                           (const uint16_t*)(base + off->down_s) + (int64_t)d * gF,
                                           (const uint16_t*)(base + off->down_b) + (int64_t)d * gF, 0, F, wrow);
                for (int i = 0; i < F; ++i) v += (double)wrow[i] * act[i];
                out[d] = act_dtype ? tfo_bf16_bits((float)v) : tfo_f32_to_f16((float)v);
            }
        }
        free(x); free(act); free(wrow);
    }
}

/* QMM reference Y[T,N] = X[T,K] . deq4(W[N,K])^T, fp32-dequantised weights,
 * double accumulation (Tests/.../TensorCore/MPPPrefillInt4QMMTests.swift:80-105;
 * prefill.metal:672-709). act_dtype as above. y_f32 out. */
void tfo_int4_qmm_ref(const uint8_t* W, const uint16_t* S, const uint16_t* B,
                      const uint16_t* X, int act_dtype, float* Y, int T, int N, int K) {
    int g = K / TFO_GROUP;
#pragma omp parallel
    {
        float* wrow = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
        for (int n = 0; n < N; ++n) {
            tfo_dequantize_int4_affine(W + (int64_t)n * (K / 2), S + (int64_t)n * g, B + (int64_t)n * g, 0, K, wrow);
            for (int t = 0; t < T; ++t) {
                double acc = 0.0;
                for (int k = 0; k < K; ++k) {
                    uint16_t xv = X[(int64_t)t * K + k];
                    acc += (double)wrow[k] * (double)(act_dtype ? tfo_bf16_to_float(xv) : tfo_f16_to_f32(xv));
                }
                Y[(int64_t)t * N + n] = (float)acc;
            }
        }
        free(wrow);
    }
}

/* ------------------------------------------------------------------------- */
/* Norms                                                                      */
/* ------------------------------------------------------------------------- */

/* Metal/Primitives/rmsnorm.metal:32-93,153-175: fp32 sum of squares (order
 * free here: double), inv = 1/sqrt(mean + eps), y = half(x * inv * w). weight
 * may be null (the no-scale form). Rows of D with a row stride. */
void tfo_rmsnorm(const uint16_t* x_f16, const uint16_t* weight_bf16, uint16_t* y_f16,
                 int T, int D, int64_t stride, float eps) {
    for (int t = 0; t < T; ++t) {
        const uint16_t* xr = x_f16 + (int64_t)t * stride;
        double ss = 0.0;
        for (int i = 0; i < D; ++i) { double v = tfo_f16_to_f32(xr[i]); ss += v * v; }
        float inv = 1.0f / sqrtf((float)(ss / D) + eps);
        for (int i = 0; i < D; ++i) {
            float v = tfo_f16_to_f32(xr[i]) * inv;
            if (weight_bf16) v *= tfo_bf16_to_float(weight_bf16[i]);
            y_f16[(int64_t)t * stride + i] = tfo_f32_to_f16(v);
        }
    }
}

/* Metal/Fusions/fused.metal:271-375:
 *   tmp  = half(h2 * inv(h2) * w2);  h12 = half(h1 + tmp)  (half add)
 *   tmp2 = half(h12 * inv(h12) * w); hidden = half(hidden + tmp2); hidden = half(hidden * half(layer_scalar)) */
void tfo_layer_tail(const uint16_t* h2_f16, const uint16_t* h1_f16, uint16_t* hidden_f16,
                    const uint16_t* w_postffn2_bf16, const uint16_t* w_postffn_bf16,
                    int T, int D, int64_t stride, float eps, float layer_scalar) {
    float* h12 = (float*)malloc(sizeof(float) * (size_t)D);
    float hs = tfo_f16_to_f32(tfo_f32_to_f16(layer_scalar));
    for (int t = 0; t < T; ++t) {
        const uint16_t* h2 = h2_f16 + (int64_t)t * stride;
        const uint16_t* h1 = h1_f16 + (int64_t)t * stride;
        uint16_t* hid = hidden_f16 + (int64_t)t * stride;
        double ss = 0.0;
        for (int i = 0; i < D; ++i) { double v = tfo_f16_to_f32(h2[i]); ss += v * v; }
        float inv = 1.0f / sqrtf((float)(ss / D) + eps);
        ss = 0.0;
        for (int i = 0; i < D; ++i) {
            float tmp = tfo_f16_to_f32(tfo_f32_to_f16(tfo_f16_to_f32(h2[i]) * inv * tfo_bf16_to_float(w_postffn2_bf16[i])));
            h12[i] = tfo_f16_to_f32(tfo_f32_to_f16(tfo_f16_to_f32(h1[i]) + tmp));
            ss += (double)h12[i] * h12[i];
        }
        float inv2 = 1.0f / sqrtf((float)(ss / D) + eps);
        for (int i = 0; i < D; ++i) {
            float tmp = tfo_f16_to_f32(tfo_f32_to_f16(h12[i] * inv2 * tfo_bf16_to_float(w_postffn_bf16[i])));
            float h = tfo_f16_to_f32(tfo_f32_to_f16(tfo_f16_to_f32(hid[i]) + tmp));
            hid[i] = tfo_f32_to_f16(h * hs);
        }
    }
    free(h12);
}

/* ------------------------------------------------------------------------- */
/* CPU baseline: the reference's affine-int4 matvec semantics, scalar, with    */
/* row partitioning over threads. Timed by the benchmark; never shipped.      */
/* ------------------------------------------------------------------------- */

int tfo_num_threads(void) {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void tfo_set_num_threads(int n) {
#if defined(_OPENMP)
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
