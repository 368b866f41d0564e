// Building blocks of the one-token int4 GEMV on mma.sync.m16n8k16: 4-bit codes enter the A operand as fp16
// subnormals (q * 2^-24, or q * 2^-20 against activations pre-scaled by 1/16: one AND per two codes), the
// activation vector is column 0 of the B operand, accumulation is fp32 inside the instruction.
#pragma once

#include "tf_common.cuh"

namespace tf {

__device__ __forceinline__ uint32_t gm_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t gm_sixteenth(uint32_t v) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&v), __half2half2(__float2half_rn(0.0625f)));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ void gm_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1,
                                       const float (&z)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z[0]), "f"(z[1]), "f"(z[2]), "f"(z[3]));
}
__device__ __forceinline__ uint2 gm_ldg64(const uint8_t* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// The 16 activations x0..x15 at columns 64 G + 16 t feed four MMAs,
//   j = 0: (x0,x4),(x2,x6)   j = 1: (x1,x5)/16,(x3,x7)/16   j = 2, 3: the same for x8..x15
// (odd columns are pre-scaled by 1/16 because their codes sit four mantissa bits higher). r[0..7] are the 16 fp16
// values as eight 32-bit words; f receives the eight B-fragment words of (G, t).
__device__ __forceinline__ void gm_make_frag(const uint32_t (&r)[8], uint32_t* f) {
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int o = 4 * h2;
        f[4 * h2 + 0] = gm_prmt(r[o], r[o + 2], 0x5410);
        f[4 * h2 + 1] = gm_prmt(r[o + 1], r[o + 3], 0x5410);
        f[4 * h2 + 2] = gm_sixteenth(gm_prmt(r[o], r[o + 2], 0x7632));
        f[4 * h2 + 3] = gm_sixteenth(gm_prmt(r[o + 1], r[o + 3], 0x7632));
    }
}

}  // namespace tf
