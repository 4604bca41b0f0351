// Packed pairs of fp32 in one 64-bit register: sm_100 executes add / mul / fma on both halves
// with one instruction (same IEEE results as two scalar operations), which halves the
// floating-point instruction count of element-wise inner loops.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace convnn {
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// 8 bfloat16 held in a uint4 -> four packed fp32 pairs (element order preserved)
__device__ __forceinline__ void bf16x8_to_f32x2(const uint4& v, f32x2 (&out)[4]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) out[e] = pack2(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xffff0000u));
}
__device__ __forceinline__ uint4 f32x2_to_bf16x8(const f32x2 (&in)[4]) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        float a, b;
        unpack2(in[e], a, b);
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        w[e] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
}  // namespace convnn
