// GELU of the bfloat16 GEMM epilogues (shared by the plain GEMM and the fused MLP kernel).
#pragma once
#include "f32x2.cuh"

namespace convnn {
// GELU for the bfloat16 epilogue.  nn.GELU()'s default is the erf form; here the tanh form
// 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) is evaluated with the hardware tanh unit.
// The two forms differ by at most 5e-4 in absolute value (well inside one bfloat16 rounding
// step of the stored activations), and this costs 7 instructions per element instead of ~17
// for a faithful erf: the activation runs in the GEMM epilogue, where instruction issue is
// what bounds the kernel.  The float32 path (SIMT GEMM) uses erff.
// Evaluated on packed pairs: x * (c0 + c1 x^2) -> tanh -> 0.5 x (1 + tanh), every step one packed
// instruction that rounds like its scalar counterpart.
__device__ __forceinline__ f32x2 gelu_pair(f32x2 x) {
    const f32x2 c1 = pack2(0.0356774081f, 0.0356774081f), c0 = pack2(0.7978845608f, 0.7978845608f);
    const f32x2 hf = pack2(0.5f, 0.5f);
    const f32x2 inner = mul2(x, fma2(c1, mul2(x, x), c0));
    float ia, ib, ta, tb;
    unpack2(inner, ia, ib);
    asm("tanh.approx.f32 %0, %1;" : "=f"(ta) : "f"(ia));
    asm("tanh.approx.f32 %0, %1;" : "=f"(tb) : "f"(ib));
    const f32x2 hx = mul2(hf, x);
    return fma2(hx, pack2(ta, tb), hx);
}

}  // namespace convnn
