// FP32-accumulate SIMT GEMM  C = A * W^T (+ bias, + GELU)  with the operand addressing
// modes the ConvNN path needs: token gather for the sampled-query projection, head-split
// stores for q/k/v, and the reference's flat head reinterpretation as the A operand of
// the output projection.  This is the float32 path (tensor cores would need a 3xTF32
// split to keep the 1e-6 similarity accuracy the top-K parity asks for) and the
// fallback for bfloat16 shapes the tcgen05 kernels do not cover.
#include "common.cuh"

namespace convnn {

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename T>
__device__ __forceinline__ const T* a_row_base(const GemmParams& p, int m) {
    const T* a = static_cast<const T*>(p.a);
    if (p.a_mode == A_ROWS) return a + (long long)m * p.lda;
    if (p.a_mode == A_TOKENS) {
        int b = m / p.rows_per_batch, r = m - b * p.rows_per_batch;
        int tok = p.cand ? p.cand[r] : r;
        return a + ((long long)b * p.T + tok) * p.lda;
    }
    return a;  // A_HEAD_QUIRK: resolved per element
}

template <typename T>
__device__ __forceinline__ float a_load(const GemmParams& p, const T* base, int m, int kk) {
    if (p.a_mode != A_HEAD_QUIRK) return to_f32<T>(base[kk]);
    // y[b, t', h*dk + c'] = flat(o[b, h])[c' * T + t']   (reference layers.py:247-259)
    int b = m / p.T, t = m - b * p.T;
    int h = kk / p.dk, c = kk - h * p.dk;
    return to_f32<T>(base[((long long)(b * p.H + h) * p.T) * p.dk + (long long)c * p.T + t]);
}

__device__ __forceinline__ float gelu_exact(float x) {
    return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
}

template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const GemmParams p) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    const int am = m0 + lr, wn = n0 + lr;
    const T* abase = am < p.M ? a_row_base<T>(p, am) : nullptr;
    const T* wbase = wn < p.N ? static_cast<const T*>(p.w) + (long long)wn * p.Kd : nullptr;
    const int ty = tid >> 4, tx = tid & 15;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < p.Kd; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int kk = k0 + lk + i;
            As[lk + i][lr] = (abase && kk < p.Kd) ? a_load<T>(p, abase, am, kk) : 0.f;
            Ws[lk + i][lr] = (wbase && kk < p.Kd) ? to_f32<T>(wbase[kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            float4 b4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            float av[4] = {a4.x, a4.y, a4.z, a4.w};
            float bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }

    T* c = static_cast<T*>(p.c);
    const T* bias = static_cast<const T*>(p.bias);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m0 + ty * 4 + i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            float r = acc[i][j];
            if (bias) r += to_f32<T>(bias[n]);
            if (p.gelu) r = gelu_exact(r);
            long long off;
            if (p.c_mode == C_ROWS) {
                off = (long long)m * p.ldc + n;
            } else {
                int h = n / p.dk, ch = n - h * p.dk;
                off = (long long)m * p.H * p.Cp + (long long)h * p.Cp + ch;
            }
            if (p.residual)
                r = to_f32<T>(from_f32<T>(r)) + to_f32<T>(static_cast<const T*>(p.residual)[(long long)m * p.ldr + n]);
            c[off] = from_f32<T>(r);
        }
    }
}

}  // namespace

int launch_gemm_simt(int dtype, const GemmParams& p, cudaStream_t st) {
    if (p.M <= 0 || p.N <= 0) return CONVNN_OK;
    dim3 grid((p.M + BM - 1) / BM, (p.N + BN - 1) / BN);
    if (dtype == CONVNN_F32)
        gemm_simt_kernel<float><<<grid, 256, 0, st>>>(p);
    else
        gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p);
    CONVNN_CHECK_LAUNCH("gemm_simt");
    return CONVNN_OK;
}

}  // namespace convnn
