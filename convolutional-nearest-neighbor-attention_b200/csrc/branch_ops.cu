// The Conv1d half of the reference's MultiHeadBranchingConv (MultiHeadConv1dAttention.forward,
// layers.py:477-500): per-head Conv1d(d_k, d_k, kernel_size, padding='same') over the tokens.
//
// Activations are token-major (B, T, H, d_k).  bfloat16 with d_k a multiple of 16: the taps are
// unfolded, U[(b, h, t), j * d_k + c] = y[b, t + j - pad, h, c] (zero outside the sequence), and
// the conv becomes U x W^T with W = (d_k, kernel_size * d_k) on the tensor-core GEMM, bias in its
// epilogue.  Everything else (float32, odd head widths) takes a direct SIMT kernel.
#include "common.cuh"

namespace convnn {
namespace {

template <typename T>
__global__ void conv1d_unfold_kernel(const T* __restrict__ y, T* __restrict__ u, int Tn, int H, int dk, int ks, int pad,
                                     long long total_vec, int vec) {
    const int per_tap = dk / vec;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec;
         i += (long long)gridDim.x * blockDim.x) {
        const int cv = (int)(i % per_tap);
        long long rest = i / per_tap;
        const int j = (int)(rest % ks);
        rest /= ks;                                   // (b * H + h) * T + t
        const int t = (int)(rest % Tn);
        const long long bh = rest / Tn;
        const int h = (int)(bh % H);
        const long long b = bh / H;
        const int tt = t + j - pad;
        T* dst = u + (rest * ks + j) * dk + (long long)cv * vec;
        if (tt >= 0 && tt < Tn) {
            const T* src = y + ((b * Tn + tt) * H + h) * dk + (long long)cv * vec;
            if (vec * sizeof(T) == 16) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
            else for (int e = 0; e < vec; ++e) dst[e] = src[e];
        } else {
            if (vec * sizeof(T) == 16) *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            else for (int e = 0; e < vec; ++e) dst[e] = from_f32<T>(0.f);
        }
    }
}

// One thread per output element (b, h, t, oc); w is (d_k out, kernel_size, d_k in).
template <typename T>
__global__ void conv1d_simt_kernel(const T* __restrict__ y, const T* __restrict__ w, const T* __restrict__ bias,
                                   T* __restrict__ o, int Tn, int H, int dk, int ks, int pad, long long total) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int oc = (int)(i % dk);
        long long rest = i / dk;
        const int t = (int)(rest % Tn);
        const long long bh = rest / Tn;
        const int h = (int)(bh % H);
        const long long b = bh / H;
        float acc = bias ? to_f32(bias[oc]) : 0.f;
        for (int j = 0; j < ks; ++j) {
            const int tt = t + j - pad;
            if (tt < 0 || tt >= Tn) continue;
            const T* src = y + ((b * Tn + tt) * H + h) * dk;
            const T* wr = w + ((long long)oc * ks + j) * dk;
            for (int c = 0; c < dk; ++c) acc = fmaf(to_f32(wr[c]), to_f32(src[c]), acc);
        }
        o[i] = from_f32<T>(acc);
    }
}

}  // namespace

// y (B, T, H, dk) -> o (B, H, T, dk); w (dk, ks, dk), bias (dk) or nullptr; `unfold` holds
// B*H*T*ks*dk elements and is only touched on the tensor-core route.
int launch_conv1d_heads(int dtype, const void* y, const void* w, const void* bias, void* o, void* unfold, int B,
                        int Tn, int H, int dk, int ks, cudaStream_t st) {
    const int pad = (ks - 1) / 2;                     // padding='same': the extra tap of an even kernel goes right
    const long long M = (long long)B * H * Tn;
    void* cs[1] = {o};
    if (dtype == CONVNN_BF16 && !force_simt() && unfold && dk % 16 == 0 && aligned16(y) && aligned16(unfold) &&
        (!bias || aligned16(bias)) && M < (1ll << 31) && gemm_tc_supported(unfold, (long long)ks * dk, w, ks * dk, dk, 1, cs, dk)) {
        const int vec = 8;
        const long long total = M * ks * (dk / vec);
        int blocks = (int)((total + 255) / 256);
        if (blocks > 148 * 16) blocks = 148 * 16;
        conv1d_unfold_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(y),
                                                                   static_cast<__nv_bfloat16*>(unfold), Tn, H, dk, ks, pad,
                                                                   total, vec);
        CONVNN_CHECK_LAUNCH("conv1d_unfold");
        GemmTcOpts go;
        go.bias = bias;
        return launch_gemm_tc(unfold, (long long)ks * dk, w, (int)M, dk, ks * dk, 1, cs, dk, go, st);
    }
    const long long total = M * dk;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == CONVNN_F32)
        conv1d_simt_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(y), static_cast<const float*>(w),
                                                         static_cast<const float*>(bias), static_cast<float*>(o), Tn, H, dk,
                                                         ks, pad, total);
    else
        conv1d_simt_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(w),
            static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(o), Tn, H, dk, ks, pad, total);
    CONVNN_CHECK_LAUNCH("conv1d_simt");
    return CONVNN_OK;
}

}  // namespace convnn
