// Neighbour weighting + gather + K-tap stride-K Conv1d (reference layers.py:389-406, 313).
//
// Weights over the K selected values (softmax, raw value, or reciprocal distance) are computed
// once per token into shared memory, then
//   depthwise            o[t, c] = sum_j w[j, c] * p[t, j] * v[idx[t, j], c]
//   standard             o[t, o] = sum_{j, c} w[o, j, c] * p[t, j] * v[idx[t, j], c]
//   depthwise-separable  depthwise, then a (d_k x C) matrix
// Kernels in this file, in the order the dispatcher tries them:
//   * depthwise, V slice of one (batch, head) resident in shared memory (one CTA per slice, the
//     K-fold neighbour reads never leave the SM; HBM sees V once and o once);
//   * depthwise, token tiles reading neighbour rows from global memory with 16-byte loads
//     (long sequences: the rows are L2-resident, fetched from HBM once);
//   * bfloat16 standard / separable on the tensor cores: a gather kernel writes the GEMM's A
//     operand (the weighted neighbour block, or the depthwise result) and gemm_tc multiplies it
//     with the (d_k, K*C) tap matrix / the (d_k, C) pointwise matrix;
//   * float32 (and fallback) standard / separable: shared-memory staged block times the weights.
// The three K-times expanded copies of V that the reference builds never exist (the tensor-core
// standard conv materialises the weighted block once, in bfloat16).
#include "common.cuh"
#include "f32x2.cuh"
#include "token_weights.cuh"

namespace convnn {
namespace {

constexpr int THREADS = 256;

template <typename T, int VEC> struct VecLoad;
template <> struct VecLoad<float, 4> {
    static __device__ __forceinline__ void load(const float* p, float* out) {
        float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* in) {
        *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
    }
};
template <> struct VecLoad<__nv_bfloat16, 8> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* out) {
        uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float2 f = __bfloat1622float2(h[e]);
            out[2 * e] = f.x; out[2 * e + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* in) {
        uint4 v;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(in[2 * e], in[2 * e + 1]);
        *reinterpret_cast<uint4*>(p) = v;
    }
};
template <typename T> struct VecLoad<T, 1> {
    static __device__ __forceinline__ void load(const T* p, float* out) { out[0] = to_f32<T>(*p); }
    static __device__ __forceinline__ void store(T* p, const float* in) { *p = from_f32<T>(in[0]); }
};

// ---- depthwise ---------------------------------------------------------------------
template <typename T, int VEC, int TT>
__global__ void __launch_bounds__(THREADS) gather_conv_dw_kernel(
    const T* __restrict__ v, const int32_t* __restrict__ idx, const float* __restrict__ val,
    const T* __restrict__ wconv, T* __restrict__ o, int T_, int H, int dk, int Cp, int K, int maximum,
    int softmax) {
    __shared__ float ps[TT][kMaxK];
    __shared__ int ns[TT][kMaxK];
    const int bh = blockIdx.y;
    const int b = bh / H, h = bh - b * H;
    const int t0 = blockIdx.x * TT;
    const int nt = min(TT, T_ - t0);
    const long long nbase = ((long long)bh * T_ + t0) * K;
    for (int e = threadIdx.x; e < nt * K; e += THREADS) ns[e / K][e % K] = idx[nbase + e];
    if (threadIdx.x < nt) token_weights(val + nbase + (long long)threadIdx.x * K, ps[threadIdx.x], K, maximum, softmax);
    __syncthreads();

    const int groups = dk / VEC;
    const T* vb = v + ((long long)b * T_ * H + h) * Cp;
    const long long tstride = (long long)H * Cp;
    for (int item = threadIdx.x; item < nt * groups; item += THREADS) {
        const int tt = item / groups, c = (item - tt * groups) * VEC;
        float acc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
        for (int j = 0; j < K; ++j) {
            float x[VEC], w[VEC];
            VecLoad<T, VEC>::load(vb + ns[tt][j] * tstride + c, x);
            VecLoad<T, VEC>::load(wconv + j * dk + c, w);
            const float pj = ps[tt][j];
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[e] = fmaf(w[e], pj * x[e], acc[e]);
        }
        VecLoad<T, VEC>::store(o + ((long long)bh * T_ + t0 + tt) * dk + c, acc);
    }
}

// ---- standard / depthwise-separable --------------------------------------------------
// Dynamic shared memory: P[TT][JC * C] floats (weighted neighbour block for JC taps, or
// the depthwise result with JC = 1 for the separable type).
template <typename T, int ITEMS>
__global__ void __launch_bounds__(THREADS) gather_conv_mat_kernel(
    const T* __restrict__ v, const int32_t* __restrict__ idx, const float* __restrict__ val,
    const T* __restrict__ wconv, const T* __restrict__ wpw, T* __restrict__ o, int T_, int H, int dk,
    int C, int Cp, int K, int maximum, int softmax, int separable, int TT, int JC) {
    extern __shared__ __align__(16) float P[];
    __shared__ float ps[32][kMaxK];
    __shared__ int ns[32][kMaxK];
    const int bh = blockIdx.y;
    const int b = bh / H, h = bh - b * H;
    const int t0 = blockIdx.x * TT;
    const int nt = min(TT, T_ - t0);
    const long long nbase = ((long long)bh * T_ + t0) * K;
    for (int e = threadIdx.x; e < nt * K; e += THREADS) ns[e / K][e % K] = idx[nbase + e];
    if (threadIdx.x < nt) token_weights(val + nbase + (long long)threadIdx.x * K, ps[threadIdx.x], K, maximum, softmax);
    __syncthreads();

    const T* vb = v + ((long long)b * T_ * H + h) * Cp;
    const long long tstride = (long long)H * Cp;
    const int tgroups = (TT + 3) / 4;
    const int n_items = dk * tgroups;
    float acc[ITEMS][4];
#pragma unroll
    for (int it = 0; it < ITEMS; ++it)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[it][e] = 0.f;

    const int ntaps = separable ? 1 : K;
    const int pstride = JC * C;
    for (int j0 = 0; j0 < ntaps; j0 += JC) {
        const int jn = min(JC, ntaps - j0);
        // fill P (zero rows for tokens past the end so the matrix step needs no guard)
        for (int e = threadIdx.x; e < TT * jn * C; e += THREADS) {
            const int tt = e / (jn * C);
            const int r = e - tt * jn * C;
            const int jj = r / C, c = r - jj * C;
            float x = 0.f;
            if (tt < nt) {
                if (separable) {
                    for (int j = 0; j < K; ++j)
                        x = fmaf(to_f32<T>(wconv[j * C + c]),
                                 ps[tt][j] * to_f32<T>(vb[ns[tt][j] * tstride + c]), x);
                } else {
                    const int j = j0 + jj;
                    x = ps[tt][j] * to_f32<T>(vb[ns[tt][j] * tstride + c]);
                }
            }
            P[tt * pstride + r] = x;
        }
        __syncthreads();
        // standard: w[oc][j*C + c] (d_k, K*C);  separable stage 1: w[oc][c] (d_k, C)
        const T* wm = separable ? wpw : wconv + (long long)j0 * C;
        const long long wld = separable ? C : (long long)K * C;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int item = threadIdx.x + it * THREADS;
            if (item < n_items) {
                const int oc = item % dk, tg = item / dk;
                const float* p0 = P + (tg * 4) * pstride;
                for (int r = 0; r < jn * C; ++r) {
                    const float w = to_f32<T>(wm[(long long)oc * wld + r]);
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (tg * 4 + e < TT) acc[it][e] = fmaf(w, p0[e * pstride + r], acc[it][e]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int item = threadIdx.x + it * THREADS;
        if (item < n_items) {
            const int oc = item % dk, tg = item / dk;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int tt = tg * 4 + e;
                if (tt < nt) o[((long long)bh * T_ + t0 + tt) * dk + oc] = from_f32<T>(acc[it][e]);
            }
        }
    }
}

template <typename T, int VEC>
int launch_dw(const convnn_desc* d, const Dims& dm, const void* v, const int32_t* idx, const float* val,
              const void* w_conv, void* o, cudaStream_t st) {
    constexpr int TT = 16;
    dim3 grid((dm.T + TT - 1) / TT, dm.B * dm.H);
    gather_conv_dw_kernel<T, VEC, TT><<<grid, THREADS, 0, st>>>(
        static_cast<const T*>(v), idx, val, static_cast<const T*>(w_conv), static_cast<T*>(o), dm.T, dm.H,
        dm.dk, dm.Cp, dm.K, d->metric != CONVNN_EUCLIDEAN, d->softmax);
    CONVNN_CHECK_LAUNCH("gather_conv_dw");
    return CONVNN_OK;
}

template <typename T>
int launch_mat(const convnn_desc* d, const Dims& dm, const void* v, const int32_t* idx, const float* val,
               const void* w_conv, const void* w_pw, void* o, cudaStream_t st) {
    constexpr int ITEMS = 4;
    const int separable = d->conv_type == CONVNN_DEPTHWISE_SEPARABLE;
    // token tile: dk * ceil(TT/4) work items must fit ITEMS passes of the CTA
    int TT = (THREADS * ITEMS / dm.dk) * 4;
    if (TT > 32) TT = 32;
    if (TT < 4) return set_error(CONVNN_E_UNSUPPORTED, "d_k=%d too large for the matrix conv kernel", dm.dk);
    const int ntaps = separable ? 1 : dm.K;
    const size_t budget = 64 * 1024;
    int JC = (int)(budget / ((size_t)TT * dm.C * sizeof(float)));
    if (JC < 1) JC = 1;
    if (JC > ntaps) JC = ntaps;
    size_t smem = (size_t)TT * JC * dm.C * sizeof(float);
    if (smem > 200 * 1024) return set_error(CONVNN_E_UNSUPPORTED, "conv tile needs %zu bytes of shared memory", smem);
    auto kern = gather_conv_mat_kernel<T, ITEMS>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    dim3 grid((dm.T + TT - 1) / TT, dm.B * dm.H);
    kern<<<grid, THREADS, smem, st>>>(static_cast<const T*>(v), idx, val, static_cast<const T*>(w_conv),
                                      static_cast<const T*>(w_pw), static_cast<T*>(o), dm.T, dm.H, dm.dk, dm.C,
                                      dm.Cp, dm.K, d->metric != CONVNN_EUCLIDEAN, d->softmax, separable, TT, JC);
    CONVNN_CHECK_LAUNCH("gather_conv_mat");
    return CONVNN_OK;
}

}  // namespace

int try_launch_gather_conv_dw_smem(const convnn_desc* d, const Dims& dm, const void* v, const int32_t* idx,
                                   const float* val, const void* w_conv, void* o, cudaStream_t st);

namespace {
// Weighted neighbour block for the tensor-core standard conv: P[(b,h,t), j*C + c] =
// bf16(p[t,j] * v[idx[t,j], c]), the A operand of a GEMM with the (d_k, K*C) tap weights.
// Rows of P are consecutive in (token, tap) order, so element e of a tile's flat (token, tap)
// list sits C channels after element e - 1.  Persistent CTAs walk tiles of TT tokens of one
// (batch, head); G = C / 8 consecutive threads cover one (token, tap) row's 16-byte units
// (G is a template constant so the per-item index arithmetic folds away; G = 0: any C).
template <int TT, int G>
__global__ void __launch_bounds__(THREADS) gather_weighted_kernel(
    const __nv_bfloat16* __restrict__ v, const int32_t* __restrict__ idx, const float* __restrict__ val,
    __nv_bfloat16* __restrict__ P, int T_, int H, int C, int Cp, int K, int maximum, int softmax, int n_bh,
    int tiles_per_bh) {
    __shared__ float ps[TT * kMaxK];
    __shared__ int ns[TT * kMaxK];
    const int groups = G > 0 ? G : C / 8;
    const int GP = G > 0 ? (G >= 32 ? 32 : G) : 1;          // threads side by side on one row
    const int g0 = threadIdx.x % GP, e0 = threadIdx.x / GP, estep = THREADS / GP;
    const int tstride = H * Cp;
    for (int tile = blockIdx.x; tile < n_bh * tiles_per_bh; tile += gridDim.x) {
        const int bh = tile / tiles_per_bh, t0 = (tile - bh * tiles_per_bh) * TT;
        const int b = bh / H, h = bh - b * H;
        const int nt = min(TT, T_ - t0);
        const long long nbase = ((long long)bh * T_ + t0) * K;
        __syncthreads();                                      // previous tile's lists are no longer read
        for (int e = threadIdx.x; e < nt * K; e += THREADS) ns[e] = idx[nbase + e] * tstride;
        if (threadIdx.x < nt)
            token_weights(val + nbase + (long long)threadIdx.x * K, ps + threadIdx.x * K, K, maximum, softmax);
        __syncthreads();
        const __nv_bfloat16* vb = v + ((long long)b * T_ * H + h) * Cp + g0 * 8;
        __nv_bfloat16* Pt = P + nbase * C + g0 * 8;
        for (int e = e0 < estep ? e0 : nt * K; e < nt * K; e += estep) {   // THREADS % GP leftover threads idle
            const __nv_bfloat16* src = vb + ns[e];
            const float pj = ps[e];
            const f32x2 p2 = pack2(pj, pj);
            __nv_bfloat16* dst = Pt + e * C;
#pragma unroll
            for (int g = 0; g < (G > 0 ? (G + 31) / 32 : 1); ++g) {
                if (G > 0) {
                    if (g * 32 + g0 < G) {
                        f32x2 x2[4];
                        bf16x8_to_f32x2(*reinterpret_cast<const uint4*>(src + g * 256), x2);
#pragma unroll
                        for (int q = 0; q < 4; ++q) x2[q] = mul2(p2, x2[q]);
                        *reinterpret_cast<uint4*>(dst + g * 256) = f32x2_to_bf16x8(x2);
                    }
                } else {
                    for (int gg = 0; gg < groups; ++gg) {
                        f32x2 x2[4];
                        bf16x8_to_f32x2(*reinterpret_cast<const uint4*>(src + gg * 8), x2);
#pragma unroll
                        for (int q = 0; q < 4; ++q) x2[q] = mul2(p2, x2[q]);
                        *reinterpret_cast<uint4*>(dst + gg * 8) = f32x2_to_bf16x8(x2);
                    }
                }
            }
        }
    }
}
}  // namespace

// bfloat16 standard / depthwise-separable conv on the tensor cores: a gather kernel builds the
// GEMM's A operand in `scratch`, the tap / pointwise weights are its (N, K) operand.
// Returns CONVNN_E_UNSUPPORTED (last_error untouched) when the shape does not qualify.
int try_launch_gather_conv_tc(const convnn_desc* d, const Dims& dm, const void* v, const int32_t* idx,
                              const float* val, const void* w_conv, const void* w_pw, void* o, void* scratch,
                              cudaStream_t st) {
    if (d->dtype != CONVNN_BF16 || d->coord || !scratch || force_simt() || dm.C % 8 != 0 || !aligned16(v) ||
        !aligned16(scratch))
        return CONVNN_E_UNSUPPORTED;
    const int M = dm.B * dm.H * dm.T;
    void* cs[1] = {o};
    int rc;
    if (d->conv_type == CONVNN_STANDARD) {
        const int Kd = dm.K * dm.C;
        if (!gemm_tc_supported(scratch, Kd, w_conv, Kd, dm.dk, 1, cs, dm.dk)) return CONVNN_E_UNSUPPORTED;
        constexpr int TT = 64;
        const int BH = dm.B * dm.H;
        const int tiles_per_bh = (dm.T + TT - 1) / TT;
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        long long grid = (long long)BH * tiles_per_bh;
        if (grid > sms * 8LL) grid = sms * 8LL;
        const int groups = dm.C / 8;
#define CONVNN_GW_LAUNCH(GV)                                                                                   \
        gather_weighted_kernel<TT, GV><<<(int)grid, THREADS, 0, st>>>(                                         \
            static_cast<const __nv_bfloat16*>(v), idx, val, static_cast<__nv_bfloat16*>(scratch), dm.T, dm.H, \
            dm.C, dm.Cp, dm.K, d->metric != CONVNN_EUCLIDEAN, d->softmax, BH, tiles_per_bh)
        if (groups == 4) CONVNN_GW_LAUNCH(4);
        else if (groups == 8) CONVNN_GW_LAUNCH(8);
        else if (groups == 24) CONVNN_GW_LAUNCH(24);
        else CONVNN_GW_LAUNCH(0);
#undef CONVNN_GW_LAUNCH
        CONVNN_CHECK_LAUNCH("gather_weighted");
        return launch_gemm_tc(scratch, Kd, w_conv, M, dm.dk, Kd, 1, cs, dm.dk, GemmTcOpts(), st);
    }
    if (d->conv_type == CONVNN_DEPTHWISE_SEPARABLE) {
        if (!gemm_tc_supported(scratch, dm.C, w_pw, dm.C, dm.dk, 1, cs, dm.dk)) return CONVNN_E_UNSUPPORTED;
        // stage 0: the depthwise kernels with the (K, C) taps, result (B, H, T, C) rounded to bf16
        rc = try_launch_gather_conv_dw_smem(d, dm, v, idx, val, w_conv, scratch, st);
        if (rc == CONVNN_E_UNSUPPORTED) {
            if (dm.dk % 8 != 0 || !aligned16(w_conv)) return CONVNN_E_UNSUPPORTED;
            rc = launch_dw<__nv_bfloat16, 8>(d, dm, v, idx, val, w_conv, scratch, st);
        }
        if (rc) return rc;
        return launch_gemm_tc(scratch, dm.C, w_pw, M, dm.dk, dm.C, 1, cs, dm.dk, GemmTcOpts(), st);
    }
    return CONVNN_E_UNSUPPORTED;
}

int launch_gather_conv_simt(const convnn_desc* d, const Dims& dm, const void* v, const int32_t* idx,
                            const float* val, const void* w_conv, const void* w_pw, void* o, void* scratch,
                            cudaStream_t st) {
    const bool f32 = d->dtype == CONVNN_F32;
    if (d->conv_type != CONVNN_DEPTHWISE) {
        const int rc = try_launch_gather_conv_tc(d, dm, v, idx, val, w_conv, w_pw, o, scratch, st);
        if (rc != CONVNN_E_UNSUPPORTED) return rc;
    }
    if (d->conv_type == CONVNN_DEPTHWISE) {
        const int rc = try_launch_gather_conv_dw_smem(d, dm, v, idx, val, w_conv, o, st);
        if (rc != CONVNN_E_UNSUPPORTED) return rc;
        const int vec = f32 ? 4 : 8;
        const bool vec_ok = dm.dk % vec == 0 && dm.Cp % vec == 0 && aligned16(v) && aligned16(o) && aligned16(w_conv);
        if (f32) return vec_ok ? launch_dw<float, 4>(d, dm, v, idx, val, w_conv, o, st)
                               : launch_dw<float, 1>(d, dm, v, idx, val, w_conv, o, st);
        return vec_ok ? launch_dw<__nv_bfloat16, 8>(d, dm, v, idx, val, w_conv, o, st)
                      : launch_dw<__nv_bfloat16, 1>(d, dm, v, idx, val, w_conv, o, st);
    }
    return f32 ? launch_mat<float>(d, dm, v, idx, val, w_conv, w_pw, o, st)
               : launch_mat<__nv_bfloat16>(d, dm, v, idx, val, w_conv, w_pw, o, st);
}

}  // namespace convnn

// ---- depthwise with the value rows resident in shared memory --------------------------
// When one (batch, head) slice of V (T x d_k) fits in shared memory, a CTA copies it in
// once with coalesced 16-byte loads and serves all K-fold neighbour reads from there, so
// HBM and L2 see V once and o once (the compulsory traffic) instead of K gathers per token.
// Thread layout: `groups` = d_k / VEC consecutive threads cover one token's channels, so a
// thread's channel group is fixed and its K x VEC tap weights stay in registers (KT > 0);
// KT == 0 is the run-time-K variant with the taps in shared memory.
namespace convnn {
namespace {

template <typename T, int VEC, int KT>
__global__ void __launch_bounds__(256) gather_conv_dw_smem_kernel(
    const T* __restrict__ v, const int32_t* __restrict__ idx, const float* __restrict__ val,
    const T* __restrict__ wconv, T* __restrict__ o, int T_, int H, int dk, int Cp, int K, int maximum,
    int softmax, int groups, int tpp) {
    extern __shared__ __align__(16) unsigned char dsm[];
    T* vs = reinterpret_cast<T*>(dsm);                                   // [T][dk]
    float* ps = reinterpret_cast<float*>(dsm + (((size_t)T_ * dk * sizeof(T) + 15) & ~(size_t)15));   // [T][K]
    int* ns = reinterpret_cast<int*>(ps + (size_t)T_ * K);               // [T][K]
    float* ws = reinterpret_cast<float*>(ns + (size_t)T_ * K);           // [K][dk] (KT == 0 only)

    const int bh = blockIdx.x;
    const int b = bh / H, h = bh - b * H;
    const T* vb = v + ((long long)b * T_ * H + h) * Cp;
    const long long tstride = (long long)H * Cp;
    const int row_vecs = dk / VEC;

    // 1. V slice -> shared memory (row-major, rows packed)
    for (int e = threadIdx.x; e < T_ * row_vecs; e += blockDim.x) {
        const int t = e / row_vecs, cvec = e - t * row_vecs;
        float tmp[VEC];
        VecLoad<T, VEC>::load(vb + t * tstride + cvec * VEC, tmp);
        VecLoad<T, VEC>::store(vs + (size_t)t * dk + cvec * VEC, tmp);
    }
    // 2. neighbour lists and their weights
    const long long nbase = (long long)bh * T_ * K;
    for (int e = threadIdx.x; e < T_ * K; e += blockDim.x) ns[e] = idx[nbase + e];
    for (int t = threadIdx.x; t < T_; t += blockDim.x) token_weights(val + nbase + (long long)t * K, ps + t * K, K, maximum, softmax);
    if (KT == 0)
        for (int e = threadIdx.x; e < K * dk; e += blockDim.x) ws[e] = to_f32<T>(wconv[e]);
    __syncthreads();

    // 3. taps
    const int cg = threadIdx.x % groups, tl = threadIdx.x / groups;
    if (tl >= tpp) return;
    const int c = cg * VEC;
    float wreg[KT > 0 ? KT : 1][VEC];
    if (KT > 0) {
#pragma unroll
        for (int j = 0; j < (KT > 0 ? KT : 1); ++j) VecLoad<T, VEC>::load(wconv + j * dk + c, wreg[j]);
    }
    T* ob = o + (long long)bh * T_ * dk + c;
    if constexpr (KT > 0 && VEC == 8 && sizeof(T) == 2) {
        // bfloat16, compile-time K: packed-pair arithmetic, tap weights as packed pairs in registers
        f32x2 w2[KT][4];
#pragma unroll
        for (int j = 0; j < KT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) w2[j][e] = pack2(wreg[j][2 * e], wreg[j][2 * e + 1]);
        for (int t = tl; t < T_; t += tpp) {
            f32x2 acc2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
            for (int j = 0; j < KT; ++j) {
                f32x2 x2[4];
                bf16x8_to_f32x2(*reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(vs) +
                                                                (size_t)ns[t * KT + j] * dk + c), x2);
                const float pj = ps[t * KT + j];
                const f32x2 p2 = pack2(pj, pj);
#pragma unroll
                for (int e = 0; e < 4; ++e) acc2[e] = fma2(w2[j][e], mul2(p2, x2[e]), acc2[e]);
            }
            float acc[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) unpack2(acc2[e], acc[2 * e], acc[2 * e + 1]);
            VecLoad<T, VEC>::store(ob + (long long)t * dk, acc);
        }
        return;
    }
    for (int t = tl; t < T_; t += tpp) {
        float acc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
        if (KT > 0) {
#pragma unroll
            for (int j = 0; j < (KT > 0 ? KT : 1); ++j) {
                float x[VEC];
                VecLoad<T, VEC>::load(vs + (size_t)ns[t * KT + j] * dk + c, x);
                const float pj = ps[t * KT + j];
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[e] = fmaf(wreg[j][e], pj * x[e], acc[e]);
            }
        } else {
            for (int j = 0; j < K; ++j) {
                float x[VEC];
                VecLoad<T, VEC>::load(vs + (size_t)ns[t * K + j] * dk + c, x);
                const float pj = ps[t * K + j];
                const float* wj = ws + j * dk + c;
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[e] = fmaf(wj[e], pj * x[e], acc[e]);
            }
        }
        VecLoad<T, VEC>::store(ob + (long long)t * dk, acc);
    }
}

template <typename T, int VEC>
int launch_dw_smem(const convnn_desc* d, const Dims& dm, const void* v, const int32_t* idx, const float* val,
                   const void* w_conv, void* o, size_t smem, cudaStream_t st) {
    const int groups = dm.dk / VEC;
    const int tpp = 256 / groups;
    const int maximum = d->metric != CONVNN_EUCLIDEAN;
#define CONVNN_DW_LAUNCH(KT)                                                                                 \
    do {                                                                                                     \
        auto kern = gather_conv_dw_smem_kernel<T, VEC, KT>;                                                  \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        kern<<<dm.B * dm.H, 256, smem, st>>>(static_cast<const T*>(v), idx, val, static_cast<const T*>(w_conv), \
                                             static_cast<T*>(o), dm.T, dm.H, dm.dk, dm.Cp, dm.K, maximum,    \
                                             d->softmax, groups, tpp);                                       \
    } while (0)
    if (dm.K == 9) CONVNN_DW_LAUNCH(9);
    else CONVNN_DW_LAUNCH(0);
#undef CONVNN_DW_LAUNCH
    CONVNN_CHECK_LAUNCH("gather_conv_dw_smem");
    return CONVNN_OK;
}

}  // namespace

// Shared-memory-resident depthwise variant; returns CONVNN_E_UNSUPPORTED (without touching
// last_error) when the slice does not fit or the layout is not vectorisable.
int try_launch_gather_conv_dw_smem(const convnn_desc* d, const Dims& dm, const void* v, const int32_t* idx,
                                   const float* val, const void* w_conv, void* o, cudaStream_t st) {
    const int rcs = try_launch_gather_conv_dw_stream(d, dm, v, idx, val, w_conv, o, st);
    if (rcs != CONVNN_E_UNSUPPORTED) return rcs;
    const bool f32 = d->dtype == CONVNN_F32;
    const int vec = f32 ? 4 : 8;
    if (dm.dk % vec != 0 || dm.Cp % vec != 0 || dm.dk / vec > 256 || !aligned16(v) || !aligned16(o) || !aligned16(w_conv))
        return CONVNN_E_UNSUPPORTED;
    size_t smem = (((size_t)dm.T * dm.dk * dm.elt + 15) & ~(size_t)15) + (size_t)dm.T * dm.K * 8;
    if (dm.K != 9) smem += (size_t)dm.K * dm.dk * 4;
    if (smem > 200 * 1024) return CONVNN_E_UNSUPPORTED;
    return f32 ? launch_dw_smem<float, 4>(d, dm, v, idx, val, w_conv, o, smem, st)
               : launch_dw_smem<__nv_bfloat16, 8>(d, dm, v, idx, val, w_conv, o, smem, st);
}

}  // namespace convnn
