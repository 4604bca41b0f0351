// Small data-movement kernels around the tensor-core GEMMs.
//   gather_rows   xq[b, r, :] = x[b, cand[r], :]   (candidate tokens of the sampled modes,
//                 reference layers.py:285, 298) so the query projection is a plain GEMM
//   merge_heads   the reference's flat head reinterpretation for H > 1 (layers.py:247-259):
//                 y[b, t', h*dk + c'] = flat(o[b, h])[c'*T + t'], a (dk x T) -> (T x dk)
//                 transpose per (batch, head), staged through shared memory so both the
//                 reads (along t') and the writes (along c') are contiguous
#include "common.cuh"

namespace convnn {
namespace {

template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, long long ldx, const int32_t* __restrict__ cand,
                                   T* __restrict__ xq, int Tn, int S, int D, long long total_vec, int vec) {
    const int per_row = D / vec;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec;
         i += (long long)gridDim.x * blockDim.x) {
        const int cv = (int)(i % per_row);
        const long long br = i / per_row;
        const int r = (int)(br % S);
        const long long b = br / S;
        const T* src = x + (b * Tn + cand[r]) * ldx + (long long)cv * vec;
        T* dst = xq + br * D + (long long)cv * vec;
        if (vec * sizeof(T) == 16) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
        } else {
            for (int e = 0; e < vec; ++e) dst[e] = src[e];
        }
    }
}

template <typename T>
__global__ void merge_heads_kernel(const T* __restrict__ o, T* __restrict__ y, int Tn, int H, int dk, int D) {
    __shared__ T tile[32][33];
    const int bh = blockIdx.z;
    const int b = bh / H, h = bh - b * H;
    const T* src = o + (long long)bh * Tn * dk;          // viewed as (dk, T): src[c * T + t]
    const int t0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int c = c0 + i, t = t0 + threadIdx.x;
        if (c < dk && t < Tn) tile[i][threadIdx.x] = src[(long long)c * Tn + t];
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int t = t0 + i, c = c0 + threadIdx.x;
        if (t < Tn && c < dk) y[((long long)b * Tn + t) * D + h * dk + c] = tile[threadIdx.x][i];
    }
}

}  // namespace

int launch_gather_rows(int dtype, const void* x, long long ldx, const int32_t* cand, void* xq, int B, int Tn, int S,
                       int D, cudaStream_t st) {
    const size_t elt = dtype == CONVNN_F32 ? 4 : 2;
    int vec = (int)(16 / elt);
    if (D % vec != 0 || ldx % vec != 0 || !aligned16(x) || !aligned16(xq)) vec = 1;
    const long long total = (long long)B * S * (D / vec);
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (dtype == CONVNN_F32)
        gather_rows_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(x), ldx, cand,
                                                         static_cast<float*>(xq), Tn, S, D, total, vec);
    else
        gather_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ldx, cand,
                                                                 static_cast<__nv_bfloat16*>(xq), Tn, S, D, total, vec);
    CONVNN_CHECK_LAUNCH("gather_rows");
    return CONVNN_OK;
}

int launch_merge_heads(int dtype, const void* o, void* y, int B, int Tn, int H, int dk, cudaStream_t st) {
    dim3 grid((Tn + 31) / 32, (dk + 31) / 32, B * H), block(32, 8);
    if (dtype == CONVNN_F32)
        merge_heads_kernel<float><<<grid, block, 0, st>>>(static_cast<const float*>(o), static_cast<float*>(y), Tn, H,
                                                         dk, H * dk);
    else
        merge_heads_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16*>(o),
                                                                 static_cast<__nv_bfloat16*>(y), Tn, H, dk, H * dk);
    CONVNN_CHECK_LAUNCH("merge_heads");
    return CONVNN_OK;
}

}  // namespace convnn
