// Depthwise gather + conv for short sequences (bfloat16, K = 9, d_k a multiple of 64),
// persistent and double-buffered.
//
// A work unit is one (batch, head) slice of V restricted to a 64-channel chunk: T rows of 128
// bytes, which one TMA copy brings into shared memory while the previous unit is being
// computed; the unit's neighbour indices and similarity values arrive beside it through
// cp.async.  A CTA keeps the same channel chunk for its whole life, so a thread's 9 x 8 tap
// weights are loaded into registers once.  Eight consecutive threads cover one token's 64
// channels: a warp reads four complete 128-byte rows per tap, which is conflict-free whatever
// rows the neighbour lists name.  Per unit the softmax weights are turned, once per token,
// into (byte offset of the neighbour row, weight) pairs so the tap loop is one 8-byte and one
// 16-byte shared-memory load plus packed fp32-pair arithmetic.
// HBM sees V once and o once; the K-fold neighbour reads stay inside the SM.
// The wait on the copy barrier is bounded; on expiry the CTA latches a status code and leaves.
#include "common.cuh"
#include "sm100.cuh"
#include "f32x2.cuh"
#include "token_weights.cuh"

namespace convnn {

__device__ int g_dw_stream_status = 0;

namespace {

using namespace sm100;

constexpr int KT = 9;              // taps
constexpr int CH = 64;             // channels per unit (one 128-byte row per token)
constexpr int TPB = 256;           // threads per CTA: 32 tokens x 8 channel groups per pass
constexpr int TOK_PASS = TPB / 8;

struct DwsParams {
    const int32_t* idx;
    const float* val;
    const __nv_bfloat16* wconv;
    __nv_bfloat16* o;
    int T, H, dk, maximum, softmax;
    int nchunks;                   // d_k / 64
    int n_slices;                  // B * H
    int ctas_per_chunk;
    uint32_t slice_bytes;          // T * 128
};

__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__global__ void __launch_bounds__(TPB, 2)
gather_conv_dw_stream_kernel(const __grid_constant__ CUtensorMap tmV, const DwsParams p) {
    extern __shared__ __align__(128) uint8_t dsm[];
    // [2][T x 128 B] V slices | [2][T*9] idx | [2][T*9] val | [T*9] (offset, weight) pairs | barriers
    const uint32_t nk = (uint32_t)p.T * KT;
    uint8_t* vs = dsm;
    int32_t* raw_idx = reinterpret_cast<int32_t*>(dsm + 2 * p.slice_bytes);
    float* raw_val = reinterpret_cast<float*>(raw_idx + 2 * nk);
    int2* np = reinterpret_cast<int2*>(raw_val + 2 * nk);                     // 2 * nk floats: stays 8-byte aligned
    uint64_t* full = reinterpret_cast<uint64_t*>(np + nk);
    __shared__ int s_fail;

    const int chunk = blockIdx.x % p.nchunks;
    const int lane_cta = blockIdx.x / p.nchunks;          // position among the CTAs of this chunk
    const int c0 = chunk * CH;
    const int cg = threadIdx.x & 7, tl = threadIdx.x >> 3;

    if (threadIdx.x == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        s_fail = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmV);
    }
    __syncthreads();

    // tap weights of this thread's 8 channels, as packed pairs
    f32x2 w2[KT][4];
#pragma unroll
    for (int j = 0; j < KT; ++j)
        bf16x8_to_f32x2(*reinterpret_cast<const uint4*>(p.wconv + j * p.dk + c0 + cg * 8), w2[j]);

    auto issue = [&](int slice, int buf) {
        const int b = slice / p.H, h = slice - b * p.H;
        if (threadIdx.x == 0) {
            mbar_expect_tx(&full[buf], p.slice_bytes);
            tma_load_4d(vs + buf * p.slice_bytes, &tmV, &full[buf], c0, h, 0, b);
        }
        const long long nbase = (long long)slice * nk;
        const uint32_t di = smem_u32(raw_idx + buf * nk), dv = smem_u32(raw_val + buf * nk);
        for (uint32_t e = threadIdx.x; e < nk; e += TPB) {
            cp_async_4(di + 4 * e, p.idx + nbase + e);
            cp_async_4(dv + 4 * e, p.val + nbase + e);
        }
        cp_async_commit();
    };

    int slice = lane_cta;
    if (slice < p.n_slices) issue(slice, 0);
    for (uint32_t it = 0; slice < p.n_slices; slice += p.ctas_per_chunk, ++it) {
        const uint32_t buf = it & 1u;
        const int next = slice + p.ctas_per_chunk;
        if (next < p.n_slices) {
            issue(next, buf ^ 1u);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();                                     // everyone's idx / val copies have landed
        // (offset, weight) pairs, one token per thread
        for (int t = threadIdx.x; t < p.T; t += TPB) {
            float pw[KT];
            token_weights(raw_val + buf * nk + t * KT, pw, KT, p.maximum, p.softmax);
            const int32_t* ni = raw_idx + buf * nk + t * KT;
#pragma unroll
            for (int j = 0; j < KT; ++j) np[t * KT + j] = make_int2(ni[j] * (CH * 2), __float_as_int(pw[j]));
        }
        // the V slice: bounded wait by one thread, outcome shared through the barrier below
        if (threadIdx.x == 0 && !mbar_wait(&full[buf], (it >> 1) & 1u, (volatile int*)&s_fail)) {
            s_fail = 1;
            atomicCAS(&g_dw_stream_status, 0, 31);
        }
        __syncthreads();
        if (s_fail) break;

        const uint8_t* vsb = vs + buf * p.slice_bytes + cg * 16;
        __nv_bfloat16* ob = p.o + (long long)slice * p.T * p.dk + c0 + cg * 8;
        for (int t = tl; t < p.T; t += TOK_PASS) {
            f32x2 acc2[4] = {0ull, 0ull, 0ull, 0ull};
            const int2* nt = np + t * KT;
#pragma unroll
            for (int j = 0; j < KT; ++j) {
                const int2 e = nt[j];
                f32x2 x2[4];
                bf16x8_to_f32x2(*reinterpret_cast<const uint4*>(vsb + e.x), x2);
                const float pj = __int_as_float(e.y);
                const f32x2 p2 = pack2(pj, pj);
#pragma unroll
                for (int q = 0; q < 4; ++q) acc2[q] = fma2(w2[j][q], mul2(p2, x2[q]), acc2[q]);
            }
            *reinterpret_cast<uint4*>(ob + (long long)t * p.dk) = f32x2_to_bf16x8(acc2);
        }
        __syncthreads();                                     // slice and pairs are free for the next copies
    }
    cp_async_wait<0>();
    if (s_fail) {
        // the wait expired: give the copy still in flight time to land before the CTA's shared
        // memory is released
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
}

}  // namespace

// Returns CONVNN_E_UNSUPPORTED (last_error untouched) when the shape does not qualify.
int try_launch_gather_conv_dw_stream(const convnn_desc* d, const Dims& dm, const void* v, const int32_t* idx,
                                     const float* val, const void* w_conv, void* o, cudaStream_t st) {
    static const int env = [] { const char* e = getenv("CONVNN_B200_DW_STREAM"); return e ? atoi(e) : -1; }();
    if (env == 0) return CONVNN_E_UNSUPPORTED;
    if (d->dtype != CONVNN_BF16 || dm.K != KT || dm.dk % CH != 0 || dm.Cp % 8 != 0 || dm.T > 256 || force_simt() ||
        !aligned16(v) || !aligned16(o) || !aligned16(w_conv))
        return CONVNN_E_UNSUPPORTED;
    DwsParams p{};
    p.idx = idx; p.val = val; p.wconv = static_cast<const __nv_bfloat16*>(w_conv);
    p.o = static_cast<__nv_bfloat16*>(o);
    p.T = dm.T; p.H = dm.H; p.dk = dm.dk; p.maximum = d->metric != CONVNN_EUCLIDEAN; p.softmax = d->softmax;
    p.nchunks = dm.dk / CH;
    p.n_slices = dm.B * dm.H;
    p.slice_bytes = (uint32_t)dm.T * CH * 2;
    const size_t nk = (size_t)dm.T * KT;
    const size_t smem = 2 * (size_t)p.slice_bytes + 2 * nk * 4 + 2 * nk * 4 + 8 + nk * 8 + 2 * 8;

    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int per_chunk = (2 * sms) / p.nchunks;
    if (per_chunk < 1) per_chunk = 1;
    if (per_chunk > p.n_slices) per_chunk = p.n_slices;
    p.ctas_per_chunk = per_chunk;

    CUtensorMap tmV;
    const uint64_t dims[4] = {(uint64_t)dm.Cp, (uint64_t)dm.H, (uint64_t)dm.T, (uint64_t)dm.B};
    const uint64_t strides[3] = {(uint64_t)dm.Cp * 2, (uint64_t)dm.H * dm.Cp * 2, (uint64_t)dm.T * dm.H * dm.Cp * 2};
    const uint32_t box[4] = {(uint32_t)CH, 1, (uint32_t)dm.T, 1};
    if (!encode_tensor_map_bf16(&tmV, v, 4, dims, strides, box, 0)) return CONVNN_E_CUDA;

    auto kern = gather_conv_dw_stream_kernel;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    kern<<<per_chunk * p.nchunks, TPB, smem, st>>>(tmV, p);
    CONVNN_CHECK_LAUNCH("gather_conv_dw_stream");
    return CONVNN_OK;
}

int read_dw_stream_status(int* out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_dw_stream_status, sizeof(int));
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    *out = v;
    return CONVNN_OK;
}

}  // namespace convnn
