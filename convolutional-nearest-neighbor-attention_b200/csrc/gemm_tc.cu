// bfloat16 GEMM  C = A * W^T (+ bias, + GELU)  on the 5th-generation tensor cores, used
// for the Q/K/V projections, the output projection, the pointwise stage of the separable
// conv and the Linear layers around the ConvNN block.
//
// A is (M, Kd) row-major with row stride lda, W is (N, Kd) row-major (nn.Linear layout):
// both are K-major operands, so TMA boxes of [rows x 64 channels] with the 128-byte
// swizzle feed tcgen05.mma directly.  A persistent CTA walks 128 x BN output tiles
// (n fastest, so the CTAs of a wave share a handful of A row blocks and all of W in L2):
//   warp 0     TMA producer, 4-stage ring of (A chunk, W chunk) pairs
//   warp 1     MMA issuer, fp32 accumulators double-buffered in TMEM
//   warps 2-5  epilogue: tcgen05.ld -> (+bias, GELU) -> bf16 -> 16-byte global stores
// The N range may be split into up to three equal parts with their own output tensors,
// which lets one launch produce k, v and q from the packed [W_k; W_v; W_q].
// Every mbarrier wait is bounded (see sm100.cuh); an expiry latches the device status.
#include "common.cuh"
#include "sm100.cuh"

namespace convnn {

__device__ int g_gemm_tc_status = 0;   // error latch of this translation unit

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int STAGES = 4;
constexpr int NTHREADS = 192;

struct GemmTcParams {
    __nv_bfloat16* c[3];
    long long ldc;
    const __nv_bfloat16* bias;
    int part_cols;         // output columns per part (N for a single output)
    int M, N, gelu;
    int KCH, KC, BN, BNpad;
    int n_m_tiles, n_n_tiles, n_tiles;
};

__device__ __forceinline__ void fail(volatile int* abort_flag, int code) {
    *abort_flag = 1;
    atomicCAS(&g_gemm_tc_status, 0, code);
}

__device__ __forceinline__ float gelu_exact(float x) {
    return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
}

// Convert W fp32 accumulators (+bias, GELU) to bf16 and store the first `valid` (a multiple
// of 8) of them at dst (16-byte aligned).
template <int W>
__device__ __forceinline__ void store_chunk(__nv_bfloat16* dst, const uint32_t (&acc)[W], const __nv_bfloat16* bias,
                                            int gelu, int valid) {
#pragma unroll
    for (int g = 0; g < W / 8; ++g) {
        if (g * 8 >= valid) break;
        uint4 packed;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float a = __uint_as_float(acc[g * 8 + 2 * e]);
            float b = __uint_as_float(acc[g * 8 + 2 * e + 1]);
            if (bias) {
                a += __bfloat162float(bias[g * 8 + 2 * e]);
                b += __bfloat162float(bias[g * 8 + 2 * e + 1]);
            }
            if (gelu) { a = gelu_exact(a); b = gelu_exact(b); }
            h[e] = __floats2bfloat162_rn(a, b);
        }
        *reinterpret_cast<uint4*>(dst + g * 8) = packed;   // N % 8 == 0: no ragged group
    }
}

__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
               const GemmTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t pitch = p.KCH * 2;
    const uint32_t a_bytes = BM * pitch, b_bytes = p.BN * pitch;
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * a_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * b_bytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* tfull = bars + 2 * STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ncols = 2u * p.BNpad;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmW);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, ncols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
                const int mt = t / p.n_n_tiles, nt = t - mt * p.n_n_tiles;
                for (int kc = 0; kc < p.KC; ++kc, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { fail(abort_flag, 11); ok = false; break; }
                    mbar_expect_tx(&full[s], a_bytes + b_bytes);
                    tma_load_2d(sA + s * a_bytes, &tmA, &full[s], kc * p.KCH, mt * BM);
                    tma_load_2d(sB + s * b_bytes, &tmW, &full[s], kc * p.KCH, nt * p.BN);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc_bf16_f32(BM, p.BN);
            uint32_t it = 0, tile = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, ++tile) {
                const uint32_t buf = tile & 1u, u = tile >> 1;
                if (!mbar_wait(&tempty[buf], (u & 1u) ^ 1u, abort_flag)) { fail(abort_flag, 12); ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * p.BNpad;
                for (int kc = 0; kc < p.KC; ++kc, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    if (!mbar_wait(&full[s], ph, abort_flag)) { fail(abort_flag, 13); ok = false; break; }
                    tc_fence_after_sync();
                    const uint64_t adesc = make_kmajor_desc(smem_u32(sA + s * a_bytes), pitch);
                    const uint64_t bdesc = make_kmajor_desc(smem_u32(sB + s * b_bytes), pitch);
                    for (int k16 = 0; k16 < p.KCH / 16; ++k16)
                        mma_bf16_ss(d_tmem, adesc + 2u * k16, bdesc + 2u * k16, idesc, (kc | k16) != 0);
                    mma_commit(&empty[s]);
                }
                if (ok) mma_commit(&tfull[buf]);
            }
        }
    } else {
        const int lq = warp & 3;
        const int r = lq * 32 + lane;
        uint32_t tile = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, ++tile) {
            const int mt = t / p.n_n_tiles, nt = t - mt * p.n_n_tiles;
            const uint32_t buf = tile & 1u, u = tile >> 1;
            const int row = mt * BM + r;
            const int n0 = nt * p.BN;
            const int part = n0 / p.part_cols;
            const int pc0 = n0 - part * p.part_cols;          // first column inside the part
            __nv_bfloat16* cbase = part == 0 ? p.c[0] : (part == 1 ? p.c[1] : p.c[2]);
            __nv_bfloat16* crow = cbase + (long long)row * p.ldc + pc0;
            const __nv_bfloat16* brow = p.bias ? p.bias + n0 : nullptr;
            const int ncol = min(p.BN, p.N - n0);             // valid columns of this tile
            ok = mbar_wait(&tfull[buf], u & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) fail(abort_flag, 14); break; }
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(lq * 32) << 16) + buf * p.BNpad;
            int c = 0;
            for (; c + 32 <= p.BN; c += 32) {
                uint32_t acc[32];
                tmem_ld_x32(taddr + c, acc);
                tmem_ld_wait();
                if (row < p.M && c < ncol) store_chunk<32>(crow + c, acc, brow ? brow + c : nullptr, p.gelu, ncol - c);
            }
            if (c < p.BN) {
                uint32_t acc[16];
                tmem_ld_x16(taddr + c, acc);
                tmem_ld_wait();
                if (row < p.M && c < ncol) store_chunk<16>(crow + c, acc, brow ? brow + c : nullptr, p.gelu, ncol - c);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[buf]);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, ncols);
    }
}

int pow2_at_least(int v, int lo) {
    int r = lo;
    while (r < v) r <<= 1;
    return r;
}

}  // namespace

// Largest tile width <= 256 that is a multiple of 16 and divides `cols`; 0 if none.
static int dividing_tile(int cols) {
    for (int bn = 256; bn >= 16; bn -= 16)
        if (cols % bn == 0) return bn;
    return 0;
}

bool gemm_tc_supported(const void* a, long long lda, const void* w, int Kd, int N, int parts, const void* const* c,
                       long long ldc) {
    if (Kd % 16 != 0 || lda % 8 != 0 || ldc % 8 != 0 || !aligned16(a) || !aligned16(w)) return false;
    for (int i = 0; i < parts; ++i)
        if (!aligned16(c[i])) return false;
    if (parts > 1) return N % parts == 0 && dividing_tile(N / parts) != 0;
    return N % 8 == 0;
}

int launch_gemm_tc(const void* a, long long lda, const void* w, const void* bias, int M, int N, int Kd, int parts,
                   void* const* c, long long ldc, int gelu, cudaStream_t st) {
    GemmTcParams p{};
    for (int i = 0; i < 3; ++i) p.c[i] = static_cast<__nv_bfloat16*>(c[i < parts ? i : 0]);
    p.ldc = ldc; p.bias = static_cast<const __nv_bfloat16*>(bias); p.gelu = gelu;
    p.M = M; p.N = N;
    p.part_cols = N / parts;
    p.KCH = Kd % 64 == 0 ? 64 : (Kd % 32 == 0 ? 32 : 16);
    p.KC = Kd / p.KCH;
    if (parts > 1) {
        p.BN = dividing_tile(p.part_cols);
    } else {
        const int nt = (N + 255) / 256;
        p.BN = (((N + nt - 1) / nt) + 15) / 16 * 16;
    }
    p.BNpad = pow2_at_least(p.BN, 32);
    p.n_m_tiles = (M + BM - 1) / BM;
    p.n_n_tiles = (N + p.BN - 1) / p.BN;
    p.n_tiles = p.n_m_tiles * p.n_n_tiles;

    const int pitch = p.KCH * 2;
    CUtensorMap tmA, tmW;
    const uint64_t dimsA[2] = {(uint64_t)Kd, (uint64_t)M}, dimsW[2] = {(uint64_t)Kd, (uint64_t)N};
    const uint64_t strA[1] = {(uint64_t)lda * 2}, strW[1] = {(uint64_t)Kd * 2};
    const uint32_t boxA[2] = {(uint32_t)p.KCH, (uint32_t)BM}, boxW[2] = {(uint32_t)p.KCH, (uint32_t)p.BN};
    if (!encode_tensor_map_bf16(&tmA, a, 2, dimsA, strA, boxA, pitch)) return CONVNN_E_CUDA;
    if (!encode_tensor_map_bf16(&tmW, w, 2, dimsW, strW, boxW, pitch)) return CONVNN_E_CUDA;

    const size_t smem = 1024 + (size_t)STAGES * (BM + p.BN) * pitch + (2 * STAGES + 4) * 8 + 16;
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = p.n_tiles < sms ? p.n_tiles : sms;
    gemm_tc_kernel<<<grid, NTHREADS, smem, st>>>(tmA, tmW, p);
    CONVNN_CHECK_LAUNCH("gemm_tc");
    return CONVNN_OK;
}

int read_gemm_tc_status(int* out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_gemm_tc_status, sizeof(int));
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    *out = v;
    return CONVNN_OK;
}

}  // namespace convnn
