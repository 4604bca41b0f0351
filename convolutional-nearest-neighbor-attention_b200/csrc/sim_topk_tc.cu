// Similarity + streaming top-K on the 5th-generation tensor cores (bfloat16 operands).
//
// Work item = 128 consecutive key tokens (rows) of one (batch, head).  A persistent CTA
// walks its items and, per item, the candidate columns in tiles of BN <= 256:
//
//   warp 0   TMA producer: per 64-channel chunk, one box of K rows (128 x 64) and one box
//            of Q rows (BN x 64) into a 4-stage shared-memory ring (128-byte swizzle),
//            straight from the (B, tokens, H, C) tensors -- no head-split copies.
//   warp 1   MMA issuer: tcgen05.mma kind::f16, M = 128, N = BN, fp32 accumulators in one
//            of two TMEM buffers, so the next tile's MMAs overlap this tile's epilogue;
//            tcgen05.commit hands the smem stage back and publishes the accumulator.
//   warps 2-5  epilogue: each thread owns one row (= its TMEM lane), pulls 32 columns at a
//            time with tcgen05.ld, converts dot products to ranking keys and keeps a
//            sorted register list of the best candidates.  The T x S matrix never leaves
//            the SM.
//
// bfloat16 products are exact in fp32 and accumulation is fp32, so the selection is as
// accurate as the SIMT float32 kernel on the same (rounded) q and k.  Every mbarrier wait
// is bounded; on expiry the CTA records a code in the device status word and drains.
#include "common.cuh"
#include "sm100.cuh"
#include "toplist.cuh"

namespace convnn {

__device__ int g_sim_topk_status = 0;

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int STAGES = 4;
constexpr int NTHREADS = 192;

struct TcParams {
    const float* qstat;
    const float* kstat;
    const int32_t* cand;
    int32_t* idx;
    float* val;
    int T, S, H, K, nsel, metric, sampled;
    int KCH;          // channels per shared-memory chunk (64, 32 or 16)
    int KC;           // chunks per tile = C / KCH
    int BN;           // candidate columns per MMA (multiple of 16, <= 256)
    int BNpad;        // TMEM columns per accumulator buffer (power of two >= BN)
    int n_row_tiles, n_col_tiles, n_items;
    float sqrt_dk;
};

__device__ __forceinline__ void fail(volatile int* abort_flag, int code) {
    *abort_flag = 1;
    atomicCAS(&g_sim_topk_status, 0, code);
}

template <int NSEL, int W>
__device__ __forceinline__ void consume(TopList<NSEL>& top, const uint32_t (&r)[W], int col0, float qv, int cv,
                                        const TcParams& p, int row, bool row_ok, float sentinel) {
#pragma unroll
    for (int j = 0; j < W; ++j) {
        const float dot = __uint_as_float(r[j]);
        float key = dot;
        if (p.metric != CONVNN_MATMUL) {
            const float s = __shfl_sync(0xffffffffu, qv, j);
            key = (p.metric == CONVNN_COSINE) ? dot * s : fmaf(2.0f, dot, -s);
        }
        if (p.sampled) {
            const int cj = __shfl_sync(0xffffffffu, cv, j);
            if (cj == row) key = sentinel;
        }
        if (row_ok && (col0 + j) < p.S && key > top.worst()) top.insert(key, col0 + j);
    }
}

template <int NSEL>
__global__ void __launch_bounds__(NTHREADS, 1)
sim_topk_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ,
                   const TcParams p) {
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
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmQ);
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
            for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
                const int bh = item / p.n_row_tiles, rt = item - bh * p.n_row_tiles;
                const int b = bh / p.H, h = bh - b * p.H;
                for (int ct = 0; ct < p.n_col_tiles && ok; ++ct) {
                    for (int kc = 0; kc < p.KC; ++kc, ++it) {
                        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                        if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { fail(abort_flag, 1); ok = false; break; }
                        mbar_expect_tx(&full[s], a_bytes + b_bytes);
                        tma_load_4d(sA + s * a_bytes, &tmK, &full[s], kc * p.KCH, h, rt * BM, b);
                        tma_load_4d(sB + s * b_bytes, &tmQ, &full[s], kc * p.KCH, h, ct * p.BN, b);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc_bf16_f32(BM, p.BN);
            uint32_t it = 0, tile = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
                for (int ct = 0; ct < p.n_col_tiles && ok; ++ct, ++tile) {
                    const uint32_t buf = tile & 1u, u = tile >> 1;
                    if (!mbar_wait(&tempty[buf], (u & 1u) ^ 1u, abort_flag)) { fail(abort_flag, 2); ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * p.BNpad;
                    for (int kc = 0; kc < p.KC; ++kc, ++it) {
                        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                        if (!mbar_wait(&full[s], ph, abort_flag)) { fail(abort_flag, 3); ok = false; break; }
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
        }
    } else {
        const int lq = warp & 3;                 // TMEM lane quarter this warp may read
        const int r = lq * 32 + lane;            // row within the tile
        uint32_t tile = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
            const int bh = item / p.n_row_tiles, rt = item - bh * p.n_row_tiles;
            const int row = rt * BM + r;
            const bool row_ok = row < p.T;
            const float* qs_row = p.qstat ? p.qstat + (long long)bh * p.S : nullptr;
            float kst = 1.0f;
            if (row_ok && p.metric != CONVNN_MATMUL) kst = p.kstat[(long long)bh * p.T + row];
            float sentinel = 0.f;
            if (p.sampled) {
                if (p.metric == CONVNN_COSINE) sentinel = -0.1f / kst;
                else if (p.metric == CONVNN_MATMUL) sentinel = -0.1f * p.sqrt_dk;
                else sentinel = kst - 1.21f;
            }
            TopList<NSEL> top;
            top.init();
            for (int ct = 0; ct < p.n_col_tiles && ok; ++ct, ++tile) {
                const uint32_t buf = tile & 1u, u = tile >> 1;
                ok = mbar_wait(&tfull[buf], u & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { if (lane == 0) fail(abort_flag, 4); break; }
                tc_fence_after_sync();
                const uint32_t taddr = tmem_base + ((uint32_t)(lq * 32) << 16) + buf * p.BNpad;
                int c = 0;
                for (; c + 32 <= p.BN; c += 32) {
                    const int col0 = ct * p.BN + c;
                    const int cl = min(col0 + lane, p.S - 1);
                    const float qv = (p.metric != CONVNN_MATMUL) ? qs_row[cl] : 0.f;
                    const int cv = p.sampled ? p.cand[cl] : -1;
                    uint32_t acc[32];
                    tmem_ld_x32(taddr + c, acc);
                    tmem_ld_wait();
                    consume<NSEL, 32>(top, acc, col0, qv, cv, p, row, row_ok, sentinel);
                }
                if (c < p.BN) {
                    const int col0 = ct * p.BN + c;
                    const int cl = min(col0 + (lane & 15), p.S - 1);
                    const float qv = (p.metric != CONVNN_MATMUL) ? qs_row[cl] : 0.f;
                    const int cv = p.sampled ? p.cand[cl] : -1;
                    uint32_t acc[16];
                    tmem_ld_x16(taddr + c, acc);
                    tmem_ld_wait();
                    consume<NSEL, 16>(top, acc, col0, qv, cv, p, row, row_ok, sentinel);
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tempty[buf]);
            }
            if (ok && row_ok) {
                const long long obase = ((long long)bh * p.T + row) * p.K;
                int off = 0;
                if (p.sampled) {
                    p.idx[obase] = row;
                    p.val[obase] = 1.0f;
                    off = 1;
                }
#pragma unroll
                for (int s = 0; s < NSEL; ++s) {
                    if (s < p.nsel) {
                        const int col = top.i[s];
                        const float key = top.v[s];
                        float v;
                        if (p.metric == CONVNN_COSINE) v = key * kst;
                        else if (p.metric == CONVNN_MATMUL) v = key / p.sqrt_dk;
                        else v = sqrtf(fmaxf(kst - key, 0.f));
                        int tok = col;
                        if (p.sampled) {
                            tok = p.cand[col];
                            if (tok == row) v = (p.metric == CONVNN_EUCLIDEAN) ? 1.1f : -0.1f;
                        }
                        p.idx[obase + off + s] = tok;
                        p.val[obase + off + s] = v;
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // a wait expired: give copies still in flight time to land before the CTA's shared
        // memory is released
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

bool sim_topk_tc_supported(const convnn_desc* d, const Dims& dm, const void* q, const void* k) {
    return d->dtype == CONVNN_BF16 && dm.Cp % 16 == 0 && aligned16(q) && aligned16(k);
}

int launch_sim_topk_tc(const convnn_desc* d, const Dims& dm, const void* q, const void* k, const float* qstat,
                       const float* kstat, const int32_t* cand, int32_t* idx, float* val, cudaStream_t st) {
    TcParams p{};
    p.qstat = qstat; p.kstat = kstat; p.cand = cand; p.idx = idx; p.val = val;
    p.T = dm.T; p.S = dm.S; p.H = dm.H; p.K = dm.K; p.nsel = dm.nsel; p.metric = d->metric; p.sampled = d->sampled;
    p.KCH = dm.Cp % 64 == 0 ? 64 : (dm.Cp % 32 == 0 ? 32 : 16);
    p.KC = dm.Cp / p.KCH;
    const int ntile = (dm.S + 255) / 256;
    p.BN = (((dm.S + ntile - 1) / ntile) + 15) / 16 * 16;
    p.BNpad = pow2_at_least(p.BN, 32);
    p.n_row_tiles = (dm.T + BM - 1) / BM;
    p.n_col_tiles = (dm.S + p.BN - 1) / p.BN;
    p.n_items = dm.B * dm.H * p.n_row_tiles;
    p.sqrt_dk = (float)sqrt((double)dm.dk);

    const int pitch = p.KCH * 2;
    CUtensorMap tmK, tmQ;
    const uint64_t dimsK[4] = {(uint64_t)dm.Cp, (uint64_t)dm.H, (uint64_t)dm.T, (uint64_t)dm.B};
    const uint64_t dimsQ[4] = {(uint64_t)dm.Cp, (uint64_t)dm.H, (uint64_t)dm.S, (uint64_t)dm.B};
    const uint64_t strK[3] = {(uint64_t)dm.Cp * 2, (uint64_t)dm.H * dm.Cp * 2, (uint64_t)dm.T * dm.H * dm.Cp * 2};
    const uint64_t strQ[3] = {(uint64_t)dm.Cp * 2, (uint64_t)dm.H * dm.Cp * 2, (uint64_t)dm.S * dm.H * dm.Cp * 2};
    const uint32_t boxK[4] = {(uint32_t)p.KCH, 1, (uint32_t)BM, 1};
    const uint32_t boxQ[4] = {(uint32_t)p.KCH, 1, (uint32_t)p.BN, 1};
    if (!encode_tensor_map_bf16(&tmK, k, 4, dimsK, strK, boxK, pitch)) return CONVNN_E_CUDA;
    if (!encode_tensor_map_bf16(&tmQ, q, 4, dimsQ, strQ, boxQ, pitch)) return CONVNN_E_CUDA;

    const size_t smem = 1024 + (size_t)STAGES * (BM + p.BN) * pitch + (2 * STAGES + 4) * 8 + 16;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = p.n_items < sms ? p.n_items : sms;

#define CONVNN_TC_LAUNCH(N)                                                                            \
    do {                                                                                               \
        auto kern = sim_topk_tc_kernel<N>;                                                             \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        kern<<<grid, NTHREADS, smem, st>>>(tmK, tmQ, p);                                               \
    } while (0)
    const int n = dm.nsel;
    if (n <= 4) CONVNN_TC_LAUNCH(4);
    else if (n <= 8) CONVNN_TC_LAUNCH(8);
    else if (n == 9) CONVNN_TC_LAUNCH(9);
    else if (n <= 12) CONVNN_TC_LAUNCH(12);
    else if (n <= 16) CONVNN_TC_LAUNCH(16);
    else if (n <= 24) CONVNN_TC_LAUNCH(24);
    else if (n == 25) CONVNN_TC_LAUNCH(25);
    else CONVNN_TC_LAUNCH(32);
#undef CONVNN_TC_LAUNCH
    CONVNN_CHECK_LAUNCH("sim_topk_tc");
    return CONVNN_OK;
}

int read_sim_topk_status(int* out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_sim_topk_status, sizeof(int));
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    *out = v;
    return CONVNN_OK;
}

}  // namespace convnn
