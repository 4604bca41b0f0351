// Similarity + streaming top-K on the 5th-generation tensor cores (bfloat16 operands).
//
// Work unit = 256 consecutive key tokens (two 128-row MMA tiles) of one (batch, head).
// A persistent CTA walks its units and, per unit, the candidate columns in tiles of
// BN <= 128 (<= 64 in the small launch shape, see below):
//
//   warp 0     TMA producer: per 64-channel chunk two boxes of K rows (128 x 64 each) and
//              ONE box of Q rows (BN x 64) shared by both row tiles, into a 2/3-stage ring
//              (128-byte swizzle), straight from the (B, tokens, H, C) tensors.
//   warp 1     MMA issuer: tcgen05.mma kind::f16, M = 128, N = BN, two accumulators per
//              column tile (one per row tile), double-buffered in TMEM across column tiles
//              (4 x BN columns), so the next tile's MMAs overlap this tile's epilogue.
//   warps 2-5  epilogue of row tile 0, warps 6-9 epilogue of row tile 1: each thread owns
//              one row (= its TMEM lane), pulls 16/32 columns at a time with tcgen05.ld,
//              turns dot products into ranking keys, filters them against the worst kept
//              key (branch-free bit mask) and inserts the survivors into a sorted
//              register list.  The T x S matrix never leaves the SM.
//
// Survivors are inserted in ascending column order with strict comparisons, so exact ties
// keep the lower candidate column.  bfloat16 products are exact in fp32 and accumulation
// is fp32, so the selection is as accurate as the float32 SIMT kernel on the same q, k.
// Every mbarrier wait is bounded; on expiry the CTA latches a code and drains.
#include "common.cuh"
#include "sm100.cuh"
#include "toplist.cuh"
#include "sim_topk_select.cuh"

namespace convnn {

__device__ int g_sim_topk_status = 0;

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int MAX_STAGES = 3;
constexpr int NTHREADS = 320;     // TMA warp, MMA warp, 2 x 4 epilogue warps
constexpr int GROUP = kSelGroup;  // threads per epilogue group
// Two launch shapes.  SMALL (short candidate lists, d_k <= 256, or <= 512 on short sequences): BN <= 64, 2 stages, 16-column
// epilogue chunks and two CTAs per SM, so four epilogue warps per scheduler hide each other's
// latency -- this regime is bound by the selection, not by the MMAs.  LARGE: BN <= 128, 3 stages,
// one CTA per SM, for long sequences where the tensor pipe is the limiter.

struct TcParams {
    const float* qstat;
    const float* kstat;
    const int32_t* cand;
    int32_t* idx;
    float* val;
    int T, S, H, K, nsel, metric, sampled;
    int KCH;          // channels per shared-memory chunk (64, 32 or 16)
    int KC;           // chunks per tile = C / KCH
    int BN;           // candidate columns per MMA (multiple of 16, <= 128)
    int BNpad;        // TMEM columns per accumulator (power of two >= BN)
    int stages;       // shared-memory ring depth (<= MAX_STAGES)
    int n_pairs, n_col_tiles, n_units;
    float sqrt_dk;
};

__device__ __forceinline__ void fail(volatile int* abort_flag, int code) {
    *abort_flag = 1;
    atomicCAS(&g_sim_topk_status, 0, code);
}

template <int NSEL, int MINB, int CW>
__global__ void __launch_bounds__(NTHREADS, MINB)
sim_topk_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ,
                   const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t pitch = p.KCH * 2;
    const uint32_t a_bytes = BM * pitch, b_bytes = p.BN * pitch;
    const uint32_t stage_bytes = 2 * a_bytes + b_bytes;
    const uint32_t STAGES = p.stages;
    uint8_t* stages = smem;                                            // [STAGES][A0 | A1 | B]
    float* keybuf = reinterpret_cast<float*>(smem + STAGES * stage_bytes);   // [2 groups][CW][GROUP]
    float* statbuf = keybuf + 2 * CW * GROUP;                                 // [8 warps][128] column statistics of the tile
    uint64_t* bars = reinterpret_cast<uint64_t*>(statbuf + 8 * 128);
    uint64_t* full = bars;
    uint64_t* empty = bars + MAX_STAGES;
    uint64_t* tfull = bars + 2 * MAX_STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ncols = 4u * p.BNpad;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 8);
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

    const uint32_t full0 = smem_u32(full), empty0 = smem_u32(empty);
    const uint32_t st0 = smem_u32(stages);

    if (warp == 0) {
        // One thread can start a TMA operation only every ~0.3 us whatever its size, while operations started
        // by different lanes overlap: the three boxes of a stage (two key tiles, one query tile) are issued by
        // lanes 0, 1 and 2 with one instruction of the warp (a unit of the ViT shape has 36 of them).
        if (lane < 3) {
            const uint32_t m3 = 0x7u;
            uint32_t s = 0, ph = 0;                  // ring slot and phase, advanced incrementally
            bool ok = true;
            for (int unit = blockIdx.x; unit < p.n_units && ok; unit += gridDim.x) {
                const int bh = unit / p.n_pairs, pp = unit - bh * p.n_pairs;
                const int b = bh / p.H, h = bh - b * p.H;
                const int row0 = pp * 2 * BM;
                const bool has1 = row0 + BM < p.T;
                const uint32_t tx = (has1 ? 2u : 1u) * a_bytes + b_bytes;
                for (int ct = 0; ct < p.n_col_tiles && ok; ++ct) {
                    const int col0 = ct * p.BN;
                    for (int kc = 0; kc < p.KC; ++kc) {
                        ok = mbar_wait_a(empty0 + 8 * s, ph ^ 1u, abort_flag);
                        ok = __all_sync(m3, ok);
                        if (!ok) { if (lane == 0) fail(abort_flag, 1); break; }
                        const uint32_t st = st0 + s * stage_bytes, fb = full0 + 8 * s;
                        if (lane == 0) mbar_expect_tx_a(fb, tx);
                        __syncwarp(m3);
                        if (lane == 0) tma_load_4d_a(st, &tmK, fb, kc * p.KCH, h, row0, b);
                        else if (lane == 1) { if (has1) tma_load_4d_a(st + a_bytes, &tmK, fb, kc * p.KCH, h, row0 + BM, b); }
                        else tma_load_4d_a(st + 2 * a_bytes, &tmQ, fb, kc * p.KCH, h, col0, b);
                        if (++s == STAGES) { s = 0; ph ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc_bf16_f32(BM, p.BN);
            const uint64_t dhi = kmajor_desc_hi(pitch);
            const int nk16 = p.KCH / 16;
            const uint32_t tfull0 = smem_u32(tfull), tempty0 = smem_u32(tempty);
            uint32_t s = 0, ph = 0, tile = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < p.n_units && ok; unit += gridDim.x) {
                const int pp = unit % p.n_pairs;
                const bool has1 = pp * 2 * BM + BM < p.T;
                for (int ct = 0; ct < p.n_col_tiles && ok; ++ct, ++tile) {
                    const uint32_t par = tile & 1u, u = tile >> 1;
                    if (!mbar_wait_a(tempty0 + 8 * par, (u & 1u) ^ 1u, abort_flag)) { fail(abort_flag, 2); ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t d0 = tmem_base + par * p.BNpad;
                    const uint32_t d1 = tmem_base + (2 + par) * p.BNpad;
                    for (int kc = 0; kc < p.KC; ++kc) {
                        if (!mbar_wait_a(full0 + 8 * s, ph, abort_flag)) { fail(abort_flag, 3); ok = false; break; }
                        tc_fence_after_sync();
                        const uint32_t sa = st0 + s * stage_bytes;
                        const uint64_t a0 = dhi | (uint64_t)(sa >> 4);
                        const uint64_t a1 = dhi | (uint64_t)((sa + a_bytes) >> 4);
                        const uint64_t bd = dhi | (uint64_t)((sa + 2 * a_bytes) >> 4);
                        mma_chunk(d0, a0, bd, idesc, nk16, kc != 0);
                        if (has1) mma_chunk(d1, a1, bd, idesc, nk16, kc != 0);
                        mma_commit_a(empty0 + 8 * s);
                        if (++s == STAGES) { s = 0; ph ^= 1u; }
                    }
                    if (ok) mma_commit_a(tfull0 + 8 * par);
                }
            }
        }
    } else {
        const int grp = (warp - 2) >> 2;         // which row tile of the pair this warp serves
        const int lq = warp & 3;                 // TMEM lane quarter this warp may read
        const int r = lq * 32 + lane;            // row within the tile
        float* ks = keybuf + grp * CW * GROUP + r;
        float* sq = statbuf + (warp - 2) * 128;
        uint32_t tile = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < p.n_units && ok; unit += gridDim.x) {
            const int bh = unit / p.n_pairs, pp = unit - bh * p.n_pairs;
            const int row = pp * 2 * BM + grp * BM + r;
            const bool row_ok = row < p.T;
            const float* qs_row = p.qstat ? p.qstat + (long long)bh * p.S : nullptr;
            float kst = 1.0f;
            if (row_ok && p.metric != CONVNN_MATMUL) kst = p.kstat[(long long)bh * p.T + row];
            const float sentinel = p.sampled ? self_sentinel(p.metric, kst, p.sqrt_dk) : 0.f;
            TopList<NSEL> top;
            top.init();
            // column statistics (4 x 32 columns cover BN <= 128), fetched one tile ahead
            float qv[4], qn[4];
            int cv[4], cn[4];
            auto fetch = [&](int ct, float (&fq)[4], int (&fc)[4]) {
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    const int cl = min(ct * p.BN + c4 * 32 + lane, p.S - 1);
                    fq[c4] = (p.metric != CONVNN_MATMUL && c4 * 32 < p.BN) ? qs_row[cl] : 0.f;
                    fc[c4] = (p.sampled && c4 * 32 < p.BN) ? p.cand[cl] : -1;
                }
            };
            fetch(0, qv, cv);
            for (int ct = 0; ct < p.n_col_tiles && ok; ++ct, ++tile) {
                const uint32_t par = tile & 1u, u = tile >> 1;
                if (ct + 1 < p.n_col_tiles) fetch(ct + 1, qn, cn);
                ok = mbar_wait(&tfull[par], u & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { if (lane == 0) fail(abort_flag, 4); break; }
                tc_fence_after_sync();
                const uint32_t taddr = tmem_base + ((uint32_t)(lq * 32) << 16) + (grp * 2 + par) * p.BNpad;
                // a warp whose 32 rows all lie past the end of the sequence has nothing to select
                const bool warp_live = pp * 2 * BM + grp * BM + lq * 32 < p.T;
                auto cand_of = [&](int c) {
                    const int c4 = c >> 5;
                    return c4 == 0 ? cv[0] : (c4 == 1 ? cv[1] : (c4 == 2 ? cv[2] : cv[3]));
                };
                // this tile's column statistics, readable by every lane as broadcast vectors
                __syncwarp();
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) sq[c4 * 32 + lane] = qv[c4];
                __syncwarp();
                if (warp_live) {
#pragma unroll 1
                    for (int c = 0; c < p.BN; c += CW) {
                        if (ct * p.BN + c >= p.S) break;         // the rest of the tile is padding
                        const int c1 = cand_of(c);
                        if (CW == 32 && c + 32 <= p.BN) {
                            uint32_t acc[32];
                            tmem_ld_x32(taddr + c, acc);
                            tmem_ld_wait();
                            consume<NSEL, 32>(top, acc, ct * p.BN + c, 0, sq + c, c1, p, row, row_ok, sentinel, ks);
                        } else {
                            uint32_t acc[16];
                            tmem_ld_x16(taddr + c, acc);
                            tmem_ld_wait();
                            consume<NSEL, 16>(top, acc, ct * p.BN + c, c & 31, sq + c, c1, p, row, row_ok, sentinel, ks);
                        }
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tempty[par]);
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) { qv[c4] = qn[c4]; cv[c4] = cn[c4]; }
            }
            if (ok && row_ok) {
                write_selection<NSEL>(top, p, ((long long)bh * p.T + row) * p.K, row, kst);
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
    if (sim_topk_tc2_wanted(d, dm)) return launch_sim_topk_tc2(d, dm, q, k, qstat, kstat, cand, idx, val, st);
    TcParams p{};
    p.qstat = qstat; p.kstat = kstat; p.cand = cand; p.idx = idx; p.val = val;
    p.T = dm.T; p.S = dm.S; p.H = dm.H; p.K = dm.K; p.nsel = dm.nsel; p.metric = d->metric; p.sampled = d->sampled;
    p.KCH = dm.Cp % 64 == 0 ? 64 : (dm.Cp % 32 == 0 ? 32 : 16);
    p.KC = dm.Cp / p.KCH;
    // (heads of 257-512 channels on short sequences: 19.3 against 22.8 us at B=256, T=197, S=64, d_k=384;
    // with 768 channels the small shape measured slower)
    const bool small_cfg = dm.nsel <= 12 && (dm.Cp <= 256 || (dm.Cp <= 512 && dm.T <= 512));
    const int bn_cap = small_cfg ? 64 : 128;
    p.stages = small_cfg ? 2 : 3;
    const int ntile = (dm.S + bn_cap - 1) / bn_cap;
    p.BN = (((dm.S + ntile - 1) / ntile) + 15) / 16 * 16;
    p.BNpad = pow2_at_least(p.BN, 32);
    p.n_pairs = (dm.T + 2 * BM - 1) / (2 * BM);
    p.n_col_tiles = (dm.S + p.BN - 1) / p.BN;
    p.n_units = dm.B * dm.H * p.n_pairs;
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

    const int cw = small_cfg ? 16 : 32;
    const size_t smem = 1024 + (size_t)p.stages * (2 * BM + p.BN) * pitch + 2 * cw * GROUP * sizeof(float) +
                        8 * 128 * sizeof(float) + (2 * MAX_STAGES + 4) * 8 + 16;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int ctas = sms * (small_cfg ? 2 : 1);
    const int grid = p.n_units < ctas ? p.n_units : ctas;

#define CONVNN_TC_LAUNCH2(N, MINB, CWV)                                                                \
    do {                                                                                               \
        auto kern = sim_topk_tc_kernel<N, MINB, CWV>;                                                  \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        kern<<<grid, NTHREADS, smem, st>>>(tmK, tmQ, p);                                               \
    } while (0)
#define CONVNN_TC_LAUNCH(N)                            \
    do {                                               \
        if (small_cfg) CONVNN_TC_LAUNCH2(N, 2, 16);    \
        else CONVNN_TC_LAUNCH2(N, 1, 32);              \
    } while (0)
    const int n = dm.nsel;
    if (n <= 4) CONVNN_TC_LAUNCH(4);
    else if (n <= 8) CONVNN_TC_LAUNCH(8);
    else if (n == 9) CONVNN_TC_LAUNCH(9);
    else if (n <= 12) CONVNN_TC_LAUNCH(12);
    else if (n <= 16) CONVNN_TC_LAUNCH2(16, 1, 32);
    else if (n <= 24) CONVNN_TC_LAUNCH2(24, 1, 32);
    else if (n == 25) CONVNN_TC_LAUNCH2(25, 1, 32);
    else CONVNN_TC_LAUNCH2(32, 1, 32);
#undef CONVNN_TC_LAUNCH
#undef CONVNN_TC_LAUNCH2
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
