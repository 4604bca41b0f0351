// Similarity + streaming top-K for long sequences on CTA pairs (tcgen05 cta_group::2).
//
// The single-CTA kernel streams a 128 x 16 slice of K rows and a 128 x 16 slice of Q rows
// out of shared memory for every 64 tensor-core cycles, which is the whole shared-memory
// port; on long sequences that, not the tensor pipe, is what bounds it.  Here two CTAs of a
// cluster form one MMA unit: a work unit is 256 key rows (128 per CTA) of one (batch,
// head), a column tile is 256 candidates of which each CTA stages HALF (128 Q rows), and
// one M = 256, N = 256, K = 16 MMA per pair reads 4 KB + 4 KB per CTA for 128 cycles of
// work: half the operand bytes per flop, and half the TMA fill per flop as well.
//
// Per CTA:  warp 0 lane 0   TMA producer (own K rows, own half of the Q rows) into a 5-stage
//                           ring; every load credits the LEADER's "full" barrier
//           warp 1 lane 0   leader only: MMA issuer; two 256-column fp32 accumulators in
//                           TMEM (ping-pong across column tiles); completions are committed
//                           to the barriers of both CTAs, one commit each
//           warps 2-5       selection over columns 0-127 of each tile, thread = key row
//           warps 6-9       selection over columns 128-255; the two lists of a row are merged
//                           through shared memory at the end of the unit (mbarrier hand-over)
// Every wait on an mbarrier is bounded; an expiry latches a status code, raises the abort
// flag of both CTAs and lets every role run to the common exit (cluster barrier, TMEM free).
#include <atomic>

#include "common.cuh"
#include "sm100.cuh"
#include "toplist.cuh"
#include "sim_topk_select.cuh"

namespace convnn {

__device__ int g_sim_topk2_status = 0;

namespace {

using namespace sm100;

constexpr int BM = 128;            // key rows per CTA
constexpr int BNH = 128;           // candidate columns staged per CTA
constexpr int BN = 2 * BNH;        // candidate columns per MMA / column tile
constexpr int KCH = 64;            // channels per shared-memory chunk (128-byte rows)
constexpr int STAGES = 5;
constexpr int NTHREADS = 320;
constexpr int CW = 32;             // accumulator columns per tcgen05.ld
constexpr uint32_t A_BYTES = BM * KCH * 2, B_BYTES = BNH * KCH * 2, STAGE_BYTES = A_BYTES + B_BYTES;

struct Tc2Params {
    const float* qstat;
    const float* kstat;
    const int32_t* cand;
    int32_t* idx;
    float* val;
    int T, S, H, K, nsel, metric, sampled;
    int KC;                        // 64-channel chunks per tile
    int n_row_units, n_col_tiles, n_units;
    float sqrt_dk;
};

__device__ __forceinline__ void fail(volatile int* abort_flag, uint32_t peer_abort, int code) {
    *abort_flag = 1;
    st_cluster_u32(peer_abort, 1u);
    atomicCAS(&g_sim_topk2_status, 0, code);
}

// NST: depth of the shared-memory ring (5; 4 where the merge buffer of a long list needs the room)
template <int NSEL, int NST>
__global__ void __launch_bounds__(NTHREADS, 1)
sim_topk_tc2_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ,
                    const Tc2Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* stages = smem;                                                   // [STAGES][A | B]
    float* keybuf = reinterpret_cast<float*>(smem + NST * STAGE_BYTES);       // [2 column halves][CW][128]
    float* mbuf = keybuf + 2 * CW * kSelGroup;                                // [2 * NSEL][128] merge hand-over
    float* statbuf = mbuf + 2 * NSEL * kSelGroup;                             // [8 warps][128] column statistics of the tile
    uint64_t* bars = reinterpret_cast<uint64_t*>(statbuf + 8 * 128);
    uint64_t* full = bars;                      // used in the leader only
    uint64_t* empty = bars + STAGES;
    uint64_t* tfull = bars + 2 * STAGES;
    uint64_t* tempty = tfull + 2;               // used in the leader only
    uint64_t* mfull = tempty + 2;               // per lane quarter: upper-half list written
    uint64_t* mempty = mfull + 4;               // per lane quarter: list consumed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mempty + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0 = leader
    const uint32_t peer = rank ^ 1u;
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 16);          // 8 selection warps of each CTA
        }
        for (int b = 0; b < 4; ++b) {
            mbar_init(&mfull[b], 1);
            mbar_init(&mempty[b], 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmQ);
    }
    __syncthreads();
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                         // both CTAs' barriers exist before any remote signal
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t full0 = smem_u32(full), empty0 = smem_u32(empty);
    const uint32_t tfull0 = smem_u32(tfull), tempty0 = smem_u32(tempty);
    const uint32_t st0 = smem_u32(stages);
    const uint32_t peer_abort = map_to_cta(smem_u32(const_cast<int*>(abort_flag)), peer);

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t lead_full0 = map_to_cta(full0, 0);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int unit = cluster_id; unit < p.n_units && ok; unit += n_clusters) {
                const int bh = unit / p.n_row_units, ru = unit - bh * p.n_row_units;
                const int b = bh / p.H, h = bh - b * p.H;
                const int row0 = ru * 2 * BM + (int)rank * BM;
                for (int ct = 0; ct < p.n_col_tiles && ok; ++ct) {
                    const int col0 = ct * BN + (int)rank * BNH;
                    for (int kc = 0; kc < p.KC; ++kc) {
                        if (!mbar_wait_a(empty0 + 8 * s, ph ^ 1u, abort_flag)) { fail(abort_flag, peer_abort, 21); ok = false; break; }
                        const uint32_t st = st0 + s * STAGE_BYTES;
                        if (rank == 0) mbar_expect_tx_a(full0 + 8 * s, 2 * STAGE_BYTES);
                        tma_load_4d_pair(st, &tmK, lead_full0 + 8 * s, kc * KCH, h, row0, b);
                        tma_load_4d_pair(st + A_BYTES, &tmQ, lead_full0 + 8 * s, kc * KCH, h, col0, b);
                        if (++s == NST) { s = 0; ph ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_idesc_bf16_f32(2 * BM, BN);
            const uint64_t dhi = kmajor_desc_hi(KCH * 2);
            const uint32_t peer_empty0 = map_to_cta(empty0, 1), peer_tfull0 = map_to_cta(tfull0, 1);
            uint32_t s = 0, ph = 0, tile = 0;
            bool ok = true;
            for (int unit = cluster_id; unit < p.n_units && ok; unit += n_clusters) {
                for (int ct = 0; ct < p.n_col_tiles && ok; ++ct, ++tile) {
                    const uint32_t par = tile & 1u, u = tile >> 1;
                    if (!mbar_wait_a(tempty0 + 8 * par, (u & 1u) ^ 1u, abort_flag)) { fail(abort_flag, peer_abort, 22); ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t d = tmem_base + par * BN;
                    for (int kc = 0; kc < p.KC; ++kc) {
                        if (!mbar_wait_a(full0 + 8 * s, ph, abort_flag)) { fail(abort_flag, peer_abort, 23); ok = false; break; }
                        tc_fence_after_sync();
                        const uint32_t sa = st0 + s * STAGE_BYTES;
                        const uint64_t ad = dhi | (uint64_t)((sa & 0x3FFFFu) >> 4);
                        const uint64_t bd = dhi | (uint64_t)(((sa + A_BYTES) & 0x3FFFFu) >> 4);
                        mma_bf16_ss_pair(d, ad, bd, idesc, kc != 0);
                        mma_bf16_ss_pair(d, ad + 2, bd + 2, idesc, 1);
                        mma_bf16_ss_pair(d, ad + 4, bd + 4, idesc, 1);
                        mma_bf16_ss_pair(d, ad + 6, bd + 6, idesc, 1);
                        mma_commit_pair(empty0 + 8 * s);
                        mma_commit_pair(peer_empty0 + 8 * s);
                        if (++s == NST) { s = 0; ph ^= 1u; }
                    }
                    if (ok) {
                        mma_commit_pair(tfull0 + 8 * par);
                        mma_commit_pair(peer_tfull0 + 8 * par);
                    }
                }
            }
        }
    } else {
        const int chalf = (warp - 2) >> 2;       // which 128 columns of each tile this warp selects from
        const int lq = warp & 3;                 // TMEM lane quarter this warp may read
        const int r = lq * 32 + lane;            // row within this CTA's 128
        float* ks = keybuf + chalf * CW * kSelGroup + r;
        float* sq = statbuf + (warp - 2) * 128;
        uint32_t it = 0;                         // units done by this CTA (phase of the merge barriers)
        const uint32_t lead_tempty0 = map_to_cta(tempty0, 0);
        uint32_t tile = 0;
        bool ok = true;
        for (int unit = cluster_id; unit < p.n_units && ok; unit += n_clusters, ++it) {
            const int bh = unit / p.n_row_units, ru = unit - bh * p.n_row_units;
            const int row = ru * 2 * BM + (int)rank * BM + r;
            const bool row_ok = row < p.T;
            const float* qs_row = p.qstat ? p.qstat + (long long)bh * p.S : nullptr;
            float kst = 1.0f;
            if (row_ok && p.metric != CONVNN_MATMUL) kst = p.kstat[(long long)bh * p.T + row];
            const float sentinel = p.sampled ? self_sentinel(p.metric, kst, p.sqrt_dk) : 0.f;
            TopList<NSEL> top;
            top.init();
            float qv[4], qn[4];
            int cv[4], cn[4];
            auto fetch = [&](int ct, float (&fq)[4], int (&fc)[4]) {
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    const int cl = min(ct * BN + chalf * BNH + c4 * 32 + lane, p.S - 1);
                    fq[c4] = p.metric != CONVNN_MATMUL ? qs_row[cl] : 0.f;
                    fc[c4] = p.sampled ? p.cand[cl] : -1;
                }
            };
            fetch(0, qv, cv);
            // a warp whose 32 rows all lie past the end of the sequence has nothing to select
            const bool warp_live = ru * 2 * BM + (int)rank * BM + lq * 32 < p.T;
            for (int ct = 0; ct < p.n_col_tiles && ok; ++ct, ++tile) {
                const uint32_t par = tile & 1u, u = tile >> 1;
                if (ct + 1 < p.n_col_tiles) fetch(ct + 1, qn, cn);
                ok = mbar_wait(&tfull[par], u & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { if (lane == 0) fail(abort_flag, peer_abort, 24); break; }
                tc_fence_after_sync();
                const uint32_t taddr = tmem_base + ((uint32_t)(lq * 32) << 16) + par * BN + chalf * BNH;
                const int cbase = ct * BN + chalf * BNH;
                // this tile's column statistics, readable by every lane as broadcast vectors
                __syncwarp();
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) sq[c4 * 32 + lane] = qv[c4];
                __syncwarp();
                if (warp_live) {
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4) {
                        if (cbase + c4 * 32 < p.S) {             // otherwise the rest of the tile is padding
                            uint32_t acc[32];
                            tmem_ld_x32(taddr + c4 * 32, acc);
                            tmem_ld_wait();
                            consume<NSEL, 32>(top, acc, cbase + c4 * 32, 0, sq + c4 * 32, cv[c4], p, row, row_ok, sentinel, ks);
                        }
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8 * par);
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) { qv[c4] = qn[c4]; cv[c4] = cn[c4]; }
            }
            if (!ok) break;                      // no hand-over after a failed wait
            // merge the two column halves of each row: the upper-half warp hands its list to the
            // lower-half warp of the same lane quarter through shared memory
            if (chalf == 1) {
                ok = mbar_wait(&mempty[lq], (it & 1u) ^ 1u, abort_flag);      // previous hand-over consumed
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { if (lane == 0) fail(abort_flag, peer_abort, 25); break; }
#pragma unroll
                for (int s = 0; s < NSEL; ++s) {
                    mbuf[(2 * s) * kSelGroup + r] = top.v[s];
                    mbuf[(2 * s + 1) * kSelGroup + r] = __int_as_float(top.i[s]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&mfull[lq]);
            } else {
                ok = mbar_wait(&mfull[lq], it & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { if (lane == 0) fail(abort_flag, peer_abort, 26); break; }
#pragma unroll
                for (int s = 0; s < NSEL; ++s)
                    top.insert_ordered(mbuf[(2 * s) * kSelGroup + r], __float_as_int(mbuf[(2 * s + 1) * kSelGroup + r]));
                __syncwarp();
                if (lane == 0) mbar_arrive(&mempty[lq]);
                if (row_ok) write_selection<NSEL>(top, p, ((long long)bh * p.T + row) * p.K, row, kst);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // a wait expired: give copies and MMAs still in flight time to finish before the
        // pair's shared memory and TMEM are released
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync_all();                          // the peer no longer signals or reads this CTA
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

}  // namespace

// The pair kernel pays off where the tensor pipe is the limiter: long key and candidate
// lists, full 64-channel chunks.
bool sim_topk_tc2_wanted(const convnn_desc* d, const Dims& dm) {
    static const int env = [] { const char* e = getenv("CONVNN_B200_SIM_PAIR"); return e ? atoi(e) : -1; }();
    if (env == 0) return false;
    if (d->dtype != CONVNN_BF16 || dm.Cp % 64 != 0) return false;
    // Lists longer than 16 double the cost of keeping two lists per row; measured break-even
    // is at many units per cluster and a few thousand candidates.
    if (dm.nsel > 16) return dm.T >= 8192 && dm.S >= 4096;
    return dm.T >= 1024 && dm.S >= 1024;
}

int launch_sim_topk_tc2(const convnn_desc* d, const Dims& dm, const void* q, const void* k, const float* qstat,
                        const float* kstat, const int32_t* cand, int32_t* idx, float* val, cudaStream_t st) {
    Tc2Params p{};
    p.qstat = qstat; p.kstat = kstat; p.cand = cand; p.idx = idx; p.val = val;
    p.T = dm.T; p.S = dm.S; p.H = dm.H; p.K = dm.K; p.nsel = dm.nsel; p.metric = d->metric; p.sampled = d->sampled;
    p.KC = dm.Cp / KCH;
    p.n_row_units = (dm.T + 2 * BM - 1) / (2 * BM);
    p.n_col_tiles = (dm.S + BN - 1) / BN;
    p.n_units = dm.B * dm.H * p.n_row_units;
    p.sqrt_dk = (float)sqrt((double)dm.dk);

    CUtensorMap tmK, tmQ;
    const uint64_t dimsK[4] = {(uint64_t)dm.Cp, (uint64_t)dm.H, (uint64_t)dm.T, (uint64_t)dm.B};
    const uint64_t dimsQ[4] = {(uint64_t)dm.Cp, (uint64_t)dm.H, (uint64_t)dm.S, (uint64_t)dm.B};
    const uint64_t strK[3] = {(uint64_t)dm.Cp * 2, (uint64_t)dm.H * dm.Cp * 2, (uint64_t)dm.T * dm.H * dm.Cp * 2};
    const uint64_t strQ[3] = {(uint64_t)dm.Cp * 2, (uint64_t)dm.H * dm.Cp * 2, (uint64_t)dm.S * dm.H * dm.Cp * 2};
    const uint32_t boxK[4] = {(uint32_t)KCH, 1, (uint32_t)BM, 1};
    const uint32_t boxQ[4] = {(uint32_t)KCH, 1, (uint32_t)BNH, 1};
    if (!encode_tensor_map_bf16(&tmK, k, 4, dimsK, strK, boxK, KCH * 2)) return CONVNN_E_CUDA;
    if (!encode_tensor_map_bf16(&tmQ, q, 4, dimsQ, strQ, boxQ, KCH * 2)) return CONVNN_E_CUDA;

    const size_t smem_fixed = 1024 + 2 * CW * kSelGroup * sizeof(float) + 8 * 128 * sizeof(float) +
                              (2 * STAGES + 12) * 8 + 16;

#define CONVNN_TC2_LAUNCH(N)                                                                                     \
    do {                                                                                                         \
        constexpr int NST = N > 24 ? STAGES - 1 : STAGES;                                                        \
        auto kern = sim_topk_tc2_kernel<N, NST>;                                                                 \
        const size_t smem = smem_fixed + (size_t)NST * STAGE_BYTES + 2 * N * kSelGroup * sizeof(float);          \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        cudaLaunchConfig_t cfg{};                                                                                \
        cudaLaunchAttribute attr[1];                                                                             \
        attr[0].id = cudaLaunchAttributeClusterDimension;                                                        \
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;                \
        cfg.blockDim = dim3(NTHREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;                             \
        cfg.attrs = attr; cfg.numAttrs = 1;                                                                      \
        cfg.gridDim = dim3(2);                                                                                   \
        /* co-resident clusters for this kernel and shared-memory size, asked once per process */       \
        static std::atomic<long long> occ_cache{-1};                                                        \
        int max_clusters = 0;                                                                               \
        const long long seen = occ_cache.load(std::memory_order_relaxed);                                   \
        if (seen >= 0 && (size_t)(seen >> 20) == smem) {                                                    \
            max_clusters = (int)(seen & 0xFFFFF);                                                           \
        } else {                                                                                            \
            e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);                                  \
            if (e != cudaSuccess || max_clusters < 1)                                                       \
                return set_error(CONVNN_E_CUDA, "cudaOccupancyMaxActiveClusters: %s", cudaGetErrorString(e)); \
            occ_cache.store(((long long)smem << 20) | max_clusters, std::memory_order_relaxed);             \
        }                                                                                                   \
        const int nc = p.n_units < max_clusters ? p.n_units : max_clusters;                                      \
        cfg.gridDim = dim3(2 * nc);                                                                              \
        e = cudaLaunchKernelEx(&cfg, kern, tmK, tmQ, p);                                                         \
        if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "sim_topk_tc2 launch: %s", cudaGetErrorString(e)); \
    } while (0)
    const int n = dm.nsel;
    if (n <= 4) CONVNN_TC2_LAUNCH(4);
    else if (n <= 8) CONVNN_TC2_LAUNCH(8);
    else if (n == 9) CONVNN_TC2_LAUNCH(9);
    else if (n <= 12) CONVNN_TC2_LAUNCH(12);
    else if (n <= 16) CONVNN_TC2_LAUNCH(16);
    else if (n <= 24) CONVNN_TC2_LAUNCH(24);
    else if (n == 25) CONVNN_TC2_LAUNCH(25);
    else CONVNN_TC2_LAUNCH(32);
#undef CONVNN_TC2_LAUNCH
    CONVNN_CHECK_LAUNCH("sim_topk_tc2");
    return CONVNN_OK;
}

int read_sim_topk2_status(int* out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_sim_topk2_status, sizeof(int));
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    *out = v;
    return CONVNN_OK;
}

}  // namespace convnn
