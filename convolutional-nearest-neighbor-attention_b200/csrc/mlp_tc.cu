// The encoder's MLP block as ONE kernel on the 5th-generation tensor cores (bfloat16):
//     out = x + ( GELU( LayerNorm(x) W1^T + b1 ) W2^T + b2 )          (reference vit.py:267-269)
// The hidden activations (rows x d_mlp, four times the size of x) never leave the SM: a CTA pair
// owns 256 rows (128 per CTA) and walks the hidden width in super-chunks of 128 columns,
//     MMA 1  acc1 = x W1'[super-chunk]^T (+ the pre-norm fold's extra K = 16 step)   M = 256, N = 128
//     GELU   h = bf16(GELU(rstd * acc1)) stored back to TMEM as two 64-column A operands (bfloat16 pairs)
//     MMA 2  acc2 += h[chunk] W2[:, chunk]^T, twice, A read from TMEM                M = 256, N = D
// with acc1 double-buffered (super-chunk n + 1 is multiplied while n is activated), all in TMEM
// (2 x 128 + D + 2 x 32 <= 512 columns): h does not pass through shared memory, whose bandwidth the
// MMAs' operand reads, the TMA writes and the epilogue already share.  The LayerNorm
// is folded as in gemm_tc.cu: W1' = W1 diag(gamma), the rows' moments (sum x, sum x^2) arrive
// from the kernel that wrote x, one warp turns them into the extra operand chunk [-mean, sigma].
// The skip connection needs no second read of x: the final epilogue adds the rounded result to
// the x tile where it lies in shared memory and a TMA store writes that tile out; it also emits
// the moments of the rows it stored (four planes, one per column quarter) for the next folded GEMM.
//
// Two CTAs of a cluster form one tcgen05 cta_group::2 unit so that each CTA fetches only half of
// every weight chunk: per 128 rows a CTA streams (d_mlp x D + D x d_mlp) / 2 weights from L2.
// Warps: 0 TMA producer of x and W1 (and the tile store), 1 issuer of MMA 1 (leader CTA), 2 extra-chunk
// preparation, 3-18 epilogue (column group x TMEM lane quarter), 19 issuer of MMA 2 (leader CTA), 20 TMA
// producer of W2 (a warp of its own: lanes of one warp that wait in different loops only take turns).
// "Operands landed" barriers live in the
// leader and are credited by both CTAs' loads; completions are committed to both CTAs.  Every
// wait is bounded; a warp whose wait expires raises the pair's abort flags and stops working, which
// makes every other wait of the pair give up: nothing can hang.
#include <atomic>

#include "common.cuh"
#include "sm100.cuh"
#include "f32x2.cuh"
#include "gelu.cuh"

namespace convnn {

__device__ int g_mlp_tc_status = 0;   // error latch of this translation unit

// Pipeline trace (a development aid, compiled in only with -DCONVNN_B200_MLP_TRACE): cluster 0 records
// nanosecond time stamps of its producer, MMA and epilogue events.
#ifdef CONVNN_B200_MLP_TRACE
__device__ unsigned long long g_mlp_trace[16 * 64];
__device__ __forceinline__ void mtrace(bool on, int ev, uint32_t g) {
    if (on && g < 64) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_mlp_trace[ev * 64 + g] = t;
    }
}
#else
__device__ __forceinline__ void mtrace(bool, int, uint32_t) {}
#endif

namespace {

using namespace sm100;

// GELU (tanh form, as in gelu.cuh) of a pair of accumulator values, result packed as bfloat16 x 2.
// With hx = 0.5 * rstd * acc (fp32):  GELU = hx + hx * tanh(u),  u = hx * (2 c0 + 8 c1 hx^2).  The
// argument u and the tanh are evaluated on the pair in half precision (three packed instructions
// and ONE special-function instruction for both values; the fp32 form costs four two-cycle packed
// instructions and two special-function instructions, and the activation of a 128 x 128 super-chunk
// is what bounds this kernel); the dominant term hx and the final multiply-add stay in fp32.  The
// half-precision tanh is accurate to ~2^-11, below the bfloat16 rounding (2^-9) of the result.
__device__ __forceinline__ uint32_t gelu_pair_bf16x2(float a, float b, f32x2 half_rstd) {
    const f32x2 hx = mul2(pack2(a, b), half_rstd);
    float ha, hb;
    unpack2(hx, ha, hb);
    uint32_t h, t;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(h) : "f"(hb), "f"(ha));
    asm("{\n\t.reg .b32 s, w;\n\t"
        "mul.rn.f16x2 s, %1, %1;\n\t"
        "fma.rn.f16x2 w, s, %2, %3;\n\t"
        "mul.rn.f16x2 w, w, %1;\n\t"
        "tanh.approx.f16x2 %0, w;\n\t}"
        : "=r"(t) : "r"(h), "r"(0x34913491u), "r"(0x3e623e62u));      // 8 c1 = 0.2854, 2 c0 = 1.5958
    float ta, tb;
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.f32.f16 %0, lo;\n\tcvt.f32.f16 %1, hi;\n\t}"
        : "=f"(ta), "=f"(tb) : "r"(t));
    float oa, ob;
    unpack2(fma2(hx, pack2(ta, tb), hx), oa, ob);
    __nv_bfloat162 hv = __floats2bfloat162_rn(oa, ob);
    return *reinterpret_cast<uint32_t*>(&hv);
}


constexpr int BM = 128;        // rows per CTA
constexpr int SC = 128;        // hidden columns per MMA 1 step ("super-chunk"): two h chunks
constexpr int CH = 64;         // hidden columns per h chunk (MMA 2 step)
constexpr int NSW2 = 5;        // ring depth of the W2 chunks
constexpr int NT = 21 * 32;    // TMA, MMA 1, extra-chunk, 16 epilogue warps, MMA 2, W2 stream

struct MlpParams {
    int M, D, DM;
    int KC;             // D / 64: 64-column sub-chunks of a row of x
    int n_sc;           // DM / 128 super-chunks
    int n_ptiles;       // 256-row tiles
    int planes;         // planes of the incoming moments
    long long mom_ld_in, mom_ld_out;
    float eps, inv_d;
    const float2* moments;
    const __nv_bfloat16* resid;   // OP: the rows x of the skip connection x + o W_o^T, stride ldr
    long long ldr;
    const __nv_bfloat16* bias2;
    float2* moments_out;   // [4][mom_ld_out] or nullptr
};

struct Smem {           // byte offsets from the 1 KB-aligned base
    uint32_t x, w1, w2, xa, rstd, bias, bars, total;
    uint32_t w1_slot, w2_slot;
};

__host__ __device__ inline Smem smem_plan(int D) {
    Smem s;
    const uint32_t KC = D / 64;
    uint32_t o = 0;
    s.x = o; o += 2u * KC * 16384u;                 // two x tiles of KC sub-chunks [128 x 64]
    s.w1_slot = KC * 8192u + 2048u;                 // [64 x 64] per sub-chunk + the fold's extra rows [64 x 16]
    s.w1 = o; o += 2u * s.w1_slot;
    s.w2_slot = ((uint32_t)(D / 2) * 128u + 1023u) & ~1023u;   // [D/2 x 64]
    s.w2 = o; o += NSW2 * s.w2_slot;
    s.xa = o; o += 2u * 4096u;
    s.rstd = o; o += 2u * BM * 4u;
    s.bias = o; o += (uint32_t)D * 2u;              // b2
    s.bars = o; o += 40u * 8u + 32u;
    s.total = o;
    return s;
}

enum Bar : int {            // indices into the barrier array
    XFULL = 0,              // [2] leader: x tile of both CTAs landed
    XFREE = 2,              // [2] local: the tile's TMA store has read the buffer
    W1FULL = 4,             // [2] leader
    A1FULL = 6,             // [2] local: acc1 super-chunk complete (= its W1 slot is free again)
    A1EMPTY = 8,            // [2] leader: 16 warps x 2 CTAs have read it
    HFULL = 16,             // [2] leader: 8 warps x 2 CTAs have written the h chunk
    HEMPTY = 18,            // [2] local: MMA 2 has read it
    A2FULL = 20,            // [1] local: acc2 of a tile complete
    A2EMPTY = 21,           // [1] leader: 16 warps x 2 CTAs have read it
    XAFULL = 22,            // [2] leader: extra chunk of both CTAs written
    OUTREADY = 24,          // [2] local: the 16 epilogue warps have finished the tile's rows in the x buffer
    STATREADY = 26,         // [2] local (OP): the 16 epilogue warps have written x1 and its partial moments
    W2FULL = 28,            // [NSW2] leader
    W2EMPTY = 33,           // [NSW2] local (committed by MMA 2)
    NBARS = 38
};

// OP: the attention layer's output projection and skip connection run first, per tile:
//     x1 = x + bf16(o W_o^T)           (reference layers.py:320 with vit.py:264)
// o arrives where x would (TMA into the x buffer), W_o passes through the W1 ring as two items of D/2
// output columns, the accumulators are the two acc1 buffers, and the epilogue warps write x1 over o in
// the x buffer (the operand of MMA 1 and the skip connection of the final epilogue) together with the
// partial moments of its rows, from which the extra-chunk warp derives mean and rstd: the block then
// needs no moments from outside.
template <bool OP>
__global__ void __launch_bounds__(NT, 1)
mlp_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmO,
              const __grid_constant__ CUtensorMap tmW1, const __grid_constant__ CUtensorMap tmWX,
              const __grid_constant__ CUtensorMap tmW2, const __grid_constant__ CUtensorMap tmWO, const MlpParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const Smem L = smem_plan(p.D);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bars);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 40);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* rstd_s = reinterpret_cast<float*>(smem + L.rstd);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                 // 0 = leader
    const int cluster_id = (int)(blockIdx.x >> 1), n_clusters = (int)(gridDim.x >> 1);
    const uint32_t base = smem_u32(smem);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t lead_bar0 = map_to_cta(bar0, 0);
    auto lbar = [&](int i) { return bar0 + 8u * (uint32_t)i; };           // local barrier i
    auto leadbar = [&](int i) { return lead_bar0 + 8u * (uint32_t)i; };   // the leader's barrier i

    if (threadIdx.x == 0) {
        auto init = [&](int i, int n, int count) { for (int k = 0; k < n; ++k) mbar_init(&bars[i + k], count); };
        init(XFULL, 2, 1); init(XFREE, 2, 1);
        init(W1FULL, 2, 1); init(A1FULL, 2, 1); init(A1EMPTY, 2, 32);
        init(W2FULL, NSW2, 1); init(W2EMPTY, NSW2, 1);
        init(HFULL, 2, 16); init(HEMPTY, 2, 1);
        init(A2FULL, 1, 1); init(A2EMPTY, 1, 32);
        init(XAFULL, 2, 2);
        init(OUTREADY, 2, 16);
        init(STATREADY, 2, 16);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmX); prefetch_tensormap(&tmO); prefetch_tensormap(&tmW1);
        prefetch_tensormap(&tmWX); prefetch_tensormap(&tmW2);
        if (OP) prefetch_tensormap(&tmWO);
    }
    __syncthreads();
    if (warp == 1) { tmem_alloc_pair(tmem_slot, 512); tmem_relinquish_pair(); }
    for (int i = threadIdx.x; i < p.D / 2; i += blockDim.x)         // b2 (or zeros) for the final epilogue
        reinterpret_cast<uint32_t*>(smem + L.bias)[i] = p.bias2 ? reinterpret_cast<const uint32_t*>(p.bias2)[i] : 0u;
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                          // both CTAs' barriers exist before any remote signal
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t peer_abort = map_to_cta(smem_u32(const_cast<int*>(abort_flag)), rank ^ 1u);
    auto give_up = [&](int code) {
        st_cluster_u32(peer_abort, 1u);
        *abort_flag = 1;
        atomicCAS(&g_mlp_tc_status, 0, code);
    };

    const int my_tiles = cluster_id < p.n_ptiles ? (p.n_ptiles - cluster_id + n_clusters - 1) / n_clusters : 0;
    const int nsc = p.n_sc;
    const uint32_t x_tile_bytes = (uint32_t)p.KC * 16384u;
    auto row0_of = [&](int it) { return (cluster_id + it * n_clusters) * 2 * BM + (int)rank * BM; };
    const uint32_t acc2_col = 2 * SC;            // TMEM: acc1[2] at columns 0 / 128, acc2 behind them
    const uint32_t h_col = 512 - 2 * (CH / 2);   // the two h chunks (bfloat16 pairs: 32 columns each) in the last 64
    // Order of the accumulator items of a tile (the same in the producer, the MMA 1 thread and the epilogue
    // warps): its super-chunks 0 .. nsc - 1 and, with OP, the two output-projection items of the NEXT tile in
    // front of super-chunk kp, so that x1, its moments and the extra operand chunk of the next tile are
    // ready long before that tile's first MMA 1; tile 0's own two items come first of all.
    const int kp = nsc >= 4 ? nsc - 2 : nsc - 1;

    if (warp == 0) {
        // ---- TMA producers (each CTA fetches its own rows of x and its half of every weight chunk).
        // One thread can start a TMA operation only every ~0.3 us, whatever its size, while operations
        // started by different lanes overlap: lanes 0 .. KC issue the sub-chunks of a W1 super-chunk (and
        // the x tiles) with one instruction of the warp; lane KC + 2 stores finished tiles and refills their
        // buffers.  The W2 stream, whose slots are released by MMA 2, has warp 20.
        const uint32_t w1_mask = (2u << p.KC) - 1u;              // lanes 0 .. KC
        if (lane <= p.KC) {
            bool ok = true;
            auto load_x = [&](int it) {
                const int xb = it & 1;
                ok = mbar_wait(&bars[XFREE + xb], ((uint32_t)(it >> 1) & 1u) ^ 1u, abort_flag);
                ok = __all_sync(w1_mask, ok);
                if (!ok) { if (lane == 0) give_up(51); return; }
                if (rank == 0 && lane == 0) mbar_expect_tx_a(lbar(XFULL + xb), 2u * x_tile_bytes);
                __syncwarp(w1_mask);
                if (lane < p.KC)
                    tma_load_2d_pair(base + L.x + xb * x_tile_bytes + lane * 16384u, &tmX, leadbar(XFULL + xb), lane * 64, row0_of(it));
            };
            if (my_tiles > 0) load_x(0);
            uint32_t n = 0;                                        // running accumulator item number
            // W_o as two items of D/2 output columns (D/4 rows per CTA), sub-chunks 8 KB apart
            auto load_wo = [&]() {
                for (int item = 0; item < 2 && ok; ++item, ++n) {
                    const uint32_t b = n & 1u;
                    ok = mbar_wait(&bars[A1FULL + b], ((n >> 1) & 1u) ^ 1u, abort_flag);
                    ok = __all_sync(w1_mask, ok);
                    if (!ok) { if (lane == 0) give_up(52); break; }
                    mtrace(cluster_id == 0 && rank == 0 && lane == 0, 1, n);
                    if (rank == 0 && lane == 0) mbar_expect_tx_a(lbar(W1FULL + b), 2u * (uint32_t)p.KC * (uint32_t)(p.D / 4) * 128u);
                    __syncwarp(w1_mask);
                    if (lane < p.KC)
                        tma_load_2d_pair(base + L.w1 + b * L.w1_slot + lane * 8192u, &tmWO, leadbar(W1FULL + b), lane * 64,
                                         item * (p.D / 2) + (int)rank * (p.D / 4));
                }
            };
            if (OP && my_tiles > 0) load_wo();
            for (int it = 0; it < my_tiles && ok; ++it) {
                for (int sc = 0; sc < nsc && ok; ++sc, ++n) {
                    if (OP && sc == kp && it + 1 < my_tiles) { load_wo(); if (!ok) break; }
                    const uint32_t b = n & 1u;
                    // the slot's previous item (n - 2) has been multiplied
                    ok = mbar_wait(&bars[A1FULL + b], ((n >> 1) & 1u) ^ 1u, abort_flag);
                    ok = __all_sync(w1_mask, ok);
                    if (!ok) { if (lane == 0) give_up(52); break; }
                    mtrace(cluster_id == 0 && rank == 0 && lane == 0, 1, n);
                    if (rank == 0 && lane == 0) mbar_expect_tx_a(lbar(W1FULL + b), 2u * L.w1_slot);
                    __syncwarp(w1_mask);
                    const uint32_t w1s = base + L.w1 + b * L.w1_slot;
                    if (lane < p.KC)
                        tma_load_2d_pair(w1s + lane * 8192u, &tmW1, leadbar(W1FULL + b), lane * 64, sc * SC + (int)rank * 64);
                    else
                        tma_load_2d_pair(w1s + p.KC * 8192u, &tmWX, leadbar(W1FULL + b), 0, sc * SC + (int)rank * 64);
                }
            }
        } else if (lane == p.KC + 2) {
            // the finished rows of a tile leave through a TMA store of the x buffer they were written into;
            // the buffer is refilled at once with the tile after the next (tile 1 is requested up front)
            auto load_next = [&](int it) {
                const uint32_t xb = (uint32_t)it & 1u;
                if (rank == 0) mbar_expect_tx_a(lbar(XFULL + xb), 2u * x_tile_bytes);
                for (int kc = 0; kc < p.KC; ++kc)
                    tma_load_2d_pair(base + L.x + xb * x_tile_bytes + kc * 16384u, &tmX, leadbar(XFULL + xb), kc * 64, row0_of(it));
            };
            if (my_tiles > 1) load_next(1);
            for (int it = 0; it < my_tiles; ++it) {
                const uint32_t xb = (uint32_t)it & 1u;
                if (!mbar_wait_a(lbar(OUTREADY + xb), (uint32_t)(it >> 1) & 1u, abort_flag)) { give_up(66); break; }
                for (int kc = 0; kc < p.KC; ++kc)
                    tma_store_2d(&tmO, smem + L.x + xb * x_tile_bytes + kc * 16384u, kc * 64, row0_of(it));
                tma_store_commit();
                tma_store_wait_read<0>();
                mbar_arrive(&bars[XFREE + xb]);                   // the buffer's contents are no longer needed
                if (it + 2 < my_tiles) load_next(it + 2);
            }
            tma_store_wait<0>();
        }
    } else if (warp == 1) {
        // ---- issuer of MMA 1 (leader only): acc1[n & 1] = x W1'[super-chunk]^T, N = 128.  A tcgen05.mma
        // costs its issuing thread ~35-50 ns whatever its size, so the steps are as wide as the pipeline
        // allows and MMA 2 has an issuing thread of its own; the barriers order the two streams.
        if (lane == 0 && rank == 0) {
            const uint32_t idesc1 = make_idesc_bf16_f32(2 * BM, SC);
            const uint64_t dhi = kmajor_desc_hi(128), dhi32 = kmajor_desc_hi(32);
            auto desc = [&](uint64_t hi, uint32_t addr) { return hi | (uint64_t)((addr & 0x3FFFFu) >> 4); };
            const uint32_t idesc0 = make_idesc_bf16_f32(2 * BM, p.D / 2);
            uint32_t n = 0;                                        // running accumulator item number
            bool ok = true;
            // the two output-projection items of tile `it`: acc1[n & 1] = o W_o[item]^T, N = D / 2
            auto mma_wo = [&](int it) {
                const uint32_t xb = (uint32_t)it & 1u;
                if (!mbar_wait_a(lbar(XFULL + xb), (uint32_t)(it >> 1) & 1u, abort_flag)) { give_up(54); ok = false; return; }
                for (int item = 0; item < 2; ++item, ++n) {
                    const uint32_t b = n & 1u;
                    if (!mbar_wait_a(lbar(A1EMPTY + b), ((n >> 1) & 1u) ^ 1u, abort_flag)) { give_up(56); ok = false; return; }
                    mtrace(cluster_id == 0, 2, n);
                    if (!mbar_wait_a(lbar(W1FULL + b), (n >> 1) & 1u, abort_flag)) { give_up(57); ok = false; return; }
                    mtrace(cluster_id == 0, 3, n);
                    tc_fence_after_sync();
                    const uint32_t xs0 = base + L.x + xb * x_tile_bytes, w0s = base + L.w1 + b * L.w1_slot;
                    for (int kc = 0; kc < p.KC; ++kc)
                        mma_chunk_pair(tmem_base + b * SC, desc(dhi, xs0 + kc * 16384u), desc(dhi, w0s + kc * 8192u), idesc0, 4, kc != 0);
                    mma_commit_pair_both(lbar(A1FULL + b));
                    mtrace(cluster_id == 0, 4, n);
                }
            };
            if (OP && my_tiles > 0) mma_wo(0);
            for (int it = 0; it < my_tiles && ok; ++it) {
                const uint32_t xb = (uint32_t)it & 1u;
                for (int sc = 0; sc < nsc && ok; ++sc, ++n) {
                    if (OP && sc == kp && it + 1 < my_tiles) { mma_wo(it + 1); if (!ok) break; }
                    const uint32_t b = n & 1u;
                    if (sc == 0) {
                        if (!OP && !mbar_wait_a(lbar(XFULL + xb), (uint32_t)(it >> 1) & 1u, abort_flag)) { give_up(54); ok = false; break; }
                        if (!mbar_wait_a(lbar(XAFULL + xb), (uint32_t)(it >> 1) & 1u, abort_flag)) { give_up(55); ok = false; break; }
                    }
                    if (!mbar_wait_a(lbar(A1EMPTY + b), ((n >> 1) & 1u) ^ 1u, abort_flag)) { give_up(56); ok = false; break; }
                    mtrace(cluster_id == 0, 2, n);
                    if (!mbar_wait_a(lbar(W1FULL + b), (n >> 1) & 1u, abort_flag)) { give_up(57); ok = false; break; }
                    mtrace(cluster_id == 0, 3, n);
                    tc_fence_after_sync();
                    const uint32_t d1 = tmem_base + b * SC;
                    const uint32_t xs = base + L.x + xb * x_tile_bytes, w1s = base + L.w1 + b * L.w1_slot;
                    for (int kc = 0; kc < p.KC; ++kc)
                        mma_chunk_pair(d1, desc(dhi, xs + kc * 16384u), desc(dhi, w1s + kc * 8192u), idesc1, 4, kc != 0);
                    // the pre-norm fold's extra step: [-mean, sigma] x [c, b']
                    mma_bf16_ss_pair(d1, desc(dhi32, base + L.xa + xb * 4096u), desc(dhi32, w1s + p.KC * 8192u), idesc1, 1);
                    mma_commit_pair_both(lbar(A1FULL + b));
                    mtrace(cluster_id == 0, 4, n);
                }
            }
        }
    } else if (warp == 19) {
        // ---- issuer of MMA 2 (leader only): acc2 (+)= h[chunk] W2[:, chunk]^T, N = D
        if (lane == 0 && rank == 0) {
            const uint32_t idesc2 = make_idesc_bf16_f32(2 * BM, p.D);
            const uint64_t dhi = kmajor_desc_hi(128);
            auto desc = [&](uint64_t hi, uint32_t addr) { return hi | (uint64_t)((addr & 0x3FFFFu) >> 4); };
            const int nch = nsc * 2;
            const uint32_t total = (uint32_t)my_tiles * (uint32_t)nch;
            const uint32_t d2 = tmem_base + acc2_col;
            uint32_t s = 0, ph = 0;
            int c = 0, it = 0;
            for (uint32_t g = 0; g < total; ++g) {
                const uint32_t hb = g & 1u;                       // h chunk = half of its super-chunk
                if (c == 0 && !mbar_wait_a(lbar(A2EMPTY), ((uint32_t)it & 1u) ^ 1u, abort_flag)) { give_up(58); break; }
                if (!mbar_wait_a(lbar(HFULL + hb), (g >> 1) & 1u, abort_flag)) { give_up(59); break; }
                mtrace(cluster_id == 0, 5, g);
                if (!mbar_wait_a(lbar(W2FULL + s), ph, abort_flag)) { give_up(60); break; }
                mtrace(cluster_id == 0, 6, g);
                tc_fence_after_sync();
                // h straight from tensor memory, where the epilogue warps put it: 8 columns per K = 16 step
                const uint64_t w2d = desc(dhi, base + L.w2 + s * L.w2_slot);
                const uint32_t ha = tmem_base + h_col + hb * 32u;
                mma_bf16_ts_pair(d2, ha, w2d, idesc2, c != 0);
                mma_bf16_ts_pair(d2, ha + 8, w2d + 2, idesc2, 1);
                mma_bf16_ts_pair(d2, ha + 16, w2d + 4, idesc2, 1);
                mma_bf16_ts_pair(d2, ha + 24, w2d + 6, idesc2, 1);
                mma_commit_pair_both(lbar(W2EMPTY + s));
                mma_commit_pair_both(lbar(HEMPTY + hb));
                if (c == nch - 1) mma_commit_pair_both(lbar(A2FULL));
                mtrace(cluster_id == 0, 7, g);
                if (++s == NSW2) { s = 0; ph ^= 1u; }
                if (++c == nch) { c = 0; ++it; }
            }
        }
    } else if (warp == 20) {
        // ---- the W2 stream, a warp of its own: lanes of one warp that wait in different loops take turns, and
        // a W2 lane next to the W1 lanes only advanced when those came out of their (long) waits
        if (lane == 0) {
            const uint32_t total = (uint32_t)my_tiles * (uint32_t)nsc * 2u;   // h chunks
            uint32_t s = 0, ph = 0;
            int c = 0;
            const int nch = nsc * 2;
            for (uint32_t g = 0; g < total; ++g) {
                if (!mbar_wait_a(lbar(W2EMPTY + s), ph ^ 1u, abort_flag)) { give_up(53); break; }
                mtrace(cluster_id == 0 && rank == 0, 0, g);
                if (rank == 0) mbar_expect_tx_a(lbar(W2FULL + s), 2u * (uint32_t)(p.D / 2) * 128u);
                tma_load_2d_pair(base + L.w2 + s * L.w2_slot, &tmW2, leadbar(W2FULL + s), c * CH, (int)rank * (p.D / 2));
                if (++s == NSW2) { s = 0; ph ^= 1u; }
                if (++c == nch) c = 0;
            }
        }
    } else if (warp == 2) {
        // ---- extra operand chunk of every tile (as in gemm_tc.cu): lane l prepares rows l, l + 32, ...
        // The moments of tile it are read with plain loads while tile it - 1 is still being worked on.
        bool ok = true;
        for (int it = 0; it < my_tiles && ok; ++it) {
            const uint32_t xb = (uint32_t)it & 1u;
            uint32_t wm[4], wsg[4];
            float rs[4];
            if (OP) {
                // x1 and the partial moments of its rows (one partial per 32-column group of an item pair,
                // kept in this buffer's extra-chunk space) are ready
                ok = mbar_wait(&bars[STATREADY + xb], (uint32_t)(it >> 1) & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { if (lane == 0) give_up(61); break; }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int row = row0_of(it) + j * 32 + lane;
                float s1 = 0.f, s2 = 0.f;
                if (OP) {
                    const float2* part = reinterpret_cast<const float2*>(smem + L.xa + xb * 4096u);
                    for (int gq = 0; gq < p.D / 64; ++gq) {
                        const float2 m = part[gq * BM + j * 32 + lane];
                        s1 += m.x; s2 += m.y;
                    }
                } else if (row < p.M)
                    for (int pl0 = 0; pl0 < p.planes; pl0 += 4) {      // four independent loads in flight per row
                        float2 m[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            m[k] = pl0 + k < p.planes ? __ldg(p.moments + (long long)(pl0 + k) * p.mom_ld_in + row)
                                                      : make_float2(0.f, 0.f);
#pragma unroll
                        for (int k = 0; k < 4; ++k) { s1 += m[k].x; s2 += m[k].y; }
                    }
                const float mean = s1 * p.inv_d;
                const float var = fmaxf(fmaf(-mean, mean, s2 * p.inv_d), 0.f) + p.eps;
                const float rstd = rsqrtf(var), sigma = var * rstd;
                rs[j] = rstd;
                const __nv_bfloat16 mh = __float2bfloat16_rn(-mean), sh = __float2bfloat16_rn(sigma);
                const __nv_bfloat16 ml = __float2bfloat16_rn(-mean - __bfloat162float(mh));
                const __nv_bfloat16 sl = __float2bfloat16_rn(sigma - __bfloat162float(sh));
                wm[j] = (uint32_t)__bfloat16_as_ushort(mh) | ((uint32_t)__bfloat16_as_ushort(ml) << 16);
                wsg[j] = (uint32_t)__bfloat16_as_ushort(sh) | ((uint32_t)__bfloat16_as_ushort(sl) << 16);
            }
            if (OP) {
                __syncwarp();                                     // every lane has read its partials: the space is rewritten below
            } else {
                // the buffer's previous tile (it - 2) is completely done: its MMAs have read the extra chunk
                // and its epilogue warps took rstd into registers at their first super-chunk
                ok = mbar_wait(&bars[XFREE + xb], ((uint32_t)(it >> 1) & 1u) ^ 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { if (lane == 0) give_up(62); break; }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = j * 32 + lane;
                const uint4 v = make_uint4(wm[j], wm[j], wsg[j], wsg[j]);
                uint4* dst = reinterpret_cast<uint4*>(smem + L.xa + xb * 4096u + r * 32);
                dst[0] = v;
                dst[1] = v;
                rstd_s[xb * BM + r] = rs[j];
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leadbar(XAFULL + xb));
        }
    } else {
        // ---- epilogue warps: 32 columns of every super-chunk through GELU, then a quarter of the tile's
        // output columns.  The GELU output is the A operand of MMA 2: the packed bfloat16 pairs go straight
        // back to tensor memory (16 columns of this warp's rows) and MMA 2 reads them there, so h never
        // passes through shared memory.  (Two groups of eight warps that alternated over the super-chunks
        // were measured too: the same time.)
        const int ew = warp - 3;
        const int cg = ew >> 2, lq = warp & 3;                    // column group, TMEM lane quarter
        const int hb = cg >> 1;                                   // h chunk this warp writes into
        const int r = lq * 32 + lane;                             // row of this thread inside the CTA's tile
        const uint32_t lane_addr = (uint32_t)(lq * 32) << 16;
        const int qcols = p.D / 4;                                // output columns of this warp: 16, 32 or 48
        bool alive = true;
        auto die = [&](int code) { if (lane == 0) give_up(code); alive = false; };
        uint32_t n = 0, ns = 0;                                   // running accumulator item / super-chunk number
        float rstd = 1.0f;
        // one super-chunk: 32 columns of acc1 -> GELU -> this warp's 64 bytes of every row of an h chunk
        auto gelu_step = [&](int it, int sc) {
            const uint32_t b = n & 1u;
            bool ok = mbar_wait(&bars[A1FULL + b], (n >> 1) & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { die(63); return; }
            mtrace(cluster_id == 0 && rank == 0 && ew == 0 && lane == 0, 8, n);
            tc_fence_after_sync();
            if (sc == 0) rstd = rstd_s[((uint32_t)it & 1u) * BM + r];
            uint32_t acc[32];
            tmem_ld_x32(tmem_base + lane_addr + b * SC + cg * 32, acc);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leadbar(A1EMPTY + b));              // acc1 buffer may be overwritten
            uint32_t pk[16];
            const f32x2 r2 = pack2(0.5f * rstd, 0.5f * rstd);
#pragma unroll
            for (int e = 0; e < 16; ++e)
                pk[e] = gelu_pair_bf16x2(__uint_as_float(acc[2 * e]), __uint_as_float(acc[2 * e + 1]), r2);
            mtrace(cluster_id == 0 && rank == 0 && ew == 0 && lane == 0, 9, n);
            // MMA 2 of the previous super-chunk has read this h chunk
            ok = mbar_wait(&bars[HEMPTY + hb], (ns & 1u) ^ 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { die(64); return; }
            mtrace(cluster_id == 0 && rank == 0 && ew == 0 && lane == 0, 10, n);
            // the packed pairs are MMA 2's A operand as they are: 16 tensor-memory columns of this warp's rows
            tc_fence_after_sync();
            tmem_st_x16(tmem_base + lane_addr + h_col + (uint32_t)hb * 32u + (uint32_t)(cg & 1) * 16u, pk);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            mtrace(cluster_id == 0 && rank == 0 && ew == 0 && lane == 0, 11, n);
            if (lane == 0) mbar_arrive_cluster(leadbar(HFULL + hb));
            ++n;
            ++ns;
        };
        // OP: x1 = x + bf16(o W_o^T) for this warp's 32 columns of both items, written over o in the x buffer
        auto outproj_prefetch = [&](int it) {
            const int grow = row0_of(it) + r;
            if (cg < p.D / 64 && grow < p.M) {
#pragma unroll
                for (int item = 0; item < 2; ++item)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(p.resid + (long long)grow * p.ldr + item * (p.D / 2) + cg * 32));
            }
        };
        auto outproj_step = [&](int it) {
            const uint32_t xb2 = (uint32_t)it & 1u;
            const uint32_t b0 = n & 1u, b1 = b0 ^ 1u;
            const int ngrp = p.D / 64;                            // 32-column groups per item
            const int grow = row0_of(it) + r;
            // both items first: the MMAs of the second still read all of o
            bool ok = mbar_wait(&bars[A1FULL + b0], (n >> 1) & 1u, abort_flag);
            if (ok) ok = mbar_wait(&bars[A1FULL + b1], ((n + 1) >> 1) & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { die(67); return; }
            tc_fence_after_sync();
            const uint32_t xrow = base + L.x + xb2 * x_tile_bytes + (uint32_t)r * 128u;
            float m1 = 0.f, m2 = 0.f;
#pragma unroll 1
            for (int item = 0; item < 2; ++item) {
                const uint32_t bi = item == 0 ? b0 : b1;
                // the skip connection's values for these 32 columns (brought into L2 a super-chunk earlier)
                uint4 rx[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    rx[j] = make_uint4(0, 0, 0, 0);
                    if (cg < ngrp && grow < p.M)
                        rx[j] = __ldg(reinterpret_cast<const uint4*>(p.resid + (long long)grow * p.ldr + item * (p.D / 2) + cg * 32 + j * 8));
                }
                uint32_t acc[32];
                if (cg < ngrp) {
                    tmem_ld_x32(tmem_base + lane_addr + bi * SC + cg * 32, acc);
                    tmem_ld_wait();
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(leadbar(A1EMPTY + bi));
                if (cg < ngrp) {
                    const int col0 = item * (p.D / 2) + cg * 32;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t xw[4] = {rx[j].x, rx[j].y, rx[j].z, rx[j].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 hv = __floats2bfloat162_rn(__uint_as_float(acc[j * 8 + 2 * e]),
                                                                      __uint_as_float(acc[j * 8 + 2 * e + 1]));
                            hv = __hadd2(hv, *reinterpret_cast<__nv_bfloat162*>(&xw[e]));
                            xw[e] = *reinterpret_cast<uint32_t*>(&hv);
                            const float lo = __uint_as_float(xw[e] << 16), hi = __uint_as_float(xw[e] & 0xffff0000u);
                            m1 += lo + hi;
                            m2 = fmaf(hi, hi, fmaf(lo, lo, m2));
                        }
                        const int col = col0 + j * 8;
                        const uint32_t addr = xrow + (uint32_t)(col >> 6) * 16384u +
                                              ((((uint32_t)(col & 63) >> 3) ^ ((uint32_t)r & 7u)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(xw[0]), "r"(xw[1]), "r"(xw[2]),
                                     "r"(xw[3])
                                     : "memory");
                    }
                }
            }
            if (cg < ngrp) reinterpret_cast<float2*>(smem + L.xa + xb2 * 4096u)[cg * BM + r] = make_float2(m1, m2);
            fence_proxy_async();                                  // x1 in the x buffer -> visible to MMA 1
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[STATREADY + xb2]);
            n += 2;
        };
        // Per tile `it`: its super-chunks 1 .. nsc - 1, then super-chunk 0 of tile it + 1 (slot sc == nsc: it is
        // activated before the final epilogue of tile it, whose last MMA 2 drains meanwhile), with the
        // output-projection step of tile it + 1 in front of slot kp.  Round it = -1 (OP only) holds what
        // precedes tile 0: its output-projection step and its super-chunk 0.
        // final epilogue of tile `it`: out = x + round(acc2 + b2), in place in the x tile
        auto final_epilogue = [&](int it) {
            const uint32_t xb = (uint32_t)it & 1u;
            if (alive) {
                bool ok = mbar_wait(&bars[A2FULL], (uint32_t)it & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) die(65);
            }
            mtrace(cluster_id == 0 && rank == 0 && ew == 0 && lane == 0, 12, it);
            if (alive) {
                tc_fence_after_sync();
                const uint32_t t2 = tmem_base + lane_addr + acc2_col + cg * qcols;
                float m1 = 0.f, m2 = 0.f;
                const uint32_t xrow = base + L.x + xb * x_tile_bytes + (uint32_t)r * 128u;
                // 16 accumulator columns at a time (few live registers: this code shares its thread with the
                // activation step)
#pragma unroll 1
                for (int k = 0; k * 16 < qcols; ++k) {
                    uint32_t a2[16];
                    tmem_ld_x16(t2 + k * 16, a2);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int col = cg * qcols + k * 16 + i * 8;
                        const uint32_t addr = xrow + (uint32_t)(col >> 6) * 16384u +
                                              ((((uint32_t)(col & 63) >> 3) ^ ((uint32_t)r & 7u)) << 4);
                        uint4 xv, bv;
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(xv.x), "=r"(xv.y), "=r"(xv.z), "=r"(xv.w)
                                     : "r"(addr) : "memory");
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(bv.x), "=r"(bv.y), "=r"(bv.z), "=r"(bv.w)
                                     : "r"(base + L.bias + (uint32_t)col * 2u) : "memory");
                        uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
                        const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            // bf16(GEMM + bias) + bf16(x) rounded to bf16: what `x + mlp(...)` on bfloat16 tensors computes
                            __nv_bfloat162 hv = __floats2bfloat162_rn(
                                __uint_as_float(a2[i * 8 + 2 * e]) + __uint_as_float(bw[e] << 16),
                                __uint_as_float(a2[i * 8 + 2 * e + 1]) + __uint_as_float(bw[e] & 0xffff0000u));
                            hv = __hadd2(hv, *reinterpret_cast<__nv_bfloat162*>(&xw[e]));
                            xw[e] = *reinterpret_cast<uint32_t*>(&hv);
                            const float lo = __uint_as_float(xw[e] << 16), hi = __uint_as_float(xw[e] & 0xffff0000u);
                            m1 += lo + hi;
                            m2 = fmaf(hi, hi, fmaf(lo, lo, m2));
                        }
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(xw[0]), "r"(xw[1]), "r"(xw[2]),
                                     "r"(xw[3])
                                     : "memory");
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(leadbar(A2EMPTY));              // acc2 may be overwritten
                // this warp's quarter of the row moments: plane cg
                const int grow = row0_of(it) + r;
                if (p.moments_out && grow < p.M) p.moments_out[(long long)cg * p.mom_ld_out + grow] = make_float2(m1, m2);
                fence_proxy_async();                              // the tile's TMA store reads the x tile's new contents
            }
            mtrace(cluster_id == 0 && rank == 0 && ew == 0 && lane == 0, 14, it);
            __syncwarp();
            if (lane == 0 && alive) mbar_arrive(&bars[OUTREADY + xb]);   // 16 of these let the TMA store go
        };
        if constexpr (OP) {
            for (int it = -1; it < my_tiles; ++it) {
                for (int sc = it < 0 ? kp : 1; sc <= nsc && alive; ++sc) {
                    if (sc == kp - 1 && it + 1 < my_tiles) outproj_prefetch(it + 1);
                    if (sc == kp && it + 1 < my_tiles) outproj_step(it + 1);
                    const int git = sc < nsc ? it : it + 1, gsc = sc < nsc ? sc : 0;
                    if (alive && git >= 0 && git < my_tiles) gelu_step(git, gsc);
                }
                if (it >= 0) final_epilogue(it);
            }
        } else {
            for (int it = 0; it < my_tiles; ++it) {
                for (int sc = it == 0 ? 0 : 1; sc <= nsc && alive; ++sc) {
                    const int git = sc < nsc ? it : it + 1, gsc = sc < nsc ? sc : 0;
                    if (alive && git < my_tiles) gelu_step(git, gsc);
                }
                final_epilogue(it);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
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

bool mlp_tc_supported(int D, int DM, int planes) {
    if (D % 64 != 0 || D < 64 || D > 192 || DM % 128 != 0 || DM < 128 || planes < 1 || planes > 16) return false;
    return smem_plan(D).total + 1024 <= 227 * 1024;
}

int mlp_tc_moment_planes() { return 4; }

int launch_mlp_tc(const void* x, long long ldx, const float* moments, int planes, float eps, const void* w1_folded,
                  const void* w1_extra, const void* w2, const void* b2, void* out, long long ldo, int M, int D, int DM,
                  float* moments_out, const void* w_o, const void* resid, long long ldr, cudaStream_t st) {
    if (!mlp_tc_supported(D, DM, planes))
        return set_error(CONVNN_E_UNSUPPORTED, "mlp_tc: D=%d d_mlp=%d planes=%d is outside the fused kernel's shapes", D, DM, planes);
    if (!aligned16(x) || !aligned16(out) || !aligned16(w1_folded) || !aligned16(w1_extra) || !aligned16(w2) ||
        (!w_o && !aligned16(moments)) || (b2 && !aligned16(b2)) || (w_o && (!aligned16(w_o) || !aligned16(resid) || ldr % 8 != 0)) || ldx % 8 != 0 || ldo % 8 != 0 || (moments_out && (reinterpret_cast<uintptr_t>(moments_out) & 7u)))
        return set_error(CONVNN_E_ALIGN, "mlp_tc: pointers must be 16-byte aligned, leading dimensions multiples of 8");
    if (w_o && DM < 256)
        return set_error(CONVNN_E_UNSUPPORTED, "mlp_tc: the fused output projection needs d_mlp >= 256");
    MlpParams p{};
    p.M = M; p.D = D; p.DM = DM; p.KC = D / 64; p.n_sc = DM / SC;
    p.moments = reinterpret_cast<const float2*>(moments);
    p.mom_ld_in = p.mom_ld_out = gemm_tc_moment_stride(M);
    p.n_ptiles = (M + 2 * BM - 1) / (2 * BM);
    p.planes = planes; p.eps = eps; p.inv_d = 1.0f / (float)D;
    p.bias2 = static_cast<const __nv_bfloat16*>(b2);
    p.resid = static_cast<const __nv_bfloat16*>(resid); p.ldr = ldr;
    p.moments_out = reinterpret_cast<float2*>(moments_out);
    CUtensorMap tmX, tmO, tmW1, tmWX, tmW2, tmWO;
    {
        const uint64_t dims[2] = {(uint64_t)D, (uint64_t)M};
        const uint32_t box[2] = {64, (uint32_t)BM};
        const uint64_t sx[1] = {(uint64_t)ldx * 2}, so[1] = {(uint64_t)ldo * 2};
        if (!encode_tensor_map_bf16(&tmX, x, 2, dims, sx, box, 128)) return CONVNN_E_CUDA;
        if (!encode_tensor_map_bf16(&tmO, out, 2, dims, so, box, 128)) return CONVNN_E_CUDA;
    }
    {
        const uint64_t dims[2] = {(uint64_t)D, (uint64_t)DM}, str[1] = {(uint64_t)D * 2};
        const uint32_t box[2] = {64, 64};
        if (!encode_tensor_map_bf16(&tmW1, w1_folded, 2, dims, str, box, 128)) return CONVNN_E_CUDA;
        const uint64_t dimsx[2] = {16, (uint64_t)DM}, strx[1] = {32};
        const uint32_t boxx[2] = {16, 64};
        if (!encode_tensor_map_bf16(&tmWX, w1_extra, 2, dimsx, strx, boxx, 32)) return CONVNN_E_CUDA;
    }
    {
        const uint64_t dims[2] = {(uint64_t)DM, (uint64_t)D}, str[1] = {(uint64_t)DM * 2};
        const uint32_t box[2] = {64, (uint32_t)(D / 2)};
        if (!encode_tensor_map_bf16(&tmW2, w2, 2, dims, str, box, 128)) return CONVNN_E_CUDA;
    }
    if (w_o) {
        const uint64_t dims[2] = {(uint64_t)D, (uint64_t)D}, str[1] = {(uint64_t)D * 2};
        const uint32_t box[2] = {64, (uint32_t)(D / 4)};
        if (!encode_tensor_map_bf16(&tmWO, w_o, 2, dims, str, box, 128)) return CONVNN_E_CUDA;
    } else {
        tmWO = tmW2;
    }
    const size_t smem = smem_plan(D).total + 1024;
    auto kern = w_o ? mlp_tc_kernel<true> : mlp_tc_kernel<false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(NT); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cfg.gridDim = dim3(2);
    static std::atomic<long long> occ_caches[2] = {{-1}, {-1}};   // co-resident clusters per kernel and shared-memory size
    std::atomic<long long>& occ_cache = occ_caches[w_o ? 1 : 0];
    int max_clusters = 0;
    const long long seen = occ_cache.load(std::memory_order_relaxed);
    if (seen >= 0 && (size_t)(seen >> 20) == smem) {
        max_clusters = (int)(seen & 0xFFFFF);
    } else {
        e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
        if (e != cudaSuccess || max_clusters < 1)
            return set_error(CONVNN_E_CUDA, "cudaOccupancyMaxActiveClusters: %s", cudaGetErrorString(e));
        occ_cache.store(((long long)smem << 20) | max_clusters, std::memory_order_relaxed);
    }
    const int nc = p.n_ptiles < max_clusters ? p.n_ptiles : max_clusters;
    cfg.gridDim = dim3(2 * nc);
    e = cudaLaunchKernelEx(&cfg, kern, tmX, tmO, tmW1, tmWX, tmW2, tmWO, p);
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "mlp_tc launch: %s", cudaGetErrorString(e));
    CONVNN_CHECK_LAUNCH("mlp_tc");
    return CONVNN_OK;
}

#ifdef CONVNN_B200_MLP_TRACE
extern "C" int convnn_b200_debug_mlp_trace(unsigned long long* host_out) {
    cudaError_t e = cudaMemcpyFromSymbol(host_out, g_mlp_trace, sizeof(unsigned long long) * 16 * 64);
    return e == cudaSuccess ? 0 : -1;
}
#endif

int read_mlp_tc_status(int* out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_mlp_tc_status, sizeof(int));
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    *out = v;
    return CONVNN_OK;
}

}  // namespace convnn
