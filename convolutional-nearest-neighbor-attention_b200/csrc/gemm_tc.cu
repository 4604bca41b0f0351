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
//   warps 2-5  epilogue of the even tiles (TMEM buffer 0), warps 6-9 of the odd tiles (buffer
//              1): tcgen05.ld -> (+bias, GELU) -> bf16 -> swizzled shared-memory slab ->
//              coalesced 16-byte global stores (+ residual); two tiles drain concurrently.
//              The WIDE variant adds warps 10-17, which take the upper half of each tile's
//              column chunks (same lane quarters, same two buffers).
// A bias whose rows fit in 24 KB of shared memory is not added in the epilogue: one extra
// K = 16 MMA per tile (a 128 x 16 operand of ones times a [BN x 16] operand holding the bias)
// preloads the accumulator with it.
// The N range may be split into up to three equal parts with their own output tensors,
// which lets one launch produce k, v and q from the packed [W_k; W_v; W_q].
// Pre-norm fold (LNF): the GEMM consumes the rows x BEFORE their LayerNorm.  With W' = W * diag(gamma),
// c[n] = sum_k W'[n,k] and b'[n] = sum_k W[n,k] beta[k] + bias[n],
//   LayerNorm(x) W^T + bias = rstd * (x W'^T - mean * c + sigma * b'),    sigma = 1 / rstd,
// so the normalised rows are never written or read.  The row moments (sum x, sum x^2; produced by
// the kernel that wrote x, see MOM) are turned by one extra warp into a 128 x 16 operand chunk
// [-mean_hi, -mean_lo, -mean_hi, -mean_lo, sigma_hi, sigma_lo, sigma_hi, sigma_lo] (bfloat16 hi + lo
// splits, both 16-byte halves alike) that one extra K = 16 MMA per tile multiplies with the
// matching [c_hi, c_hi, c_lo, c_lo, b'_hi, b'_hi, b'_lo, b'_lo | 0 ...] rows fetched with the W tile;
// the epilogue multiplies by rstd.
// Row moments out (MOM): the epilogue of a GEMM with a skip connection also emits, per row and per
// (column tile, column half), the sum and the sum of squares of the values it stored.
// Every mbarrier wait is bounded (see sm100.cuh); an expiry latches the device status.
#include <atomic>

#include "common.cuh"
#include "sm100.cuh"
#include "f32x2.cuh"
#include "gelu.cuh"

namespace convnn {

__device__ int g_gemm_tc_status = 0;   // error latch of this translation unit

// Pipeline trace (a development aid, compiled in only with -DCONVNN_B200_GEMM_TRACE): when
// enabled, CTA 0 records SM clock stamps of its producer, MMA and epilogue events; four regions
// of 512 slots (producer, MMA, epilogue half 0 / 1).
#ifdef CONVNN_B200_GEMM_TRACE
__device__ int g_gemm_trace_on = 0;
__device__ unsigned long long g_gemm_trace[4 * 512];
#endif

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int MAX_STAGES = 8;
constexpr int NTHREADS = 320;         // TMA warp, MMA warp, 2 x 4 epilogue warps
constexpr int NTHREADS_WIDE = 576;    // ... or 2 x 8 epilogue warps (each tile's columns split in two)
constexpr int MOM_SLOTS = 4;          // pre-norm fold: ring of row-moment tiles (128 rows x planes), fetched
constexpr int MOM_AHEAD = 3;          // this many tiles ahead of their use

struct GemmTcParams {
    __nv_bfloat16* c[3];
    long long ldc;
    const __nv_bfloat16* bias;       // added in the epilogue, or
    const __nv_bfloat16* mma_bias;   // preloaded into the accumulator by one extra K = 16 MMA per tile
    const __nv_bfloat16* residual;   // added after rounding the GEMM result (torch: y = x + linear(...))
    long long ldr;
    float* stat[3];        // per part: per-(row, head) statistic of the stored values, or nullptr
    int stat_mode;         // CONVNN_COSINE: 1/max(norm, 1e-12); otherwise the squared norm
    int stat_pieces;       // 1, or the number of column tiles a head spans (stat[] then holds raw partial sums,
    long long stat_plane;  // one plane of stat_plane floats per piece)
    int dk, heads, rows_per_batch;   // head geometry of the statistic: stat[(b*heads + h)*rows_per_batch + r]
    int part_cols;         // output columns per part (N for a single output)
    int M, N, gelu;
    int KCH, KC, BN, BNpad;
    int n_m_tiles, n_n_tiles, n_tiles;
    int stages;            // depth of the shared-memory ring
    int wstat;             // 1: the whole W tile (BN x Kd) stays in shared memory; the ring holds A only
    int tiles_per_cta;     // wstat: each CTA owns a contiguous range of the n-major tile list
    // pre-norm fold: the moments of the A rows, [ln_planes][mom_ld] (sum, sum of squares) partial sums,
    // arrive through the tensor map tmM
    int ln_planes;
    float ln_eps, ln_inv_k;
    float2* moments_out;   // MOM: [2 * n_n_tiles][mom_ld] partial moments of the stored rows
    long long mom_ld;      // plane stride of moments_out (M rounded up to an even count)
};

__device__ __forceinline__ void fail(volatile int* abort_flag, int code) {
    *abort_flag = 1;
    atomicCAS(&g_gemm_tc_status, 0, code);
}
// CTA-pair variant: the peer's waits give up as well
__device__ __forceinline__ void fail_pair(volatile int* abort_flag, uint32_t peer_abort, int code) {
    st_cluster_u32(peer_abort, 1u);
    fail(abort_flag, code);
}

#ifdef CONVNN_B200_GEMM_TRACE
__device__ __forceinline__ bool trace_enabled() { return g_gemm_trace_on != 0; }
__device__ __forceinline__ void trace(bool on, int region, int& n) {
    if (on && n < 512) g_gemm_trace[region * 512 + n++] = clock64();
}
#else
__device__ __forceinline__ bool trace_enabled() { return false; }
__device__ __forceinline__ void trace(bool, int, int&) {}
#endif

// Epilogue, phase A (thread = one output row): 32 fp32 accumulators (+bias, GELU) -> bf16,
// written as four 16-byte slots into this warp's 32 x 64-byte staging slab.  Slot s of row
// l lands in physical slot s ^ ((l >> 1) & 3) (precomputed in `sts`), which makes both this
// row-wise write and the 8-rows-per-instruction read-back of phase B free of bank
// conflicts.  With STAT it returns the sum of squares of the ROUNDED values (the statistic
// is defined on what is stored), accumulated in four independent partial sums.
template <bool STAT, bool BIAS, bool GELU, bool LNF>
__device__ __forceinline__ float stage_chunk(const uint32_t (&sts)[4], const uint32_t (&acc)[32],
                                             const __nv_bfloat16* bias, int bias_valid, float rstd) {
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint32_t pk[4];
        uint4 bv = make_uint4(0, 0, 0, 0);
        if (BIAS) {
            if (g * 8 < bias_valid) bv = *reinterpret_cast<const uint4*>(bias + g * 8);
        }
        const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float a = __uint_as_float(acc[g * 8 + 2 * e]);
            float b = __uint_as_float(acc[g * 8 + 2 * e + 1]);
            if (LNF && !(BIAS || GELU)) { a *= rstd; b *= rstd; }
            if (BIAS || GELU) {
                // both elements of the pair go through one packed instruction per step; the
                // packed operations round like their scalar counterparts
                f32x2 x = pack2(a, b);
                if (LNF) x = mul2(x, pack2(rstd, rstd));
                if (BIAS) x = add2(x, pack2(__uint_as_float(bw[e] << 16), __uint_as_float(bw[e] & 0xffff0000u)));
                if (GELU) x = gelu_pair(x);
                unpack2(x, a, b);
            }
            __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            pk[e] = *reinterpret_cast<uint32_t*>(&h);
            if (STAT) {
                const float rx = __uint_as_float(pk[e] << 16), ry = __uint_as_float(pk[e] & 0xffff0000u);
                if (e & 1) { s2 = fmaf(rx, rx, s2); s3 = fmaf(ry, ry, s3); }
                else { s0 = fmaf(rx, rx, s0); s1 = fmaf(ry, ry, s1); }
            }
        }
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sts[g]), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]),
                     "r"(pk[3])
                     : "memory");
    }
    return (s0 + s1) + (s2 + s3);
}

// PAIR: two CTAs of a cluster form one MMA unit (tcgen05 cta_group::2): a tile is 256 rows (128
// per CTA) by BN columns of which each CTA stages BN / 2 rows of W, so every CTA reads and
// fetches half the W bytes per flop.  The even CTA issues the MMAs; loads of both CTAs credit its
// "full" barriers, completions are committed to the barriers of both CTAs, and the epilogue
// warps of both release the accumulator on the leader's "tempty" barriers.  Streaming mode only.
template <bool STAT, bool BIAS, bool GELU, bool RES, bool WIDE, bool PAIR, bool LNF = false, bool MOM = false>
__global__ void __launch_bounds__((WIDE ? NTHREADS_WIDE : NTHREADS) + (LNF ? 32 : 0), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
               const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmM,
               const GemmTcParams p) {
    static_assert(!(LNF && (PAIR || BIAS || RES)), "the pre-norm fold is built for single CTAs without bias / skip");
    static_assert(!MOM || (RES && WIDE && !PAIR && !LNF), "row moments come from the wide skip-connection epilogue");
    constexpr int STATW = WIDE ? 18 : 10;                      // LNF: the warp that prepares the extra operand chunk
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t pitch = p.KCH * 2;
    const int bn_cta = PAIR ? p.BN / 2 : p.BN;               // rows of W staged by this CTA
    const uint32_t a_bytes = BM * pitch, b_bytes = bn_cta * pitch;
    const uint32_t STAGES = p.stages;
    static_assert(!(PAIR && STAT), "the pair schedule has no fused statistic");
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;     // 0 = leader
    const int cta_id = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int n_ctas = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    constexpr int TM = PAIR ? 2 * BM : BM;                    // rows per tile
    uint8_t* sA = smem;                                        // [STAGES][128 x KCH]
    uint8_t* sB = smem + STAGES * a_bytes;                     // ring [STAGES] or resident [KC] chunks of W
    uint8_t* slabs = sB + (p.wstat ? p.KC : STAGES) * b_bytes; // one 2 KB slab per epilogue warp
    // bias through the tensor cores: a 128 x 16 operand of ones (4 KB) and, per output column, a
    // 16-element row holding the bias in element 0 (32 B per column, all column tiles)
    uint8_t* ones = slabs + (WIDE ? 16 : 8) * 2048;
    uint8_t* btile = ones + (p.mma_bias ? 4096 : 0);
    // pre-norm fold: the extra A chunk of both accumulator buffers (2 x 4 KB), the extra W rows of the
    // resident tile (bn_cta x 32 B) and rstd of the rows of both buffers, from a 1 KB boundary
    uint8_t* xa = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(btile + (p.mma_bias ? (size_t)p.n_n_tiles * bn_cta * 32 : 0)) + 1023) & ~(uintptr_t)1023);
    uint8_t* xb = xa + 2 * 4096;
    float* rstd_s = reinterpret_cast<float*>(xb + (((size_t)bn_cta * 32 + 1023) & ~(size_t)1023));
    uint8_t* mring = reinterpret_cast<uint8_t*>(rstd_s + 2 * BM);      // [MOM_SLOTS][ln_planes][128] float2
    uint64_t* bars = LNF ? reinterpret_cast<uint64_t*>(mring + (size_t)MOM_SLOTS * p.ln_planes * 1024)
                         : reinterpret_cast<uint64_t*>(btile + (p.mma_bias ? (size_t)p.n_n_tiles * bn_cta * 32 : 0));
    static_assert(!(STAT && WIDE) || LNF, "the statistic with sixteen epilogue warps is built for the pre-norm fold");
    uint64_t* full = bars;
    uint64_t* empty = bars + MAX_STAGES;
    uint64_t* tfull = bars + 2 * MAX_STAGES;
    uint64_t* tempty = tfull + 2;
    uint64_t* wfull = tempty + 2;                              // resident W tile landed
    uint64_t* xfull = wfull + 1;                               // LNF: extra A chunk of buffer 0 / 1 written
    uint64_t* mfull = xfull + 2;                               // LNF: moment tile landed in ring slot 0..3
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mfull + MOM_SLOTS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // STAT with sixteen epilogue warps: the upper column half's warp hands its part of a row's sum of squares
    // to the lower half's warp here, [accumulator buffer][tile parity of that buffer][row], and then publishes
    // the count of tiles it has handed over in ssx_seq[buffer * 4 + lane quarter]
    float* ssx = reinterpret_cast<float*>(tmem_slot + 4);
    volatile uint32_t* ssx_seq = reinterpret_cast<volatile uint32_t*>(ssx + 4 * BM);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ncols = 2u * p.BNpad;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], (WIDE ? 8 : 4) * (PAIR ? 2 : 1));
        }
        mbar_init(wfull, 1);
        mbar_init(&xfull[0], 1);
        mbar_init(&xfull[1], 1);
        for (int i = 0; i < MOM_SLOTS; ++i) mbar_init(&mfull[i], 1);
        if (STAT && WIDE)
            for (int i = 0; i < 8; ++i) ssx_seq[i] = 0u;
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmW);
        if (LNF) { prefetch_tensormap(&tmX); prefetch_tensormap(&tmM); }
    }
    if (PAIR) __syncthreads();                  // barriers initialised before the pair-wide allocation returns
    if (warp == 1) {
        if (PAIR) { tmem_alloc_pair(tmem_slot, ncols); tmem_relinquish_pair(); }
        else { tmem_alloc(tmem_slot, ncols); tmem_relinquish(); }
    }
    if (p.mma_bias) {
        // D = ones * btile^T = bias[n] in every row.  Both 16-byte halves of a row of `ones`
        // start with 1.0 and a btile row holds its bias in exactly one half, so the product
        // does not depend on how the 32-byte swizzle orders the halves.
        const uint4 one_v = make_uint4(0x00003F80u, 0u, 0u, 0u);      // bf16 1.0 in element 0
        for (int i = threadIdx.x; i < BM * 2; i += blockDim.x) reinterpret_cast<uint4*>(ones)[i] = one_v;
        const int ncols_all = p.n_n_tiles * bn_cta;
        for (int n = threadIdx.x; n < ncols_all; n += blockDim.x) {
            uint32_t b = 0;
            // row n of this CTA's bias tile: column tile n / bn_cta, this CTA's part of its columns
            const int col = (n / bn_cta) * p.BN + (int)rank * bn_cta + n % bn_cta;
            if (col < p.N) b = *reinterpret_cast<const unsigned short*>(p.mma_bias + col);
            reinterpret_cast<uint4*>(btile)[2 * n] = make_uint4(b, 0u, 0u, 0u);
            reinterpret_cast<uint4*>(btile)[2 * n + 1] = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async();                    // generic-proxy writes -> visible to the MMA's reads
    }
    tc_fence_before_sync();
    __syncthreads();
    if (PAIR) cluster_sync_all();               // both CTAs' barriers exist before any remote signal
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t peer_abort = PAIR ? map_to_cta(smem_u32(const_cast<int*>(abort_flag)), rank ^ 1u) : 0u;
    auto give_up = [&](int code) {
        if (PAIR) fail_pair(abort_flag, peer_abort, code);
        else fail(abort_flag, code);
    };

    // Tile order.  Streaming mode: tile k of this CTA is blockIdx.x + k * gridDim.x in the m-major
    // list (n fastest).  W-resident mode: a contiguous range of the n-major list (m fastest), so
    // the W tile changes at most a few times per CTA.
    const int first = p.wstat ? cta_id * p.tiles_per_cta : cta_id;
    const int step = p.wstat ? 1 : n_ctas;
    const int last = p.wstat ? min(first + p.tiles_per_cta, p.n_tiles) : p.n_tiles;
    auto tile_mn = [&](int t, int& mt, int& nt) {
        if (p.wstat) { nt = t / p.n_m_tiles; mt = t - nt * p.n_m_tiles; }
        else { mt = t / p.n_n_tiles; nt = t - mt * p.n_n_tiles; }
    };

    const uint32_t full0 = smem_u32(full), empty0 = smem_u32(empty), wfull_a = smem_u32(wfull);
    const uint32_t sA0 = smem_u32(sA), sB0 = smem_u32(sB);

    if (warp == 0) {
        if (lane == 0) {
            uint32_t s = 0, ph = 0, wloads = 0;      // ring slot and its phase, advanced incrementally
            uint32_t last_s = 0, last_ph = 0;
            bool any = false;
            int cur_nt = -1;
            bool ok = true;
            const bool tr = !PAIR && trace_enabled() && blockIdx.x == 0;
            int tn = 0;
            trace(tr, 0, tn);
            const uint32_t tx = (a_bytes + (p.wstat ? 0u : b_bytes)) * (PAIR ? 2u : 1u);
            const uint32_t lead_full0 = PAIR ? map_to_cta(full0, 0) : full0;
            for (int t = first; t < last && ok; t += step) {
                int mt, nt;
                tile_mn(t, mt, nt);
                if (p.wstat && nt != cur_nt) {
                    // every MMA that reads the old W tile has completed once the most recently
                    // filled ring stage has been released
                    if (any && !mbar_wait_a(empty0 + 8 * last_s, last_ph, abort_flag)) { give_up(15); ok = false; break; }
                    mbar_expect_tx_a(wfull_a, p.KC * b_bytes + (LNF ? (uint32_t)bn_cta * 32u : 0u));
                    for (int kc = 0; kc < p.KC; ++kc)
                        tma_load_2d_a(sB0 + kc * b_bytes, &tmW, wfull_a, kc * p.KCH, nt * p.BN);
                    if (LNF) tma_load_2d_a(smem_u32(xb), &tmX, wfull_a, 0, nt * p.BN);
                    cur_nt = nt;
                    ++wloads;
                }
                trace(tr, 0, tn);
                const int m0 = mt * TM + (int)rank * BM, n0 = nt * p.BN + (int)rank * bn_cta;
                for (int kc = 0; kc < p.KC; ++kc) {
                    if (!mbar_wait_a(empty0 + 8 * s, ph ^ 1u, abort_flag)) { give_up(11); ok = false; break; }
                    if (PAIR) {
                        if (rank == 0) mbar_expect_tx_a(full0 + 8 * s, tx);
                        tma_load_2d_pair(sA0 + s * a_bytes, &tmA, lead_full0 + 8 * s, kc * p.KCH, m0);
                        tma_load_2d_pair(sB0 + s * b_bytes, &tmW, lead_full0 + 8 * s, kc * p.KCH, n0);
                    } else {
                        mbar_expect_tx_a(full0 + 8 * s, tx);
                        tma_load_2d_a(sA0 + s * a_bytes, &tmA, full0 + 8 * s, kc * p.KCH, m0);
                        if (!p.wstat) tma_load_2d_a(sB0 + s * b_bytes, &tmW, full0 + 8 * s, kc * p.KCH, n0);
                    }
                    last_s = s; last_ph = ph; any = true;
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_idesc_bf16_f32(TM, p.BN);
            const uint64_t dhi = kmajor_desc_hi(pitch);
            const int nk16 = p.KCH / 16;
            const uint32_t tfull0 = smem_u32(tfull), tempty0 = smem_u32(tempty);
            const bool mbias = p.mma_bias != nullptr;
            const uint64_t dhi32 = kmajor_desc_hi(32);
            const uint64_t ones_desc = dhi32 | (uint64_t)((smem_u32(ones) & 0x3FFFFu) >> 4);
            const uint32_t btile0 = smem_u32(btile) & 0x3FFFFu;
            uint32_t s = 0, ph = 0, tile = 0, wloads = 0, last_stage = 0;
            int cur_nt = -1;
            bool ok = true;
            const bool tr = !PAIR && trace_enabled() && blockIdx.x == 0;
            int tn = 0;
            const uint32_t peer_empty0 = PAIR ? map_to_cta(empty0, 1) : 0u;
            const uint32_t peer_tfull0 = PAIR ? map_to_cta(tfull0, 1) : 0u;
            for (int t = first; t < last && ok; t += step, ++tile) {
                const uint32_t buf = tile & 1u, u = tile >> 1;
                if (!mbar_wait_a(tempty0 + 8 * buf, (u & 1u) ^ 1u, abort_flag)) { give_up(12); ok = false; break; }
                trace(tr, 1, tn);                           // accumulator buffer free
                int mt = 0, nt = 0;
                if (p.wstat || mbias) tile_mn(t, mt, nt);
                if (p.wstat) {
                    if (nt != cur_nt) {
                        if (!mbar_wait_a(wfull_a, wloads & 1u, abort_flag)) { give_up(16); ok = false; break; }
                        cur_nt = nt;
                        ++wloads;
                    }
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * p.BNpad;
                if (mbias) {                                 // accumulator := bias, the chunks add to it
                    const uint64_t bias_desc = dhi32 | (uint64_t)((btile0 + (uint32_t)nt * bn_cta * 32u) >> 4);
                    if (PAIR) mma_bf16_ss_pair(d_tmem, ones_desc, bias_desc, idesc, 0);
                    else mma_bf16_ss(d_tmem, ones_desc, bias_desc, idesc, 0);
                }
                for (int kc = 0; kc < p.KC; ++kc) {
                    if (!mbar_wait_a(full0 + 8 * s, ph, abort_flag)) { give_up(13); ok = false; break; }
                    tc_fence_after_sync();
                    const uint64_t adesc = dhi | (uint64_t)(((sA0 + s * a_bytes) & 0x3FFFFu) >> 4);
                    const uint64_t bdesc = dhi | (uint64_t)(((sB0 + (p.wstat ? (uint32_t)kc : s) * b_bytes) & 0x3FFFFu) >> 4);
                    if (PAIR) {
                        mma_chunk_pair(d_tmem, adesc, bdesc, idesc, nk16, (kc != 0) | mbias);
                        mma_commit_pair(empty0 + 8 * s);
                        mma_commit_pair(peer_empty0 + 8 * s);
                    } else {
                        mma_chunk(d_tmem, adesc, bdesc, idesc, nk16, (kc != 0) | mbias);
                        // LNF: the tile's last stage is released behind the extra MMA below.  The producer takes
                        // the release of the most recently filled stage as "every MMA that reads the resident W
                        // tile has completed" before it loads the next W tile, and the extra MMA reads the
                        // extra rows that travel with that tile.
                        if (LNF && kc == p.KC - 1) last_stage = s;
                        else mma_commit_a(empty0 + 8 * s);
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
                if (LNF && ok) {
                    // accumulator += [-mean, sigma] x [c, b']: the chunk the extra warp wrote for this buffer
                    if (!mbar_wait_a(smem_u32(&xfull[buf]), u & 1u, abort_flag)) { give_up(17); ok = false; break; }
                    tc_fence_after_sync();
                    const uint64_t xa_desc = dhi32 | (uint64_t)(((smem_u32(xa) + buf * 4096u) & 0x3FFFFu) >> 4);
                    const uint64_t xb_desc = dhi32 | (uint64_t)((smem_u32(xb) & 0x3FFFFu) >> 4);
                    mma_bf16_ss(d_tmem, xa_desc, xb_desc, idesc, 1);
                    mma_commit_a(empty0 + 8 * last_stage);
                }
                if (ok) {
                    if (PAIR) { mma_commit_pair(tfull0 + 8 * buf); mma_commit_pair(peer_tfull0 + 8 * buf); }
                    else mma_commit_a(tfull0 + 8 * buf);
                }
                trace(tr, 1, tn);                           // tile issued
            }
        }
    } else if (LNF && warp == STATW) {
        // Extra operand chunk of every tile: lane l prepares rows l, l + 32, l + 64, l + 96.  The
        // moments of a tile (128 rows x planes, 1 KB per plane) are fetched by TMA into a ring of
        // four slots, three tiles ahead of their use, so their DRAM latency is off the tile cadence.
        const uint32_t slot_bytes = (uint32_t)p.ln_planes * 1024u;
        auto fetch = [&](uint32_t k, int t) {                 // tile number k of this CTA, tile id t
            int mt, nt;
            tile_mn(t, mt, nt);
            const uint32_t slot = k % MOM_SLOTS;
            mbar_expect_tx(&mfull[slot], slot_bytes);
            tma_load_2d(mring + slot * slot_bytes, &tmM, &mfull[slot], mt * BM * 2, 0);
        };
        if (lane == 0)
            for (int k = 0; k < MOM_AHEAD; ++k)
                if (first + k * step < last) fetch((uint32_t)k, first + k * step);
        uint32_t tile = 0;
        bool ok = true;
        for (int t = first; t < last && ok; t += step, ++tile) {
            const uint32_t buf = tile & 1u, u = tile >> 1, slot = tile % MOM_SLOTS;
            // the slot tile + MOM_AHEAD lands in was read during the previous iteration (all lanes
            // passed its __syncwarp)
            if (lane == 0 && t + MOM_AHEAD * step < last) fetch(tile + MOM_AHEAD, t + MOM_AHEAD * step);
            ok = mbar_wait(&mfull[slot], (tile / MOM_SLOTS) & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) give_up(19); break; }
            const float2* mt_s = reinterpret_cast<const float2*>(mring + slot * slot_bytes);
            uint32_t wm[4], wsg[4];
            float rs[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float s1 = 0.f, s2 = 0.f;
                for (int pl = 0; pl < p.ln_planes; ++pl) {    // rows past M read the TMA's zero fill
                    const float2 m = mt_s[pl * BM + j * 32 + lane];
                    s1 += m.x; s2 += m.y;
                }
                const float mean = s1 * p.ln_inv_k;
                const float var = fmaxf(fmaf(-mean, mean, s2 * p.ln_inv_k), 0.f) + p.ln_eps;
                const float rstd = rsqrtf(var), sigma = var * rstd;
                rs[j] = rstd;
                // hi + lo bfloat16 splits: the products with the hi + lo splits of c and b' keep ~16 bits
                const __nv_bfloat16 mh = __float2bfloat16_rn(-mean), sh = __float2bfloat16_rn(sigma);
                const __nv_bfloat16 ml = __float2bfloat16_rn(-mean - __bfloat162float(mh));
                const __nv_bfloat16 sl = __float2bfloat16_rn(sigma - __bfloat162float(sh));
                wm[j] = (uint32_t)__bfloat16_as_ushort(mh) | ((uint32_t)__bfloat16_as_ushort(ml) << 16);
                wsg[j] = (uint32_t)__bfloat16_as_ushort(sh) | ((uint32_t)__bfloat16_as_ushort(sl) << 16);
            }
            ok = mbar_wait(&tempty[buf], (u & 1u) ^ 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) give_up(18); break; }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = j * 32 + lane;
                const uint4 v = make_uint4(wm[j], wm[j], wsg[j], wsg[j]);
                uint4* dst = reinterpret_cast<uint4*>(xa + buf * 4096 + r * 32);
                dst[0] = v;
                dst[1] = v;
                rstd_s[buf * BM + r] = rs[j];
            }
            fence_proxy_async();                    // generic-proxy writes -> visible to the MMA's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(&xfull[buf]);
        }
    } else {
        const int half = ((warp - 2) >> 2) & 1;  // which TMEM buffer / tile parity this warp drains
        const int chalf = (warp - 2) >> 3;       // WIDE: which half of the tile's column chunks
        const int lq = warp & 3;
        // columns [c_begin, c_end) of every tile belong to this warp (whole 32-column chunks)
        const int nchunk = (p.BN + 31) >> 5;
        const int csplit = WIDE ? min(p.BN, 32 * ((nchunk + 1) >> 1)) : p.BN;
        const int c_begin = chalf ? csplit : 0, c_end = chalf ? p.BN : csplit;
        const int r = lq * 32 + lane;
        const uint32_t slab = smem_u32(slabs + (warp - 2) * 2048);
        // shared-memory addresses of this lane's four 16-byte slots, for the row-wise write
        // (sts) and for the 8-rows-per-instruction read-back (lds), fixed for the whole kernel
        uint32_t sts[4], lds[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            sts[g] = slab + lane * 64 + ((g ^ ((lane >> 1) & 3)) << 4);
            const int rl = g * 8 + (lane >> 2), sl = lane & 3;
            lds[g] = slab + rl * 64 + ((sl ^ ((rl >> 1) & 3)) << 4);
        }
        uint32_t tile = half;
        bool ok = true;
        const bool tr = !PAIR && trace_enabled() && blockIdx.x == 0 && lq == 0 && lane == 0 && chalf == 0;
        const uint32_t lead_tempty0 = PAIR ? map_to_cta(smem_u32(tempty), 0) : 0u;
        int tn = 0;
        for (int t = first + half * step; t < last && ok; t += 2 * step, tile += 2) {
            int mt, nt;
            tile_mn(t, mt, nt);
            const uint32_t buf = tile & 1u, u = tile >> 1;
            const int row = mt * TM + (int)rank * BM + r;
            const int n0 = nt * p.BN;
            const int part = n0 / p.part_cols;
            const int pc0 = n0 - part * p.part_cols;          // first column inside the part
            __nv_bfloat16* cbase = part == 0 ? p.c[0] : (part == 1 ? p.c[1] : p.c[2]);
            float* stat = part == 0 ? p.stat[0] : (part == 1 ? p.stat[1] : p.stat[2]);
            const int ncol = min(p.BN, p.N - n0);             // valid columns of this tile
            // phase-B pointers of this lane: row g*8 + lane/4 of the warp's slab, columns (lane%4)*8..
            __nv_bfloat16* optr[4];
            const __nv_bfloat16* rptr[4];
            bool rok[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const int grow = mt * TM + (int)rank * BM + lq * 32 + g * 8 + (lane >> 2);
                rok[g] = grow < p.M;
                optr[g] = cbase + (long long)grow * p.ldc + pc0 + (lane & 3) * 8;
                rptr[g] = RES ? p.residual + (long long)grow * p.ldr + n0 + (lane & 3) * 8 : nullptr;
            }
            if (RES && t + 2 * step < last && (lane & 3) == 0) {
                // the skip connection's rows of this warp's NEXT tile: brought into L2 now, so that the loads in
                // that tile's chunk loop (issued only a chunk ahead of their use) do not wait on DRAM
                int mt2, nt2;
                tile_mn(t + 2 * step, mt2, nt2);
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int grow2 = mt2 * TM + (int)rank * BM + lq * 32 + g * 8 + (lane >> 2);
                    if (grow2 < p.M)
                        for (int c = c_begin; c < c_end && nt2 * p.BN + c < p.N; c += 32)
                            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.residual + (long long)grow2 * p.ldr + nt2 * p.BN + c));
                }
            }
            // statistic bookkeeping without divisions in the chunk loop
            int head = 0, head_left = 0;
            long long stat_base = 0;
            long long stat_piece = 0;
            if (STAT) {
                head = pc0 / p.dk;
                head_left = p.dk;
                if (p.stat_pieces > 1) {              // this tile is one piece of one head
                    stat_piece = (long long)((pc0 - head * p.dk) / p.BN) * p.stat_plane;
                    head_left = p.BN;
                }
                const int bb = row / p.rows_per_batch, rr = row - bb * p.rows_per_batch;
                stat_base = (long long)bb * p.heads * p.rows_per_batch + rr;
            }
            ok = mbar_wait(&tfull[buf], u & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) give_up(14); break; }
            trace(tr, 2 + half, tn);                        // accumulator ready
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(lq * 32) << 16) + buf * p.BNpad;
            const float rstd = LNF ? rstd_s[buf * BM + r] : 1.0f;
            float mo1[4] = {0.f, 0.f, 0.f, 0.f}, mo2[4] = {0.f, 0.f, 0.f, 0.f};   // MOM: this lane's partial moments
            float ss = 0.f;
            // TMEM reads run one chunk ahead of the conversion / store work (ping-pong registers)
            uint32_t ra[32], rb[32];
            uint4 resa[4], resb[4];                           // residual slices, loaded a chunk ahead of their use
            auto load_res = [&](int c, uint4 (&dst)[4]) {
                if (RES) {
                    const bool cok = c + (lane & 3) * 8 < ncol;
#pragma unroll
                    for (int g = 0; g < 4; ++g)
                        dst[g] = (rok[g] && cok) ? *reinterpret_cast<const uint4*>(rptr[g] + c) : make_uint4(0, 0, 0, 0);
                }
            };
            auto issue = [&](int c, uint32_t (&dst)[32]) {
                if (c + 32 <= p.BN) {
                    tmem_ld_x32(taddr + c, dst);
                } else {                                      // BN % 32 == 16: upper half is padding
                    uint32_t lo[16];
                    tmem_ld_x16(taddr + c, lo);
#pragma unroll
                    for (int j = 0; j < 16; ++j) { dst[j] = lo[j]; dst[16 + j] = 0u; }
                }
            };
            auto finish = [&](int c, const uint32_t (&acc)[32], const uint4 (&resv)[4], uint4 (&resn)[4]) {
                if (!WIDE && c + 32 < p.BN) load_res(c + 32, resn);    // next chunk's residual, a chunk ahead of its use
                const float css = stage_chunk<STAT, BIAS, GELU, LNF>(sts, acc, BIAS ? p.bias + n0 + c : nullptr, ncol - c, rstd);
                if (STAT) {
                    if (stat) {
                        ss += css;
                        head_left -= 32;
                        if (!WIDE && head_left == 0) {        // chunk ends a head (dk % 32 == 0)
                            if (row < p.M)
                                stat[stat_piece + stat_base + (long long)head * p.rows_per_batch] =
                                    (p.stat_mode == CONVNN_COSINE && p.stat_pieces == 1) ? 1.0f / fmaxf(sqrtf(ss), 1e-12f) : ss;
                            ss = 0.f;
                            head_left = p.dk;
                            ++head;
                        }
                    }
                }
                __syncwarp();
                // phase B: 8 rows x 64 bytes per instruction, coalesced
                const bool cok = c + (lane & 3) * 8 < ncol;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint32_t v0, v1, v2, v3;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                                 : "r"(lds[g]) : "memory");
                    if (rok[g] && cok) {
                        uint4 v = make_uint4(v0, v1, v2, v3);
                        if (RES) {
                            // bf16 + bf16 rounded to bf16 (one packed instruction per pair): exactly
                            // what the reference's `x + layer(x)` on bfloat16 tensors computes
                            const uint4 rv = resv[g];
                            __nv_bfloat162* vh = reinterpret_cast<__nv_bfloat162*>(&v);
                            const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
                            for (int e = 0; e < 4; ++e) vh[e] = __hadd2(vh[e], rh[e]);
                        }
                        if (MOM) {
                            const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float lo = __uint_as_float(vw[e] << 16), hi = __uint_as_float(vw[e] & 0xffff0000u);
                                mo1[g] += lo + hi;
                                mo2[g] = fmaf(hi, hi, fmaf(lo, lo, mo2[g]));
                            }
                        }
                        *reinterpret_cast<uint4*>(optr[g] + c) = v;
                    }
                }
                __syncwarp();
            };
            if constexpr (WIDE) {
                // four warps per scheduler cover each other's latencies: one chunk in flight per warp
                for (int c = c_begin; c < c_end; c += 32) {
                    load_res(c, resa);
                    issue(c, ra);
                    tmem_ld_wait();
                    finish(c, ra, resa, resa);
                }
            } else {
                issue(0, ra);
                load_res(0, resa);
                for (int c = 0; c < p.BN; c += 64) {
                    tmem_ld_wait();
                    if (c + 32 < p.BN) issue(c + 32, rb);
                    finish(c, ra, resa, resb);
                    if (c + 32 < p.BN) {
                        tmem_ld_wait();
                        if (c + 64 < p.BN) issue(c + 64, ra);
                        finish(c + 32, rb, resb, resa);
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(lead_tempty0 + 8 * buf);
                else mbar_arrive(&tempty[buf]);
            }
            if (STAT && WIDE) {
                // one head per tile (dk = BN): this warp has the sum over its half of the columns; the upper
                // half's warp hands its part over, the lower half's warp writes the statistic.  A slot is
                // rewritten two tiles of this buffer later, after both warps have released the accumulator
                // in between; the wait is bounded like every other.
                if (stat) {
                    float* slot = ssx + ((buf * 2u + (u & 1u)) * BM) + r;
                    volatile uint32_t* seq = ssx_seq + half * 4 + lq;
                    if (chalf) {
                        *slot = ss;
                        __threadfence_block();
                        __syncwarp();
                        if (lane == 0) *seq = u + 1u;
                    } else {
                        bool got = *seq >= u + 1u;
                        if (!got) {
                            const unsigned long long t0 = global_timer_ns();
                            for (uint32_t i = 0; i < kWaitPollLimit && !got; ++i) {
                                got = *seq >= u + 1u;
                                if (!got && (i & 255u) == 255u && (*abort_flag || global_timer_ns() - t0 > kWaitBudgetNs)) break;
                            }
                        }
                        got = __all_sync(0xffffffffu, got);
                        if (!got) { if (lane == 0) give_up(20); ok = false; }
                        __threadfence_block();
                        if (got && row < p.M) {
                            const float tot = ss + *reinterpret_cast<volatile float*>(slot);
                            stat[stat_base + (long long)head * p.rows_per_batch] =
                                p.stat_mode == CONVNN_COSINE ? 1.0f / fmaxf(sqrtf(tot), 1e-12f) : tot;
                        }
                    }
                }
            }
            if (MOM) {
                // the four lanes that share a row add up; plane = (column tile, column half)
                float2* mplane = p.moments_out + (long long)(nt * 2 + chalf) * p.mom_ld;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float a = mo1[g], b = mo2[g];
                    a += __shfl_xor_sync(0xffffffffu, a, 1); b += __shfl_xor_sync(0xffffffffu, b, 1);
                    a += __shfl_xor_sync(0xffffffffu, a, 2); b += __shfl_xor_sync(0xffffffffu, b, 2);
                    const int grow = mt * TM + (int)rank * BM + lq * 32 + g * 8 + (lane >> 2);
                    if ((lane & 3) == 0 && grow < p.M) mplane[grow] = make_float2(a, b);
                }
            }
            trace(tr, 2 + half, tn);                        // tile drained
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (PAIR) cluster_sync_all();               // the peer no longer signals or reads this CTA
    if (warp == 1) {
        tc_fence_after_sync();
        if (PAIR) tmem_dealloc_pair(tmem_base, ncols);
        else tmem_dealloc(tmem_base, ncols);
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

// Whether the per-(row, head) statistic can be produced by the GEMM epilogue: a tile must
// cover whole heads and a 32-column chunk must never straddle two heads.
bool gemm_tc_can_fuse_stats(int part_cols, int dk) {
    const int bn = dividing_tile(part_cols);
    return bn != 0 && dk % 32 == 0 && bn % dk == 0;
}

// Shared-memory plan of the pre-norm fold (W-resident mode is required: the extra W rows travel with
// the W tile).  Returns the ring depth (>= 3) or 0 when the W tile does not fit.
static int prenorm_stages(int BN, int Kd, bool wide, int planes, bool wide_stat = false) {
    const int KCH = Kd % 64 == 0 ? 64 : (Kd % 32 == 0 ? 32 : 16);
    const size_t pitch = (size_t)KCH * 2, a_bytes = BM * pitch, w_tile = (size_t)(Kd / KCH) * BN * pitch;
    const size_t fixed = 1024 + (wide ? 16 : 8) * 2048 + 1024 + 2 * 4096 + (((size_t)BN * 32 + 1023) & ~(size_t)1023) +
                         2 * BM * 4 + (size_t)MOM_SLOTS * planes * 1024 + (2 * MAX_STAGES + 7 + MOM_SLOTS) * 8 + 16 + (wide_stat ? 2048 + 64 : 0);
    if (fixed + w_tile + 3 * a_bytes > 226 * 1024) return 0;
    const int st = (int)((226 * 1024 - fixed - w_tile) / a_bytes);
    return st > MAX_STAGES ? MAX_STAGES : st;
}

static int tile_width(int N, int parts, bool has_stat) {
    if (parts > 1 || has_stat) return dividing_tile(N / parts);
    const int nt = (N + 255) / 256;
    return (((N + nt - 1) / nt) + 15) / 16 * 16;
}

// Planes of partial row moments a GEMM with `moments_out` writes for N output columns.
int gemm_tc_moment_planes(int N) { return 2 * ((N + tile_width(N, 1, false) - 1) / tile_width(N, 1, false)); }

bool gemm_tc_prenorm_supported(int N, int Kd, int parts, bool has_stat, bool gelu) {
    if (Kd % 16 != 0 || N % 8 != 0 || (parts > 1 && N % parts != 0)) return false;
    const int bn = tile_width(N, parts, has_stat);
    // the rows of A come from a GEMM with Kd output columns (or from row_moments: one plane)
    return bn != 0 && prenorm_stages(bn, Kd, gelu && !has_stat, gemm_tc_moment_planes(Kd)) >= 3;
}

long long gemm_tc_moment_stride(long long M) { return (M + 1) & ~1ll; }

int gemm_tc_stat_pieces(int part_cols, int dk) {
    const int bn = dividing_tile(part_cols);
    if (bn == 0 || dk % 32 != 0) return 0;
    if (bn % dk == 0) return 1;
    if (bn % 32 == 0 && dk % bn == 0 && dk / bn <= 8) return dk / bn;
    return 0;
}

namespace {
// out[i] = f(sum over pieces of partial[piece][i]): the statistic of heads that span several tiles
__global__ void stat_combine_kernel(const float* __restrict__ partial, long long plane, int pieces, long long n,
                                    int cosine, float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = 0.f;
    for (int p = 0; p < pieces; ++p) s += partial[(long long)p * plane + i];
    out[i] = cosine ? 1.0f / fmaxf(sqrtf(s), 1e-12f) : s;
}
}  // namespace

int launch_gemm_tc(const void* a, long long lda, const void* w, int M, int N, int Kd, int parts, void* const* c,
                   long long ldc, const GemmTcOpts& o, cudaStream_t st) {
    GemmTcParams p{};
    for (int i = 0; i < 3; ++i) {
        p.c[i] = static_cast<__nv_bfloat16*>(c[i < parts ? i : 0]);
        p.stat[i] = i < parts ? o.stat[i] : nullptr;
    }
    p.ldc = ldc; p.bias = static_cast<const __nv_bfloat16*>(o.bias); p.gelu = o.gelu;
    p.mma_bias = nullptr;
    p.residual = static_cast<const __nv_bfloat16*>(o.residual); p.ldr = o.ldr;
    p.stat_pieces = 1; p.stat_plane = 0;
    p.stat_mode = o.stat_mode; p.dk = o.dk > 0 ? o.dk : 32; p.heads = o.heads; p.rows_per_batch = o.rows_per_batch > 0 ? o.rows_per_batch : 1;
    p.M = M; p.N = N;
    p.part_cols = N / parts;
    p.KCH = Kd % 64 == 0 ? 64 : (Kd % 32 == 0 ? 32 : 16);
    p.KC = Kd / p.KCH;
    p.BN = tile_width(N, parts, o.stat[0] != nullptr);
    const bool lnf = o.ln_moments != nullptr;
    p.ln_planes = o.ln_planes; p.ln_eps = o.ln_eps; p.ln_inv_k = 1.0f / (float)Kd;
    p.moments_out = static_cast<float2*>(static_cast<void*>(o.moments_out));
    p.mom_ld = gemm_tc_moment_stride(M);
    if (lnf && (o.bias || o.residual || !o.ln_wextra || o.ln_planes < 1 || o.moments_out))
        return set_error(CONVNN_E_UNSUPPORTED, "gemm_tc: the pre-norm fold takes no bias / skip connection (fold the bias)");
    p.BNpad = pow2_at_least(p.BN, 32);
    float* stat_final[3] = {p.stat[0], p.stat[1], p.stat[2]};
    if (o.stat[0] || o.stat[1] || o.stat[2]) {
        const int pieces = gemm_tc_stat_pieces(p.part_cols, p.dk);
        if (pieces == 0 || (pieces > 1 && !o.stat_scratch))
            return set_error(CONVNN_E_UNSUPPORTED, "gemm_tc: the statistic cannot be fused for d_k=%d with %d-column tiles",
                             p.dk, p.BN);
        if (pieces > 1) {
            p.stat_pieces = pieces;
            p.stat_plane = (long long)M * p.heads;
            float* sc = o.stat_scratch;
            for (int i = 0; i < parts; ++i)
                if (p.stat[i]) { p.stat[i] = sc; sc += (long long)pieces * p.stat_plane; }
        }
    }
    p.n_m_tiles = (M + BM - 1) / BM;
    p.n_n_tiles = (N + p.BN - 1) / p.BN;
    p.n_tiles = p.n_m_tiles * p.n_n_tiles;

    const int pitch = p.KCH * 2;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // W-resident mode when the whole BN x Kd tile of W fits beside a useful ring of A chunks and
    // a CTA sees several row tiles per W tile; otherwise both operands stream through the ring.
    const bool has_stat = p.stat[0] || p.stat[1] || p.stat[2];
    // Bias through the tensor cores (one extra K = 16 MMA per tile instead of an unpack and an add
    // per element in the epilogue) when the bias rows of all column tiles fit in 24 KB.
    const size_t bias_rows = (size_t)p.n_n_tiles * p.BN * 32;
    const bool bias_by_mma = p.bias && !has_stat && bias_rows <= 24 * 1024;
    if (o.moments_out && (!o.residual || o.gelu || has_stat || (p.bias && !bias_by_mma)))
        return set_error(CONVNN_E_UNSUPPORTED, "gemm_tc: row moments are produced by the skip-connection epilogue only");
    // An epilogue that does more than convert and store (bias added per element, GELU, skip
    // connection) is bound by its own instruction latencies: sixteen epilogue warps (each tile's
    // columns split between two warps per TMEM lane quarter) cover them better than eight warps
    // with ping-pong registers.
    // The statistic epilogue of the folded K/V/Q projection too, where a tile is one head (the two warps
    // of a row exchange their halves of the sum of squares).
    const bool wide_stat = lnf && has_stat && p.stat_pieces == 1 && p.dk == p.BN && p.BN % 64 == 0 &&
                           prenorm_stages(p.BN, Kd, true, o.ln_planes, true) >= 3;
    const bool wide = wide_stat || (!has_stat && ((o.bias && !bias_by_mma) || o.gelu || o.residual));
    size_t fixed = 1024 + (wide ? 16 : 8) * 2048 + (2 * MAX_STAGES + 7 + MOM_SLOTS) * 8 + 16;
    // W-resident mode is judged against 200 KB (with more, shapes whose W tile barely fits would
    // be left with a ring too short to cover the TMA latency); the streaming ring takes all the
    // shared memory there is, which is worth 5-10 % on deep reductions (K >= 384).
    size_t budget = 200 * 1024;
    const size_t budget_stream = 226 * 1024;
    if (bias_by_mma) {
        p.mma_bias = p.bias;
        p.bias = nullptr;
        fixed += 4096 + bias_rows;
        budget = 226 * 1024;
    }
    const size_t a_bytes = (size_t)BM * pitch, b_bytes = (size_t)p.BN * pitch;
    const size_t w_tile = (size_t)p.KC * b_bytes;
    p.wstat = (w_tile + 3 * a_bytes + fixed <= budget && p.n_tiles >= 2 * sms) ? 1 : 0;
    int lnf_stages = 0;
    if (lnf) {
        lnf_stages = prenorm_stages(p.BN, Kd, wide, o.ln_planes, wide_stat);
        if (lnf_stages < 3)
            return set_error(CONVNN_E_UNSUPPORTED, "gemm_tc: the pre-norm fold needs the %d x %d tile of W resident in shared memory", p.BN, Kd);
        p.wstat = 1;
    }
    // CTA pairs (M = 256 tiles, each CTA staging half of the W rows) where both operands stream and
    // the reduction is deep enough for operand traffic to matter.
    static const bool pair_allowed = [] { const char* e = getenv("CONVNN_B200_GEMM_PAIR"); return !(e && e[0] == '0'); }();
    // Measured: +5-7 % with many column tiles (N >= 1024), a loss with one to three of them, and
    // never worth a worse last wave (tiles of 256 rows on sms / 2 clusters quantise differently).
    bool pair = pair_allowed && !p.wstat && parts == 1 && !has_stat && p.KCH == 64 && Kd >= 384 && N >= 1024 &&
                p.BN % 32 == 0 && !o.moments_out;
    if (pair) {
        const long long tp = (long long)((M + 2 * BM - 1) / (2 * BM)) * p.n_n_tiles, nc = sms / 2;
        const double eff_pair = (double)tp / (double)(((tp + nc - 1) / nc) * nc);
        const double eff_one = (double)p.n_tiles / (double)(((p.n_tiles + sms - 1) / sms) * sms);
        pair = tp >= 2 * nc && eff_pair >= 0.97 * eff_one;
    }
    if (pair && o.bias && !bias_by_mma) {
        // each CTA keeps the bias rows of its half of the columns only
        const size_t rows_cta = bias_rows / 2;
        if (rows_cta <= 24 * 1024) {
            p.mma_bias = p.bias;
            p.bias = nullptr;
            fixed += 4096 + rows_cta;
        } else {
            pair = false;
        }
    } else if (pair && bias_by_mma) {
        fixed -= bias_rows / 2;
    }
    if (pair && wide && !(o.gelu || o.residual)) fixed -= 8 * 2048;   // the plain pair epilogue has eight warps
    int grid;
    size_t smem;
    if (pair) {
        p.n_m_tiles = (M + 2 * BM - 1) / (2 * BM);
        p.n_tiles = p.n_m_tiles * p.n_n_tiles;
        const size_t stage = a_bytes + b_bytes / 2;
        int st = (int)((budget_stream - fixed) / stage);
        p.stages = st > MAX_STAGES ? MAX_STAGES : st;
        smem = fixed + (size_t)p.stages * stage;
        grid = 0;                                  // clusters are counted at launch
    } else if (p.wstat) {
        p.tiles_per_cta = (p.n_tiles + sms - 1) / sms;
        grid = (p.n_tiles + p.tiles_per_cta - 1) / p.tiles_per_cta;
        if (lnf) {
            p.stages = lnf_stages;
            smem = 226 * 1024;
        } else {
            int st_a = (int)((budget - fixed - w_tile) / a_bytes);
            p.stages = st_a > MAX_STAGES ? MAX_STAGES : st_a;
            smem = fixed + w_tile + (size_t)p.stages * a_bytes;
        }
    } else {
        grid = p.n_tiles < sms ? p.n_tiles : sms;
        int st_ab = (int)((budget_stream - fixed) / (a_bytes + b_bytes));
        p.stages = st_ab > 6 ? 6 : (st_ab < 2 ? 2 : st_ab);
        smem = fixed + (size_t)p.stages * (a_bytes + b_bytes);
    }
    CUtensorMap tmA, tmW, tmX, tmM;
    const uint64_t dimsA[2] = {(uint64_t)Kd, (uint64_t)M}, dimsW[2] = {(uint64_t)Kd, (uint64_t)N};
    const uint64_t strA[1] = {(uint64_t)lda * 2}, strW[1] = {(uint64_t)Kd * 2};
    const uint32_t boxA[2] = {(uint32_t)p.KCH, (uint32_t)BM};
    const uint32_t boxW[2] = {(uint32_t)p.KCH, (uint32_t)(pair ? p.BN / 2 : p.BN)};
    if (!encode_tensor_map_bf16(&tmA, a, 2, dimsA, strA, boxA, pitch)) return CONVNN_E_CUDA;
    if (!encode_tensor_map_bf16(&tmW, w, 2, dimsW, strW, boxW, pitch)) return CONVNN_E_CUDA;
    if (lnf) {
        // the extra W rows: (N, 16) bfloat16, 32 bytes per row, fetched with the 32-byte swizzle
        const uint64_t dimsX[2] = {16, (uint64_t)N}, strX[1] = {32};
        const uint32_t boxX[2] = {16, (uint32_t)p.BN};
        if (!aligned16(o.ln_wextra)) return set_error(CONVNN_E_ALIGN, "gemm_tc: the folded extra rows must be 16-byte aligned");
        if (!encode_tensor_map_bf16(&tmX, o.ln_wextra, 2, dimsX, strX, boxX, 32)) return CONVNN_E_CUDA;
        // the moments as float32 [planes][2 * stride]: a tile is 256 floats (128 rows) of every plane;
        // rows past M read as zero
        const uint64_t dimsM[2] = {(uint64_t)2 * M, (uint64_t)o.ln_planes}, strM[1] = {(uint64_t)gemm_tc_moment_stride(M) * 8};
        const uint32_t boxM[2] = {256, (uint32_t)o.ln_planes};
        if (!aligned16(o.ln_moments)) return set_error(CONVNN_E_ALIGN, "gemm_tc: the row moments must be 16-byte aligned");
        if (o.ln_planes > 16) return set_error(CONVNN_E_UNSUPPORTED, "gemm_tc: at most 16 planes of row moments");
        if (!encode_tensor_map_f32(&tmM, o.ln_moments, 2, dimsM, strM, boxM)) return CONVNN_E_CUDA;
    } else {
        tmX = tmW;
        tmM = tmW;
    }
    if (has_stat && (p.bias || p.residual || p.gelu))
        return set_error(CONVNN_E_UNSUPPORTED, "gemm_tc: statistics cannot be combined with bias / GELU / residual");
    if (p.gelu && p.residual) return set_error(CONVNN_E_UNSUPPORTED, "gemm_tc: GELU with a residual is not built");
#define CONVNN_GEMM_LAUNCH1(S, B, G, R, W)                                                                  \
    do {                                                                                                    \
        auto kern = gemm_tc_kernel<S, B, G, R, W, false>;                                                   \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        kern<<<grid, W ? NTHREADS_WIDE : NTHREADS, smem, st>>>(tmA, tmW, tmX, tmM, p);                           \
    } while (0)
#define CONVNN_GEMM_LAUNCH_X(S, G, R, W, LNFv, MOMv)                                                        \
    do {                                                                                                    \
        auto kern = gemm_tc_kernel<S, false, G, R, W, false, LNFv, MOMv>;                                   \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        kern<<<grid, (W ? NTHREADS_WIDE : NTHREADS) + (LNFv ? 32 : 0), smem, st>>>(tmA, tmW, tmX, tmM, p);       \
    } while (0)
#define CONVNN_GEMM_LAUNCH_PAIR(G, R, W)                                                                    \
    do {                                                                                                    \
        auto kern = gemm_tc_kernel<false, false, G, R, W, true>;                                            \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        cudaLaunchConfig_t cfg{};                                                                           \
        cudaLaunchAttribute attr[1];                                                                        \
        attr[0].id = cudaLaunchAttributeClusterDimension;                                                   \
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;           \
        cfg.blockDim = dim3(W ? NTHREADS_WIDE : NTHREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;    \
        cfg.attrs = attr; cfg.numAttrs = 1;                                                                 \
        cfg.gridDim = dim3(2);                                                                              \
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
        const int nc = p.n_tiles < max_clusters ? p.n_tiles : max_clusters;                                 \
        cfg.gridDim = dim3(2 * nc);                                                                         \
        e = cudaLaunchKernelEx(&cfg, kern, tmA, tmW, tmX, tmM, p);                                                    \
        if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "gemm_tc pair launch: %s", cudaGetErrorString(e)); \
    } while (0)
#define CONVNN_GEMM_LAUNCH(S, B, G, R)                          \
    do {                                                        \
        if (wide) CONVNN_GEMM_LAUNCH1(false, B, G, R, true);    \
        else CONVNN_GEMM_LAUNCH1(S, B, G, R, false);            \
    } while (0)
    if (lnf) {
        if (has_stat && wide) CONVNN_GEMM_LAUNCH_X(true, false, false, true, true, false);
        else if (has_stat) CONVNN_GEMM_LAUNCH_X(true, false, false, false, true, false);
        else if (p.gelu) CONVNN_GEMM_LAUNCH_X(false, true, false, true, true, false);
        else CONVNN_GEMM_LAUNCH_X(false, false, false, false, true, false);
    } else if (o.moments_out) {
        CONVNN_GEMM_LAUNCH_X(false, false, true, true, false, true);
    } else
    if (pair) {
        if (p.gelu) CONVNN_GEMM_LAUNCH_PAIR(true, false, true);
        else if (p.residual) CONVNN_GEMM_LAUNCH_PAIR(false, true, true);
        else CONVNN_GEMM_LAUNCH_PAIR(false, false, false);
    } else
    if (has_stat) CONVNN_GEMM_LAUNCH1(true, false, false, false, false);
    else if (p.gelu) { if (p.bias) CONVNN_GEMM_LAUNCH(false, true, true, false); else CONVNN_GEMM_LAUNCH(false, false, true, false); }
    else if (p.bias && p.residual) CONVNN_GEMM_LAUNCH(false, true, false, true);
    else if (p.bias) CONVNN_GEMM_LAUNCH(false, true, false, false);
    else if (p.residual) CONVNN_GEMM_LAUNCH(false, false, false, true);
    else CONVNN_GEMM_LAUNCH(false, false, false, false);
#undef CONVNN_GEMM_LAUNCH
#undef CONVNN_GEMM_LAUNCH1
#undef CONVNN_GEMM_LAUNCH_PAIR
#undef CONVNN_GEMM_LAUNCH_X
    CONVNN_CHECK_LAUNCH("gemm_tc");
    if (p.stat_pieces > 1) {
        for (int i = 0; i < parts; ++i) {
            if (!stat_final[i]) continue;
            const long long n = p.stat_plane;
            stat_combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(p.stat[i], p.stat_plane, p.stat_pieces, n,
                                                                            p.stat_mode == CONVNN_COSINE, stat_final[i]);
            CONVNN_CHECK_LAUNCH("stat_combine");
        }
    }
    return CONVNN_OK;
}

#ifdef CONVNN_B200_GEMM_TRACE
// Copies up to 2048 recorded clock stamps to `host_out` (host memory), clears the trace and
// switches recording on or off.  Synchronises the device.
extern "C" int convnn_b200_debug_gemm_trace(int enable, unsigned long long* host_out, int n) {
    cudaError_t e = cudaSuccess;
    if (host_out && n > 0) {
        if (n > 4 * 512) n = 4 * 512;
        e = cudaMemcpyFromSymbol(host_out, g_gemm_trace, sizeof(unsigned long long) * n);
        if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    }
    static const unsigned long long zeros[4 * 512] = {0};
    e = cudaMemcpyToSymbol(g_gemm_trace, zeros, sizeof(zeros));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_gemm_trace_on, &enable, sizeof(int));
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaMemcpyToSymbol: %s", cudaGetErrorString(e));
    return CONVNN_OK;
}
#endif

int read_gemm_tc_status(int* out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_gemm_tc_status, sizeof(int));
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    *out = v;
    return CONVNN_OK;
}

}  // namespace convnn
