// Similarity + streaming top-K on the FP32 SIMT pipes.
//
// One thread owns one key token (a row of the similarity matrix) of one (batch, head);
// a CTA owns 128 consecutive rows.  Candidate columns are visited in increasing order in
// tiles of 64; the 128x64 tile of dot products lives in registers (64 accumulators per
// thread), is turned into a ranking key and is filtered against the thread's sorted
// list, so the T x S matrix never exists in memory.  Strict comparisons while scanning
// left to right make the lower candidate column win exact ties.
//
// Ranking keys (larger is better) and the values reported for the survivors:
//   cosine     key = dot * qinv[j]            val = key * kinv[i]
//   matmul     key = dot                      val = key / sqrt(d_k)
//   euclidean  key = 2*dot - |q_j|^2          val = sqrt(max(|k_i|^2 - key, 0))
// The sampled modes replace the entry (cand[j] == i) by the reference's finite sentinel
// (-0.1, or 1.1 for euclidean; layers.py:234-235, 291-292) expressed in key space.
//
// This is the float32 path of the library (accuracy ~1e-7 so that index sets match the
// reference down to 1e-6 gaps) and the fallback for bfloat16 shapes outside the tcgen05
// kernel's envelope.
#pragma once
#include <math_constants.h>

#include "common.cuh"
#include "toplist.cuh"

namespace convnn {
namespace simt_topk {

constexpr int ROWS = 128;   // rows (key tokens) per CTA = threads per CTA
constexpr int COLS = 64;    // candidate columns per register tile
constexpr int CK = 32;      // channels staged per step

template <typename T, int KCAP>
__global__ void __launch_bounds__(ROWS) sim_topk_simt_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const float* __restrict__ qstat,
    const float* __restrict__ kstat, const int32_t* __restrict__ cand, int32_t* __restrict__ idx,
    float* __restrict__ val, int T_, int S, int H, int Cp, int K, int nsel, int metric, int sampled,
    float sqrt_dk) {
    __shared__ float ks[CK][ROWS + 1];
    __shared__ __align__(16) float qs[COLS][CK + 4];
    __shared__ float qst[COLS];
    __shared__ int cnd[COLS];

    const int tid = threadIdx.x;
    const int bh = blockIdx.y;
    const int b = bh / H, h = bh - b * H;
    const int row0 = blockIdx.x * ROWS;
    const int row = row0 + tid;
    const bool row_ok = row < T_;

    const T* kb = k + ((long long)b * T_ * H + h) * Cp;   // + token * H*Cp + c
    const T* qb = q + ((long long)b * S * H + h) * Cp;
    const long long tstride = (long long)H * Cp;

    float kst = 0.f;
    if (row_ok && metric != CONVNN_MATMUL) kst = kstat[((long long)b * H + h) * T_ + row];
    float sentinel = -CUDART_INF_F;
    if (sampled) {
        if (metric == CONVNN_COSINE) sentinel = -0.1f / kst;
        else if (metric == CONVNN_MATMUL) sentinel = -0.1f * sqrt_dk;
        else sentinel = kst - 1.21f;
    }

    TopList<KCAP> top;
    top.init();

    const int lc = tid & 31, lr = tid >> 5;   // staging: channel lc, rows / columns lr + 4*i

    for (int c0 = 0; c0 < S; c0 += COLS) {
        float acc[COLS];
#pragma unroll
        for (int j = 0; j < COLS; ++j) acc[j] = 0.f;

        if (tid < COLS) {
            int col = c0 + tid;
            qst[tid] = (col < S && metric != CONVNN_MATMUL) ? qstat[((long long)b * H + h) * S + col] : 0.f;
            cnd[tid] = (sampled && col < S) ? cand[col] : -1;
        }

        for (int ch0 = 0; ch0 < Cp; ch0 += CK) {
            __syncthreads();   // previous chunk fully consumed
            const bool ch_ok = ch0 + lc < Cp;
#pragma unroll 4
            for (int i = 0; i < ROWS / 4; ++i) {
                int r = lr + 4 * i;
                int tok = row0 + r;
                ks[lc][r] = (ch_ok && tok < T_) ? to_f32<T>(kb[tok * tstride + ch0 + lc]) : 0.f;
            }
#pragma unroll 4
            for (int i = 0; i < COLS / 4; ++i) {
                int j = lr + 4 * i;
                int col = c0 + j;
                qs[j][lc] = (ch_ok && col < S) ? to_f32<T>(qb[col * tstride + ch0 + lc]) : 0.f;
            }
            __syncthreads();
#pragma unroll
            for (int c4 = 0; c4 < CK; c4 += 4) {
                const float k0 = ks[c4 + 0][tid], k1 = ks[c4 + 1][tid];
                const float k2 = ks[c4 + 2][tid], k3 = ks[c4 + 3][tid];
#pragma unroll
                for (int j = 0; j < COLS; ++j) {
                    const float4 q4 = *reinterpret_cast<const float4*>(&qs[j][c4]);
                    float a = acc[j];
                    a = fmaf(k0, q4.x, a);
                    a = fmaf(k1, q4.y, a);
                    a = fmaf(k2, q4.z, a);
                    a = fmaf(k3, q4.w, a);
                    acc[j] = a;
                }
            }
        }

        if (row_ok) {
#pragma unroll
            for (int j = 0; j < COLS; ++j) {
                const int col = c0 + j;
                if (col < S) {
                    float key;
                    if (metric == CONVNN_COSINE) key = acc[j] * qst[j];
                    else if (metric == CONVNN_MATMUL) key = acc[j];
                    else key = fmaf(2.0f, acc[j], -qst[j]);
                    if (sampled && cnd[j] == row) key = sentinel;
                    if (key > top.worst()) top.insert(key, col);
                }
            }
        }
        __syncthreads();   // qst / cnd are rewritten by the next tile
    }

    if (!row_ok) return;
    const long long obase = (((long long)b * H + h) * T_ + row) * K;
    int off = 0;
    if (sampled) {
        idx[obase] = row;
        val[obase] = 1.0f;
        off = 1;
    }
#pragma unroll
    for (int s = 0; s < KCAP; ++s) {
        if (s < nsel) {
            const int col = top.i[s];
            const float key = top.v[s];
            float v;
            if (metric == CONVNN_COSINE) v = key * kst;
            else if (metric == CONVNN_MATMUL) v = key / sqrt_dk;
            else v = sqrtf(fmaxf(kst - key, 0.f));
            int tok = col;
            if (sampled) {
                tok = cand[col];
                if (tok == row) v = (metric == CONVNN_EUCLIDEAN) ? 1.1f : -0.1f;
            }
            idx[obase + off + s] = tok;
            val[obase + off + s] = v;
        }
    }
}

template <typename T>
int dispatch(const convnn_desc* d, const Dims& dm, const void* q, const void* k, const float* qstat,
             const float* kstat, const int32_t* cand, int32_t* idx, float* val, cudaStream_t st) {
    dim3 grid((dm.T + ROWS - 1) / ROWS, dm.B * dm.H);
    const float sq = (float)sqrt((double)dm.dk);
#define CONVNN_LAUNCH(KC)                                                                           \
    sim_topk_simt_kernel<T, KC><<<grid, ROWS, 0, st>>>(static_cast<const T*>(q), static_cast<const T*>(k), \
        qstat, kstat, cand, idx, val, dm.T, dm.S, dm.H, dm.Cp, dm.K, dm.nsel, d->metric, d->sampled, sq)
    const int n = dm.nsel;
    if (n <= 4) CONVNN_LAUNCH(4);
    else if (n <= 8) CONVNN_LAUNCH(8);
    else if (n <= 12) CONVNN_LAUNCH(12);
    else if (n <= 16) CONVNN_LAUNCH(16);
    else CONVNN_LAUNCH(32);
#undef CONVNN_LAUNCH
    CONVNN_CHECK_LAUNCH("sim_topk_simt");
    return CONVNN_OK;
}

}  // namespace simt_topk
}  // namespace convnn
