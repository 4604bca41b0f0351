// Selection step shared by the tensor-core similarity kernels: a thread owns one key row
// (= its TMEM lane) and is handed W accumulator columns of that row at a time.
#pragma once
#include "common.cuh"
#include "toplist.cuh"
#include "f32x2.cuh"

namespace convnn {

constexpr int kSelGroup = 128;    // threads per epilogue group = stride of the key staging buffer

// Columns 0 .. W-1 of a row: insertion number j only touches the first j + 1 slots.
template <int NSEL, int W, int J>
__device__ __forceinline__ void prefix_insert(TopList<NSEL>& top, const float (&key)[W], bool row_ok, int left) {
    if constexpr (J < W) {
        if (row_ok && J < left) top.template insert_sorted_first<J>(key[J], J);
        prefix_insert<NSEL, W, J + 1>(top, key, row_ok, left);
    }
}

// One chunk of W accumulator columns of this thread's row: keys, then either plain inserts
// (the first 32 columns of a row, where most values enter the list anyway) or a threshold
// mask followed by a drain loop that only visits the survivors.
// qs points at the W column statistics of this chunk in shared memory (16-byte aligned, the same
// for every lane: broadcast loads); cv holds the candidate token of column (32-aligned base +
// lane).  P needs the fields metric, sampled and S (number of candidate columns).
template <int NSEL, int W, class P>
__device__ __forceinline__ void consume(TopList<NSEL>& top, const uint32_t (&acc)[W], int col0, int lane_off,
                                        const float* qs, int cv, const P& p, int row, bool row_ok, float sentinel,
                                        float* ks) {
    float key[W];
    if (p.metric != CONVNN_MATMUL) {
        const f32x2 two = pack2(2.0f, 2.0f);
#pragma unroll
        for (int j4 = 0; j4 < W / 4; ++j4) {
            const float4 s4 = *reinterpret_cast<const float4*>(qs + 4 * j4);
            const f32x2 d01 = pack2(__uint_as_float(acc[4 * j4]), __uint_as_float(acc[4 * j4 + 1]));
            const f32x2 d23 = pack2(__uint_as_float(acc[4 * j4 + 2]), __uint_as_float(acc[4 * j4 + 3]));
            f32x2 k01, k23;
            if (p.metric == CONVNN_COSINE) {
                k01 = mul2(d01, pack2(s4.x, s4.y));
                k23 = mul2(d23, pack2(s4.z, s4.w));
            } else {
                k01 = fma2(two, d01, pack2(-s4.x, -s4.y));
                k23 = fma2(two, d23, pack2(-s4.z, -s4.w));
            }
            unpack2(k01, key[4 * j4], key[4 * j4 + 1]);
            unpack2(k23, key[4 * j4 + 2], key[4 * j4 + 3]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < W; ++j) key[j] = __uint_as_float(acc[j]);
    }
    if (p.sampled) {
#pragma unroll
        for (int j = 0; j < W; ++j) {
            const int cj = __shfl_sync(0xffffffffu, cv, lane_off + j);
            if (cj == row) key[j] = sentinel;
        }
    }
    const int left = p.S - col0;                       // valid columns from col0 on
    if (col0 < 32) {
        if (col0 == 0) {                               // the list is still filling up
            prefix_insert<NSEL, W, 0>(top, key, row_ok, left);
        } else {
#pragma unroll
            for (int j = 0; j < W; ++j)
                if (row_ok && j < left) top.insert_sorted(key[j], col0 + j);
        }
        return;
    }
    const float thr = top.worst();
    uint32_t mask = 0;
#pragma unroll
    for (int j = 0; j < W; ++j) mask |= (key[j] > thr) ? (1u << j) : 0u;
    if (left < W) mask &= (left <= 0) ? 0u : ((1u << left) - 1u);
    if (!row_ok) mask = 0;
    // The warp runs as many drain steps as its busiest lane has survivors (one reduction instead of
    // a vote per step); each step loads the next survivor's key while the current one is inserted.
    const int steps = __reduce_max_sync(0xffffffffu, __popc(mask));
    if (steps) {
        // keys go through shared memory so the drain loop can pick column j per lane
#pragma unroll
        for (int j = 0; j < W; ++j) ks[j * kSelGroup] = key[j];
        int j = mask ? __ffs(mask) - 1 : 0;
        float k = ks[j * kSelGroup];
        for (int it = 0; it < steps; ++it) {
            const bool live = mask != 0;
            const float kc = k;
            const int jc = j;
            mask &= mask - 1;
            j = mask ? __ffs(mask) - 1 : 0;
            k = ks[j * kSelGroup];
            if (live && kc > top.worst()) top.insert_sorted(kc, col0 + jc);
        }
    }
}

// Ranking key of a sampled row's own column: the finite stand-in the reference uses
// (-0.1 for the "larger is better" metrics, +1.1 for the distance), expressed in key units.
__device__ __forceinline__ float self_sentinel(int metric, float kst, float sqrt_dk) {
    if (metric == CONVNN_COSINE) return -0.1f / kst;
    if (metric == CONVNN_MATMUL) return -0.1f * sqrt_dk;
    return kst - 1.21f;
}

// Writes one row's selected (token, value) pairs: keys back to similarity values, candidate
// columns back to token indices, the row itself in slot 0 for the sampled modes.
template <int NSEL, class P>
__device__ __forceinline__ void write_selection(const TopList<NSEL>& top, const P& p, long long obase, int row,
                                                float kst) {
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

}  // namespace convnn
