// Register-resident sorted list of the best N (key, column) pairs seen so far.
// Every index is a compile-time constant after unrolling, so both arrays stay in
// registers.  Larger key is better; among equal keys the one inserted first stays ahead,
// which, with columns offered in increasing order, keeps the lower column.
#pragma once
#include <math_constants.h>

namespace convnn {

template <int N>
struct TopList {
    float v[N];
    int i[N];

    __device__ __forceinline__ void init() {
#pragma unroll
        for (int s = 0; s < N; ++s) {
            v[s] = -CUDART_INF_F;
            i[s] = 0;   // a valid token index even if a slot is never filled
        }
    }
    __device__ __forceinline__ float worst() const { return v[N - 1]; }

    // Precondition: key > worst().
    __device__ __forceinline__ void insert(float key, int col) {
        v[N - 1] = key;
        i[N - 1] = col;
#pragma unroll
        for (int s = N - 1; s > 0; --s) {
            const bool up = v[s] > v[s - 1];
            const float hv = up ? v[s] : v[s - 1], lv = up ? v[s - 1] : v[s];
            const int hi = up ? i[s] : i[s - 1], li = up ? i[s - 1] : i[s];
            v[s - 1] = hv; v[s] = lv;
            i[s - 1] = hi; i[s] = li;
        }
    }

    // Same result as insert() for any key (no precondition), written so that every slot is
    // computed from the OLD neighbours with independent compare/select pairs: no serial
    // dependency chain through the list, which matters when one warp per scheduler runs it.
    __device__ __forceinline__ void insert_sorted(float key, int col) {
#pragma unroll
        for (int s = N - 1; s >= 1; --s) {
            const bool gt = key > v[s];
            const bool gtp = key > v[s - 1];
            v[s] = gt ? (gtp ? v[s - 1] : key) : v[s];
            i[s] = gt ? (gtp ? i[s - 1] : col) : i[s];
        }
        const bool g0 = key > v[0];
        v[0] = g0 ? key : v[0];
        i[0] = g0 ? col : i[0];
    }

    // insert_sorted() for a list that has received at most J insertions so far: slots above J
    // still hold the initial -inf and would only be shifted onto each other, so they are left out.
    template <int J>
    __device__ __forceinline__ void insert_sorted_first(float key, int col) {
        constexpr int TOP = J < N - 1 ? J : N - 1;
#pragma unroll
        for (int s = TOP; s >= 1; --s) {
            const bool gt = key > v[s];
            const bool gtp = key > v[s - 1];
            v[s] = gt ? (gtp ? v[s - 1] : key) : v[s];
            i[s] = gt ? (gtp ? i[s - 1] : col) : i[s];
        }
        const bool g0 = key > v[0];
        v[0] = g0 ? key : v[0];
        i[0] = g0 ? col : i[0];
    }

    // Insert under the full (key, column) order: among equal keys the lower column ranks
    // first wherever it came from.  Used to merge lists built over interleaved column ranges,
    // where "inserted first" no longer means "lower column".
    __device__ __forceinline__ static bool ranks_before(float k, int c, float v0, int i0) {
        return k > v0 || (k == v0 && c < i0);
    }
    __device__ __forceinline__ void insert_ordered(float key, int col) {
#pragma unroll
        for (int s = N - 1; s >= 1; --s) {
            const bool gt = ranks_before(key, col, v[s], i[s]);
            const bool gtp = ranks_before(key, col, v[s - 1], i[s - 1]);
            v[s] = gt ? (gtp ? v[s - 1] : key) : v[s];
            i[s] = gt ? (gtp ? i[s - 1] : col) : i[s];
        }
        const bool g0 = ranks_before(key, col, v[0], i[0]);
        v[0] = g0 ? key : v[0];
        i[0] = g0 ? col : i[0];
    }
};

}  // namespace convnn
