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
};

}  // namespace convnn
