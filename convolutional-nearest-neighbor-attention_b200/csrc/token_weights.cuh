// Weights over a token's K selected similarity values.
#pragma once

namespace convnn {

// p[j] for one token (layers.py:352-355, 394-397): softmax(+-val), val, or 1/(val+1e-8).
__device__ __forceinline__ void token_weights(const float* __restrict__ val, float* __restrict__ p, int K,
                                              bool maximum, bool softmax) {
    if (softmax) {
        float m = -3.402823466e38f;
        for (int j = 0; j < K; ++j) {
            float x = maximum ? val[j] : -val[j];
            m = fmaxf(m, x);
        }
        float s = 0.f;
        for (int j = 0; j < K; ++j) {
            float e = expf((maximum ? val[j] : -val[j]) - m);
            p[j] = e;
            s += e;
        }
        for (int j = 0; j < K; ++j) p[j] = p[j] / s;
    } else {
        for (int j = 0; j < K; ++j) p[j] = maximum ? val[j] : 1.0f / (val[j] + 1e-8f);
    }
}

}  // namespace convnn
