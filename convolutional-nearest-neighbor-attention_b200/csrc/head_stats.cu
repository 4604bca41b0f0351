// Per-(row, head) post-pass over a projected q / k / v tensor (B, rows, H, Cp):
// writes the optional coordinate channel (reference layers.py:439-450) and the padding
// channels, and reduces the statistic the similarity needs from the STORED values
// (so that a bfloat16 tensor's norm is the norm of the rounded vector):
//   cosine    -> 1 / max(||t||, 1e-12)   (F.normalize's eps, layers.py:337-338)
//   euclidean -> ||t||^2                  (layers.py:328-329)
#include "common.cuh"

namespace convnn {
namespace {

// torch.linspace(-1, 1, steps)[i] in float32: stepped from the start below the middle
// and back from the end above it.
__device__ __forceinline__ float linspace_pm1(int i, int steps) {
    if (steps <= 1) return -1.0f;
    float step = 2.0f / (float)(steps - 1);
    return (i < steps / 2) ? (-1.0f + step * (float)i) : (1.0f - step * (float)(steps - 1 - i));
}

template <typename T>
__global__ void head_stats_kernel(T* t, float* stat, int B, int rows, int H, int dk, int C, int Cp,
                                  int coord, int metric) {
    const int warps_per_block = blockDim.x >> 5;
    const long long total = (long long)B * rows * H;
    const int lane = threadIdx.x & 31;
    for (long long w = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); w < total;
         w += (long long)gridDim.x * warps_per_block) {
        int h = (int)(w % H);
        long long br = w / H;
        int r = (int)(br % rows);
        int b = (int)(br / rows);
        T* p = t + (br * H + h) * Cp;
        if (coord) {
            for (int c = dk + lane; c < Cp; c += 32)
                p[c] = from_f32<T>(c == dk ? linspace_pm1(r, rows) : 0.0f);
            __syncwarp();
        }
        if (stat) {
            float ss = 0.f;
            constexpr int VEC = 16 / sizeof(T);
            if (C % VEC == 0 && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
                for (int c = lane * VEC; c < C; c += 32 * VEC) {     // 16-byte loads
                    const uint4 raw = *reinterpret_cast<const uint4*>(p + c);
                    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
                    for (int j = 0; j < VEC; ++j) {
                        const float v = to_f32<T>(e[j]);
                        ss = fmaf(v, v, ss);
                    }
                }
            } else {
                for (int c = lane; c < C; c += 32) {
                    float v = to_f32<T>(p[c]);
                    ss = fmaf(v, v, ss);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) {
                float s = (metric == CONVNN_COSINE) ? 1.0f / fmaxf(sqrtf(ss), 1e-12f) : ss;
                stat[((long long)b * H + h) * rows + r] = s;
            }
        }
    }
}

}  // namespace

int launch_head_fill_and_stats(const convnn_desc* d, const Dims& dm, void* t, int rows, float* stat,
                               cudaStream_t st) {
    if (!d->coord && !stat) return CONVNN_OK;
    long long total = (long long)dm.B * rows * dm.H;
    int blocks = (int)((total + 7) / 8);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    if (d->dtype == CONVNN_F32)
        head_stats_kernel<float><<<blocks, 256, 0, st>>>(static_cast<float*>(t), stat, dm.B, rows, dm.H,
                                                        dm.dk, dm.C, dm.Cp, d->coord, d->metric);
    else
        head_stats_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<__nv_bfloat16*>(t), stat, dm.B,
                                                                rows, dm.H, dm.dk, dm.C, dm.Cp, d->coord,
                                                                d->metric);
    CONVNN_CHECK_LAUNCH("head_stats");
    return CONVNN_OK;
}

}  // namespace convnn
