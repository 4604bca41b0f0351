// Memory-bound pieces of the ViT encoder around the ConvNN block (callers of the hot
// path): LayerNorm, patch unfolding and the token-embedding tail.  One warp per row,
// 16-byte loads and stores, statistics in fp32, one rounding to the storage type at each
// point where the reference's eager ops would round (reference vit.py:100-135, 247-270).
#include "common.cuh"
#include "f32x2.cuh"

namespace convnn {
namespace {

template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float* out) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < Vec16<T>::N; ++j) out[j] = to_f32<T>(e[j]);
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float* in) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int j = 0; j < Vec16<T>::N; ++j) e[j] = from_f32<T>(in[j]);
    *reinterpret_cast<uint4*>(p) = raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// LayerNorm of `rows` rows of length D.  NV = 16-byte vectors held per lane (row cached in
// registers).  Output row r goes to y + out_row(r) * ldy; with `pe` != nullptr the kernel
// is the embedding tail: row r = (b, n) of the patch projection lands at token 1 + n of
// image b with pe[1 + n] added after rounding, and `cls_rows` extra rows write cls + pe[0].
template <typename T, int NV, bool EMBED>
__global__ void __launch_bounds__(256) layernorm_kernel(const T* __restrict__ x, long long ldx,
                                                        const T* __restrict__ gamma, const T* __restrict__ beta,
                                                        float eps, T* __restrict__ y, long long ldy, long long rows,
                                                        int D, const T* __restrict__ pe, const T* __restrict__ cls,
                                                        int Np, long long cls_rows, float2* __restrict__ moments) {
    // moments (or nullptr): (sum, sum of squares) of every STORED output row, indexed by output row: what the
    // pre-norm fold of the first GEMM behind the embedding needs
    constexpr int V = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const long long wpb = blockDim.x >> 5;
    const int nvec = D / V;
    for (long long r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows + cls_rows; r += (long long)gridDim.x * wpb) {
        if (EMBED && r >= rows) {              // class-token row of image b: cls + pe[0]
            const long long b = r - rows;
            T* out = y + b * (Np + 1) * ldy;
            float m1 = 0.f, m2 = 0.f;
            for (int i = lane; i < nvec; i += 32) {
                float c[V], p0[V];
                load_vec<T>(cls + i * V, c);
                load_vec<T>(pe + i * V, p0);
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    c[j] += p0[j];
                    const float rv = to_f32<T>(from_f32<T>(c[j]));
                    m1 += rv;
                    m2 = fmaf(rv, rv, m2);
                }
                store_vec<T>(out + i * V, c);
            }
            if (moments) {
                m1 = warp_sum(m1);
                m2 = warp_sum(m2);
                if (lane == 0) moments[b * (Np + 1)] = make_float2(m1, m2);
            }
            continue;
        }
        const T* in = x + r * ldx;
        long long orow = r;
        const T* perow = nullptr;
        if (EMBED && pe) {
            const long long b = r / Np, n = r - b * Np;
            orow = b * (Np + 1) + 1 + n;
            perow = pe + (1 + n) * (long long)D;
        }
        float v[NV][V];
        uint4 pv_raw[EMBED ? NV : 1];           // the positional row, fetched with the input row
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int i = lane + 32 * k;
            if (i < nvec) {
                load_vec<T>(in + i * V, v[k]);
                if (EMBED && perow) pv_raw[EMBED ? k : 0] = *reinterpret_cast<const uint4*>(perow + i * V);
#pragma unroll
                for (int j = 0; j < V; ++j) s += v[k][j];
            }
        }
        const float mean = warp_sum(s) / (float)D;
        float q = 0.f;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int i = lane + 32 * k;
            if (i < nvec) {
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    const float d = v[k][j] - mean;
                    q = fmaf(d, d, q);
                }
            }
        }
        const float rstd = rsqrtf(warp_sum(q) / (float)D + eps);
        T* out = y + orow * ldy;
        float m1 = 0.f, m2 = 0.f;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int i = lane + 32 * k;
            if (i < nvec) {
                float g[V], bt[V], o[V];
                load_vec<T>(gamma + i * V, g);
                load_vec<T>(beta + i * V, bt);
#pragma unroll
                for (int j = 0; j < V; ++j) o[j] = (v[k][j] - mean) * rstd * g[j] + bt[j];
                if (EMBED && perow) {
                    const T* pv = reinterpret_cast<const T*>(&pv_raw[EMBED ? k : 0]);
#pragma unroll
                    for (int j = 0; j < V; ++j) o[j] = to_f32<T>(from_f32<T>(o[j])) + to_f32<T>(pv[j]);
                }
                if (EMBED && moments) {
#pragma unroll
                    for (int j = 0; j < V; ++j) {
                        const float rv = to_f32<T>(from_f32<T>(o[j]));
                        m1 += rv;
                        m2 = fmaf(rv, rv, m2);
                    }
                }
                store_vec<T>(out + i * V, o);
            }
        }
        if (EMBED && moments) {
            m1 = warp_sum(m1);
            m2 = warp_sum(m2);
            if (lane == 0) moments[orow] = make_float2(m1, m2);
        }
    }
}

// bfloat16 rows of at most 256 channels: one 16-byte vector per lane and row, arithmetic on packed
// fp32 pairs, affine parameters held in registers.  Same results as the generic kernel.  A warp
// works on R consecutive rows at a time and requests the next R while it does so: what bounds
// the kernel is the number of bytes an SM has in flight, not its arithmetic.
// EMBED: the embedding tail of the generic kernel (row (b, n) lands at token 1 + n of image b with pe[1 + n]
// added after rounding, `cls_rows` class-token rows cls + pe[0], optional moments of every stored row);
// rows < 2^31.
template <int R, int MINB, bool EMBED>
__global__ void __launch_bounds__(256, MINB) layernorm_bf16_row256_kernel(
    const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ gamma,
    const __nv_bfloat16* __restrict__ beta, float eps, __nv_bfloat16* __restrict__ y, long long ldy, long long rows,
    int D, const __nv_bfloat16* __restrict__ pe, const __nv_bfloat16* __restrict__ cls, int Np, long long cls_rows,
    float2* __restrict__ moments) {
    const int lane = threadIdx.x & 31;
    const long long wpb = blockDim.x >> 5;
    const bool act = lane < D / 8;
    const float invD = 1.0f / (float)D;
    f32x2 g2[4], b2[4];
    {
        const uint4 z = make_uint4(0, 0, 0, 0);
        bf16x8_to_f32x2(act ? *reinterpret_cast<const uint4*>(gamma + lane * 8) : z, g2);
        bf16x8_to_f32x2(act ? *reinterpret_cast<const uint4*>(beta + lane * 8) : z, b2);
    }
    const long long stride = (long long)gridDim.x * wpb * R;
    long long r0 = (blockIdx.x * wpb + (threadIdx.x >> 5)) * R;
    uint4 nxt[R];
#pragma unroll
    for (int j = 0; j < R; ++j)
        nxt[j] = (act && r0 + j < rows) ? *reinterpret_cast<const uint4*>(x + (r0 + j) * ldx + lane * 8) : make_uint4(0, 0, 0, 0);
    for (; r0 < rows; r0 += stride) {
        f32x2 d2[R][4];
        float mean[R], q[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            bf16x8_to_f32x2(nxt[j], d2[j]);
            float s0, s1;
            unpack2(add2(add2(d2[j][0], d2[j][1]), add2(d2[j][2], d2[j][3])), s0, s1);
            mean[j] = s0 + s1;
        }
#pragma unroll
        for (int j = 0; j < R; ++j)                        // next rows' loads overlap this group's arithmetic
            if (act && r0 + stride + j < rows)
                nxt[j] = *reinterpret_cast<const uint4*>(x + (r0 + stride + j) * ldx + lane * 8);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int j = 0; j < R; ++j) mean[j] += __shfl_xor_sync(0xffffffffu, mean[j], o);
#pragma unroll
        for (int j = 0; j < R; ++j) {
            mean[j] *= invD;
            const f32x2 nm = pack2(-mean[j], -mean[j]);
            f32x2 q2 = 0ull;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                d2[j][e] = add2(d2[j][e], nm);
                q2 = fma2(d2[j][e], d2[j][e], q2);
            }
            float q0, q1;
            unpack2(q2, q0, q1);
            q[j] = act ? q0 + q1 : 0.f;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int j = 0; j < R; ++j) q[j] += __shfl_xor_sync(0xffffffffu, q[j], o);
        float m1[R], m2[R];
        long long orow[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const float rstd = rsqrtf(q[j] * invD + eps);
            m1[j] = m2[j] = 0.f;
            orow[j] = r0 + j;
            if (act && r0 + j < rows) {
                const f32x2 r2 = pack2(rstd, rstd);
                f32x2 o2[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) o2[e] = fma2(mul2(d2[j][e], r2), g2[e], b2[e]);
                uint4 ov = f32x2_to_bf16x8(o2);
                if (EMBED) {
                    const unsigned rr = (unsigned)(r0 + j), b = rr / (unsigned)Np, n = rr - b * (unsigned)Np;
                    orow[j] = (long long)b * (Np + 1) + 1 + n;
                    f32x2 pf[4];
                    bf16x8_to_f32x2(*reinterpret_cast<const uint4*>(pe + (long long)(1 + n) * D + lane * 8), pf);
                    bf16x8_to_f32x2(ov, o2);                       // the rounded LayerNorm output, then + pe
#pragma unroll
                    for (int e = 0; e < 4; ++e) o2[e] = add2(o2[e], pf[e]);
                    ov = f32x2_to_bf16x8(o2);
                    if (moments) {
                        const uint32_t w[4] = {ov.x, ov.y, ov.z, ov.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xffff0000u);
                            m1[j] += lo + hi;
                            m2[j] = fmaf(hi, hi, fmaf(lo, lo, m2[j]));
                        }
                    }
                }
                *reinterpret_cast<uint4*>(y + orow[j] * ldy + lane * 8) = ov;
            }
        }
        if (EMBED && moments) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int j = 0; j < R; ++j) {
                    m1[j] += __shfl_xor_sync(0xffffffffu, m1[j], o);
                    m2[j] += __shfl_xor_sync(0xffffffffu, m2[j], o);
                }
#pragma unroll
            for (int j = 0; j < R; ++j)
                if (lane == 0 && r0 + j < rows) {
                    const unsigned rr = (unsigned)(r0 + j), b = rr / (unsigned)Np, n = rr - b * (unsigned)Np;
                    moments[(long long)b * (Np + 1) + 1 + n] = make_float2(m1[j], m2[j]);
                }
        }
    }
    if (EMBED) {
        // class-token rows: cls + pe[0], one warp per image
        const long long gw = blockIdx.x * wpb + (threadIdx.x >> 5), nw = (long long)gridDim.x * wpb;
        for (long long b = gw; b < cls_rows; b += nw) {
            float s1 = 0.f, s2 = 0.f;
            if (act) {
                f32x2 c2[4], p2[4];
                bf16x8_to_f32x2(*reinterpret_cast<const uint4*>(cls + lane * 8), c2);
                bf16x8_to_f32x2(*reinterpret_cast<const uint4*>(pe + lane * 8), p2);
#pragma unroll
                for (int e = 0; e < 4; ++e) c2[e] = add2(c2[e], p2[e]);
                const uint4 ov = f32x2_to_bf16x8(c2);
                *reinterpret_cast<uint4*>(y + b * (Np + 1) * ldy + lane * 8) = ov;
                const uint32_t w[4] = {ov.x, ov.y, ov.z, ov.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xffff0000u);
                    s1 += lo + hi;
                    s2 = fmaf(hi, hi, fmaf(lo, lo, s2));
                }
            }
            if (moments) {
                s1 = warp_sum(s1);
                s2 = warp_sum(s2);
                if (lane == 0) moments[b * (Np + 1)] = make_float2(s1, s2);
            }
        }
    }
}

// rows (b, py, px) x columns (c, i, j) <- img[b, c, py*P + i, px*P + j]: the unfold that
// turns Conv2d(kernel = stride = P) into a GEMM with the (D, C*P*P) weight view.  VT is an
// unsigned integer type carrying VE = sizeof(VT) / sizeof(T) contiguous elements of a patch row.
template <typename T, typename VT>
__global__ void __launch_bounds__(256) patchify_kernel(const T* __restrict__ img, T* __restrict__ out, int C, int Hh,
                                                       int Ww, int P) {
    // One CTA per (image, row of patches): C * P image rows of Ww elements, read in image order
    // (whole rows, coalesced) and stored as the P-element runs of the patches' rows.  The index
    // arithmetic is 32-bit inside the strip; four vectors per thread are in flight.
    constexpr int V = sizeof(VT) / sizeof(T);
    constexpr int U = 4;
    const int Hp = Hh / P, Wp = Ww / P;
    const int b = blockIdx.x / Hp, py = blockIdx.x - b * Hp;
    const int vrow = Ww / V, vpp = P / V;            // vectors per image row / per patch row
    const int n = C * P * vrow;
    const long long cpp = (long long)C * P * P;
    const T* src0 = img + ((long long)b * C * Hh + (long long)py * P) * Ww;
    T* dst0 = out + (long long)blockIdx.x * Wp * cpp;
    for (int e0 = threadIdx.x; e0 < n; e0 += 256 * U) {
        VT v[U];
        int r[U], xv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int e = e0 + u * 256;
            if (e < n) {
                r[u] = e / vrow;                     // c * P + i
                xv[u] = e - r[u] * vrow;
                const int c = r[u] / P, i = r[u] - c * P;
                v[u] = *reinterpret_cast<const VT*>(src0 + ((long long)c * Hh + i) * Ww + xv[u] * V);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (e0 + u * 256 < n) {
                const int px = xv[u] / vpp, jv = xv[u] - px * vpp;
                *reinterpret_cast<VT*>(dst0 + px * cpp + r[u] * P + jv * V) = v[u];
            }
        }
    }
}

// The same unfold for images that are still 8-bit (what an image decoder hands over): the
// loader's ToTensor + Normalize, out = (img / 255 - mean[c]) * inv_std[c], happens on the way.
// VEC pixels of one patch row per vector (8: one 8-byte load, 16 / 32 bytes stored).
template <typename T, int VEC>
__global__ void __launch_bounds__(256) patchify_u8_kernel(const uint8_t* __restrict__ img, const float* __restrict__ mean,
                                                          const float* __restrict__ inv_std, T* __restrict__ out, int C,
                                                          int Hh, int Ww, int P) {
    constexpr int U = VEC == 8 ? 4 : 8;
    const int Hp = Hh / P, Wp = Ww / P;
    const int b = blockIdx.x / Hp, py = blockIdx.x - b * Hp;
    const int vrow = Ww / VEC, vpp = P / VEC;
    const int n = C * P * vrow;
    const long long cpp = (long long)C * P * P;
    const uint8_t* src0 = img + ((long long)b * C * Hh + (long long)py * P) * Ww;
    T* dst0 = out + (long long)blockIdx.x * Wp * cpp;
    for (int e0 = threadIdx.x; e0 < n; e0 += 256 * U) {
        uint8_t raw[U][VEC];
        int r[U], xv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int e = e0 + u * 256;
            if (e < n) {
                r[u] = e / vrow;
                xv[u] = e - r[u] * vrow;
                const int c = r[u] / P, i = r[u] - c * P;
                const uint8_t* src = src0 + ((long long)c * Hh + i) * Ww + xv[u] * VEC;
                if (VEC == 8) *reinterpret_cast<uint2*>(raw[u]) = *reinterpret_cast<const uint2*>(src);
                else raw[u][0] = src[0];
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (e0 + u * 256 < n) {
                const int c = r[u] / P;
                const float m = mean[c], is = inv_std[c];
                const int px = xv[u] / vpp, jv = xv[u] - px * vpp;
                T* dst = dst0 + px * cpp + r[u] * P + jv * VEC;
                float f[VEC];
#pragma unroll
                for (int k = 0; k < VEC; ++k) f[k] = ((float)raw[u][k] * (1.0f / 255.0f) - m) * is;
                if (VEC == 8) {
                    store_vec<T>(dst, f);
                    if (Vec16<T>::N == 4) store_vec<T>(dst + 4, f + 4);
                } else {
                    dst[0] = from_f32<T>(f[0]);
                }
            }
        }
    }
}

template <typename T, typename VT>
void patchify_launch(const void* img, void* out, int B, int C, int Hh, int Ww, int P, cudaStream_t st) {
    patchify_kernel<T, VT><<<B * (Hh / P), 256, 0, st>>>(static_cast<const T*>(img), static_cast<T*>(out), C, Hh, Ww, P);
}

template <typename T>
int ln_dispatch(const void* x, long long ldx, const void* gamma, const void* beta, float eps, void* y, long long ldy,
                long long rows, int D, const void* pe, const void* cls, int Np, long long cls_rows, float* moments,
                cudaStream_t st) {
    constexpr int V = Vec16<T>::N;
    const int nvec = D / V;
    const int nv = (nvec + 31) / 32;
    long long total = rows + cls_rows;
    int blocks = (int)((total + 7) / 8);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    // the plain LayerNorm is a kernel of its own: the embedding tail's extra state costs it registers (64 -> 100 at
    // 768 channels) and with them half of its resident warps
#define CONVNN_LN(NVV)                                                                                          \
    do {                                                                                                        \
        if (pe)                                                                                                 \
            layernorm_kernel<T, NVV, true><<<blocks, 256, 0, st>>>(static_cast<const T*>(x), ldx,              \
                static_cast<const T*>(gamma), static_cast<const T*>(beta), eps, static_cast<T*>(y), ldy, rows, D, \
                static_cast<const T*>(pe), static_cast<const T*>(cls), Np, cls_rows, reinterpret_cast<float2*>(moments)); \
        else                                                                                                    \
            layernorm_kernel<T, NVV, false><<<blocks, 256, 0, st>>>(static_cast<const T*>(x), ldx,             \
                static_cast<const T*>(gamma), static_cast<const T*>(beta), eps, static_cast<T*>(y), ldy, rows, D, \
                nullptr, nullptr, 0, 0, nullptr);                                                               \
    } while (0)
    if (nv <= 1) CONVNN_LN(1);
    else if (nv <= 2) CONVNN_LN(2);
    else if (nv <= 4) CONVNN_LN(4);
    else if (nv <= 8) CONVNN_LN(8);
    else return set_error(CONVNN_E_UNSUPPORTED, "layernorm: D=%d is larger than this build supports", D);
#undef CONVNN_LN
    CONVNN_CHECK_LAUNCH("layernorm");
    return CONVNN_OK;
}

}  // namespace

int launch_layernorm(int dtype, const void* x, long long ldx, const void* gamma, const void* beta, float eps, void* y,
                     long long ldy, long long rows, int D, const void* pe, const void* cls, int Np,
                     long long cls_rows, float* moments, cudaStream_t st) {
    const int V = dtype == CONVNN_F32 ? 4 : 8;
    if (D % V != 0 || ldx % V != 0 || ldy % V != 0 || !aligned16(x) || !aligned16(y) || !aligned16(gamma) ||
        !aligned16(beta) || (pe && (!aligned16(pe) || !aligned16(cls))))
        return set_error(CONVNN_E_ALIGN, "layernorm: D, strides and pointers must be multiples of 16 bytes");
    if (moments && !pe) return set_error(CONVNN_E_INVALID, "layernorm: row moments come from the embedding tail only");
    if (dtype == CONVNN_BF16 && D <= 256 && (pe ? (cls != nullptr && rows < (1ll << 31) && Np > 0) : !moments)) {
        // Two 8-warp CTAs per SM (the kernel keeps 121 registers: four rows in flight and four
        // requested per warp), measured 9.6 us at 50 k rows of 192 channels against 11.0 us with
        // one row per step and four CTAs per SM; register-capped variants that spill are twice as slow.
        constexpr int R = 4, MINB = 2;
        int blocks = (int)((rows + 8 * R - 1) / (8 * R));
        if (blocks > 148 * MINB) blocks = 148 * MINB;
        if (blocks < 1) blocks = 1;
        const auto* xb = static_cast<const __nv_bfloat16*>(x);
        const auto *gb = static_cast<const __nv_bfloat16*>(gamma), *bb = static_cast<const __nv_bfloat16*>(beta);
        if (pe)
            layernorm_bf16_row256_kernel<R, MINB, true><<<blocks, 256, 0, st>>>(
                xb, ldx, gb, bb, eps, static_cast<__nv_bfloat16*>(y), ldy, rows, D, static_cast<const __nv_bfloat16*>(pe),
                static_cast<const __nv_bfloat16*>(cls), Np, cls_rows, reinterpret_cast<float2*>(moments));
        else
            layernorm_bf16_row256_kernel<R, MINB, false><<<blocks, 256, 0, st>>>(
                xb, ldx, gb, bb, eps, static_cast<__nv_bfloat16*>(y), ldy, rows, D, nullptr, nullptr, 0, 0, nullptr);
        CONVNN_CHECK_LAUNCH("layernorm_bf16_row256");
        return CONVNN_OK;
    }
    if (dtype == CONVNN_F32)
        return ln_dispatch<float>(x, ldx, gamma, beta, eps, y, ldy, rows, D, pe, cls, Np, cls_rows, moments, st);
    return ln_dispatch<__nv_bfloat16>(x, ldx, gamma, beta, eps, y, ldy, rows, D, pe, cls, Np, cls_rows, moments, st);
}

namespace {
// One warp per row: (sum, sum of squares) of a bfloat16 row, what the pre-norm fold of the GEMM
// needs from the producer of its rows.  Used once per forward (the rows the embedding wrote); every
// later set of moments comes out of a GEMM epilogue.
__global__ void __launch_bounds__(256) row_moments_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                          long long rows, int D, float2* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane * 8; c < D; c += 256) {
        const uint4 v = *reinterpret_cast<const uint4*>(x + r * ldx + c);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xffff0000u);
            s1 += lo + hi;
            s2 = fmaf(hi, hi, fmaf(lo, lo, s2));
        }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (lane == 0) out[r] = make_float2(s1, s2);
}

// One warp per output row n of a Linear that follows a LayerNorm: w_folded[n, k] = round(w[n, k] *
// gamma[k]) and the 16-element extra row [c_hi, c_hi, c_lo, c_lo, b_hi, b_hi, b_lo, b_lo, 0 x 8] with
// c = sum_k w_folded[n, k] (of the ROUNDED products, so that x W'^T - mean c cancels exactly) and
// b = sum_k w[n, k] beta[k] + bias[n], each as a bfloat16 hi + lo pair.
__global__ void __launch_bounds__(256) fold_layernorm_kernel(const __nv_bfloat16* __restrict__ w,
                                                             const __nv_bfloat16* __restrict__ bias,
                                                             const __nv_bfloat16* __restrict__ gamma,
                                                             const __nv_bfloat16* __restrict__ beta, int N, int K,
                                                             __nv_bfloat16* __restrict__ wf,
                                                             __nv_bfloat16* __restrict__ wx) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    float c = 0.f, b = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float wv = __bfloat162float(w[(long long)n * K + k]);
        const __nv_bfloat16 f = __float2bfloat16_rn(wv * __bfloat162float(gamma[k]));
        wf[(long long)n * K + k] = f;
        c += __bfloat162float(f);
        b = fmaf(wv, __bfloat162float(beta[k]), b);
    }
    c = warp_sum(c);
    b = warp_sum(b);
    if (lane == 0) {
        if (bias) b += __bfloat162float(bias[n]);
        const __nv_bfloat16 ch = __float2bfloat16_rn(c), bh = __float2bfloat16_rn(b);
        const __nv_bfloat16 cl = __float2bfloat16_rn(c - __bfloat162float(ch));
        const __nv_bfloat16 bl = __float2bfloat16_rn(b - __bfloat162float(bh));
        const __nv_bfloat16 z = __float2bfloat16_rn(0.f);
        const __nv_bfloat16 row[16] = {ch, ch, cl, cl, bh, bh, bl, bl, z, z, z, z, z, z, z, z};
#pragma unroll
        for (int j = 0; j < 16; ++j) wx[(long long)n * 16 + j] = row[j];
    }
}
}  // namespace

int launch_row_moments(const void* x, long long ldx, long long rows, int D, float* moments, cudaStream_t st) {
    if (D % 8 != 0 || ldx % 8 != 0 || !aligned16(x) || (reinterpret_cast<uintptr_t>(moments) & 7u))
        return set_error(CONVNN_E_ALIGN, "row_moments: D and ldx must be multiples of 8 elements, x 16-byte aligned");
    row_moments_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ldx, rows, D,
                                                                  reinterpret_cast<float2*>(moments));
    CONVNN_CHECK_LAUNCH("row_moments");
    return CONVNN_OK;
}

int launch_fold_layernorm(const void* w, const void* bias, const void* gamma, const void* beta, int N, int K,
                          void* w_folded, void* w_extra, cudaStream_t st) {
    fold_layernorm_kernel<<<(N + 7) / 8, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(bias),
        static_cast<const __nv_bfloat16*>(gamma), static_cast<const __nv_bfloat16*>(beta), N, K,
        static_cast<__nv_bfloat16*>(w_folded), static_cast<__nv_bfloat16*>(w_extra));
    CONVNN_CHECK_LAUNCH("fold_layernorm");
    return CONVNN_OK;
}

int launch_patchify_u8(int dtype, const uint8_t* img, const float* mean, const float* inv_std, void* out, int B, int C,
                       int Hh, int Ww, int P, cudaStream_t st) {
    if (Hh % P != 0 || Ww % P != 0) return set_error(CONVNN_E_INVALID, "patchify: image not divisible into patches");
    const bool v8 = P % 8 == 0 && Ww % 8 == 0 && (reinterpret_cast<uintptr_t>(img) & 7u) == 0 && aligned16(out);
#define CONVNN_PU8(T, V) patchify_u8_kernel<T, V><<<B * (Hh / P), 256, 0, st>>>(img, mean, inv_std, static_cast<T*>(out), C, Hh, Ww, P)
    if (dtype == CONVNN_F32) { if (v8) CONVNN_PU8(float, 8); else CONVNN_PU8(float, 1); }
    else { if (v8) CONVNN_PU8(__nv_bfloat16, 8); else CONVNN_PU8(__nv_bfloat16, 1); }
#undef CONVNN_PU8
    CONVNN_CHECK_LAUNCH("patchify_u8");
    return CONVNN_OK;
}

int launch_patchify(int dtype, const void* img, void* out, int B, int C, int Hh, int Ww, int P, cudaStream_t st) {
    if (Hh % P != 0 || Ww % P != 0) return set_error(CONVNN_E_INVALID, "patchify: image not divisible into patches");
    if (!aligned16(img) || !aligned16(out)) return set_error(CONVNN_E_ALIGN, "patchify: pointers must be 16-byte aligned");
    const int elt = dtype == CONVNN_F32 ? 4 : 2;
    int vb = 16;                                      // widest vector (bytes) that divides a patch row
    while (vb > elt && (P * elt) % vb != 0) vb >>= 1;
    if (dtype == CONVNN_F32) {
        if (vb == 16) patchify_launch<float, uint4>(img, out, B, C, Hh, Ww, P, st);
        else if (vb == 8) patchify_launch<float, uint2>(img, out, B, C, Hh, Ww, P, st);
        else patchify_launch<float, uint32_t>(img, out, B, C, Hh, Ww, P, st);
    } else {
        if (vb == 16) patchify_launch<__nv_bfloat16, uint4>(img, out, B, C, Hh, Ww, P, st);
        else if (vb == 8) patchify_launch<__nv_bfloat16, uint2>(img, out, B, C, Hh, Ww, P, st);
        else if (vb == 4) patchify_launch<__nv_bfloat16, uint32_t>(img, out, B, C, Hh, Ww, P, st);
        else patchify_launch<__nv_bfloat16, uint16_t>(img, out, B, C, Hh, Ww, P, st);
    }
    CONVNN_CHECK_LAUNCH("patchify");
    return CONVNN_OK;
}

}  // namespace convnn
