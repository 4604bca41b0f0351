// Softmax attention  o = softmax(q k^T / sqrt(d_k)) v  per (batch, head): the other half of the
// reference's MultiHeadBranchingAttention (MultiHeadAttention.forward, layers.py:105-130).
//
// bfloat16, up to 256 tokens, d_k a multiple of 16 up to 128 -- the tensor-core kernel.  A work
// unit is 128 query rows of one (batch, head); the whole key range is one MMA tile:
//   warp 0     TMA producer: Q rows (128 x d_k) and K rows (BN x d_k) as K-major swizzled chunks,
//              V rows (BN x d_k) token-major.
//   warp 1     MMA issuer.  MMA 1: S = Q K^T (M = 128, N = BN = tokens rounded up to 16) into
//              TMEM.  MMA 2: O = P V with P (bfloat16, written by the softmax warps) as the
//              K-major A operand and V^T as the K-major B operand; O lands in the first d_k
//              columns of the same accumulator once every row of S has been consumed.
//   warps 2-5  a thread owns one query row (its TMEM lane): row maximum, p = exp2((s - max) *
//              log2(e)/sqrt(d_k)), row sum; p goes to shared memory in the 128-byte-swizzled
//              operand layout.  Before that the four warps transpose V (token-major, as the
//              projection stores it) into the K-major V^T chunks MMA 2 needs.  Finally O / sum is
//              read back from TMEM, rounded and stored.
// P and the Q / K chunks share one shared-memory region (Q and K are dead once S is complete), so two
// CTAs fit on an SM at ViT shapes and cover each other's serial phases.
// Every mbarrier wait is bounded; on expiry the CTA latches a code and drains.
//
// Anything else (float32, longer sequences, other head widths) takes a plain SIMT kernel, one warp
// per query row.
#include <math_constants.h>

#include "common.cuh"
#include "sm100.cuh"
#include "f32x2.cuh"

namespace convnn {

__device__ int g_attention_status = 0;

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int NTHREADS = 192;      // TMA warp, MMA warp, 4 softmax warps
constexpr int CW = 16;

struct AttnParams {
    __nv_bfloat16* o;              // (B, T, H * dk)
    int T, H, dk, D;
    int KCH, KC;                   // channels per chunk / chunks of the Q K^T reduction
    int BN, BNpad;                 // key columns of the score tile, TMEM columns
    int NKC2;                      // 64-token chunks of the P V reduction
    int n_row_tiles, n_units;
    uint32_t p_region_bytes;       // shared by P and the Q / K chunks
    float scale_log2;              // log2(e) / sqrt(dk)
};

__device__ __forceinline__ void fail(volatile int* abort_flag, int code) {
    *abort_flag = 1;
    atomicCAS(&g_attention_status, 0, code);
}

__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&r)[CW]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
                 : "memory");
}

__global__ void __launch_bounds__(NTHREADS, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t pitch = p.KCH * 2;
    const uint32_t a_bytes = BM * pitch, b_bytes = p.BN * pitch;
    const uint32_t v_bytes = (uint32_t)p.BN * p.dk * 2;
    const uint32_t vt_chunk = (uint32_t)p.dk * 128;            // one V^T chunk: d_k rows of 64 tokens
    uint8_t* sP = smem;                                        // [NKC2][128 rows x 128 B]; aliases sQ | sK
    uint8_t* sQ = smem;                                        // [KC][128 x pitch]
    uint8_t* sK = smem + p.KC * a_bytes;                       // [KC][BN x pitch]
    uint8_t* sVt = smem + p.p_region_bytes;                    // [NKC2][dk rows x 128 B]
    uint8_t* sV = sVt + p.NKC2 * vt_chunk;                     // [BN][dk] token-major
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + ((v_bytes + 15) & ~15u));
    uint64_t* qk_full = bars;
    uint64_t* v_full = bars + 1;
    uint64_t* v_empty = bars + 2;
    uint64_t* s_full = bars + 3;
    uint64_t* p_ready = bars + 4;
    uint64_t* o_full = bars + 5;
    uint64_t* t_empty = bars + 6;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ncols = (uint32_t)p.BNpad;

    if (threadIdx.x == 0) {
        mbar_init(qk_full, 1);
        mbar_init(v_full, 1);
        mbar_init(v_empty, 4);
        mbar_init(s_full, 1);
        mbar_init(p_ready, 4);
        mbar_init(o_full, 1);
        mbar_init(t_empty, 4);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, ncols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < p.n_units && ok; unit += gridDim.x, ++it) {
                const uint32_t ph = it & 1u;
                const int bh = unit / p.n_row_tiles, rt = unit - bh * p.n_row_tiles;
                const int b = bh / p.H, h = bh - b * p.H;
                // Q / K land where the previous unit's P was: MMA 2 must have finished reading it
                if (it > 0 && !mbar_wait(o_full, ph ^ 1u, abort_flag)) { fail(abort_flag, 61); ok = false; break; }
                mbar_expect_tx(qk_full, p.KC * (a_bytes + b_bytes));
                for (int kc = 0; kc < p.KC; ++kc) {
                    tma_load_4d(sQ + kc * a_bytes, &tmQ, qk_full, kc * p.KCH, h, rt * BM, b);
                    tma_load_4d(sK + kc * b_bytes, &tmK, qk_full, kc * p.KCH, h, 0, b);
                }
                if (!mbar_wait(v_empty, ph ^ 1u, abort_flag)) { fail(abort_flag, 62); ok = false; break; }
                mbar_expect_tx(v_full, v_bytes);
                tma_load_4d(sV, &tmV, v_full, 0, h, 0, b);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc1 = make_idesc_bf16_f32(BM, p.BN);
            const uint32_t idesc2 = make_idesc_bf16_f32(BM, p.dk);
            const uint64_t dhi = kmajor_desc_hi(pitch), dhi128 = kmajor_desc_hi(128);
            const int nk16 = p.KCH / 16;
            const uint32_t sQ0 = smem_u32(sQ), sK0 = smem_u32(sK), sP0 = smem_u32(sP), sVt0 = smem_u32(sVt);
            uint32_t it = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < p.n_units && ok; unit += gridDim.x, ++it) {
                const uint32_t ph = it & 1u;
                if (!mbar_wait(t_empty, ph ^ 1u, abort_flag)) { fail(abort_flag, 63); ok = false; break; }
                if (!mbar_wait(qk_full, ph, abort_flag)) { fail(abort_flag, 64); ok = false; break; }
                tc_fence_after_sync();
                for (int kc = 0; kc < p.KC; ++kc) {
                    const uint64_t ad = dhi | (uint64_t)(((sQ0 + kc * a_bytes) & 0x3FFFFu) >> 4);
                    const uint64_t bd = dhi | (uint64_t)(((sK0 + kc * b_bytes) & 0x3FFFFu) >> 4);
                    mma_chunk(tmem_base, ad, bd, idesc1, nk16, kc != 0);
                }
                mma_commit(s_full);
                if (!mbar_wait(p_ready, ph, abort_flag)) { fail(abort_flag, 65); ok = false; break; }
                tc_fence_after_sync();
                uint32_t acc = 0;
                for (int kc2 = 0; kc2 < p.NKC2; ++kc2) {
                    const uint64_t ad = dhi128 | (uint64_t)(((sP0 + kc2 * 16384u) & 0x3FFFFu) >> 4);
                    const uint64_t bd = dhi128 | (uint64_t)(((sVt0 + kc2 * vt_chunk) & 0x3FFFFu) >> 4);
                    for (int k16 = 0; k16 < 4; ++k16) {
                        if (kc2 * 64 + k16 * 16 >= p.BN) break;
                        mma_bf16_ss(tmem_base, ad + 2 * k16, bd + 2 * k16, idesc2, acc);
                        acc = 1;
                    }
                }
                mma_commit(o_full);
            }
        }
    } else {
        const int lq = warp & 3;
        const int r = lq * 32 + lane;            // query row within the tile = TMEM lane
        const int st = threadIdx.x - 64;         // 0 .. 127 among the softmax threads
        const uint32_t taddr = tmem_base + ((uint32_t)(lq * 32) << 16);
        const uint32_t sP_row = smem_u32(sP) + r * 128;
        uint32_t it = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < p.n_units && ok; unit += gridDim.x, ++it) {
            const uint32_t ph = it & 1u;
            const int bh = unit / p.n_row_tiles, rt = unit - bh * p.n_row_tiles;
            const int b = bh / p.H, h = bh - b * p.H;
            const int row = rt * BM + r;
            // ---- V (token-major) -> V^T chunks: [channel][64 tokens], 16-byte segments swizzled ------
            ok = mbar_wait(v_full, ph, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) fail(abort_flag, 66); break; }
            {
                // item i = (segment of 8 tokens sg, channel c), i = sg * dk + c, visited with stride 128:
                // (sg, c) advance by (128 / dk, 128 % dk) with a carry, no division in the loop
                const int nseg = p.BN / 8;
                const int dsg = 128 / p.dk, dc = 128 - dsg * p.dk;
                int sg = st / p.dk, c = st - sg * p.dk;
                const unsigned short* v16 = reinterpret_cast<const unsigned short*>(sV);
                while (sg < nseg) {
                    const int t0 = sg * 8;
                    const unsigned short* src = v16 + t0 * p.dk + c;
                    uint32_t w[4];
#pragma unroll
                    for (int e2 = 0; e2 < 4; ++e2) {
                        const uint32_t lo = src[(2 * e2) * p.dk], hi = src[(2 * e2 + 1) * p.dk];
                        w[e2] = lo | (hi << 16);
                    }
                    const int kc2 = t0 >> 6, seg = (t0 & 63) >> 3;
                    uint8_t* dst = sVt + kc2 * vt_chunk + c * 128 + ((seg ^ (c & 7)) << 4);
                    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                    sg += dsg;
                    c += dc;
                    if (c >= p.dk) { c -= p.dk; ++sg; }
                }
            }
            fence_proxy_async();                 // the transposed tile is read by the MMA (async proxy)
            __syncwarp();
            if (lane == 0) mbar_arrive(v_empty);
            // ---- scores -> probabilities -----------------------------------------------------------
            ok = mbar_wait(s_full, ph, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) fail(abort_flag, 67); break; }
            tc_fence_after_sync();
            // row maximum; only the last chunk can hold columns past the sequence
            float m = -CUDART_INF_F;
#pragma unroll 1
            for (int c = 0; c < p.BN; c += CW) {
                uint32_t acc[CW];
                tmem_ld_x16(taddr + c, acc);
                tmem_ld_wait_on(acc);
                if (c + CW > p.T) {
#pragma unroll
                    for (int j = 0; j < CW; ++j)
                        if (c + j >= p.T) acc[j] = 0xff800000u;          // -inf
                }
                float m4[4];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    m4[q4] = fmaxf(fmaxf(__uint_as_float(acc[4 * q4]), __uint_as_float(acc[4 * q4 + 1])),
                                   fmaxf(__uint_as_float(acc[4 * q4 + 2]), __uint_as_float(acc[4 * q4 + 3])));
                m = fmaxf(m, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
            }
            // p = 2^(s * scale - m * scale): one fused multiply-add and one hardware exp2 per score
            const float ms = -m * p.scale_log2;
            f32x2 sum2 = 0ull;
#pragma unroll 1
            for (int c = 0; c < p.BN; c += CW) {
                uint32_t acc[CW];
                tmem_ld_x16(taddr + c, acc);
                tmem_ld_wait_on(acc);
                if (c + CW > p.T) {
#pragma unroll
                    for (int j = 0; j < CW; ++j)
                        if (c + j >= p.T) acc[j] = 0xff800000u;          // -inf: probability 0
                }
                uint32_t pk[8];
#pragma unroll
                for (int j2 = 0; j2 < 8; ++j2) {
                    float p0, p1;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(fmaf(__uint_as_float(acc[2 * j2]), p.scale_log2, ms)));
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(fmaf(__uint_as_float(acc[2 * j2 + 1]), p.scale_log2, ms)));
                    sum2 = add2(sum2, pack2(p0, p1));
                    __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
                    pk[j2] = *reinterpret_cast<uint32_t*>(&hh);
                }
                const int kc2 = c >> 6, seg = (c & 63) >> 3;
                const uint32_t base = sP_row + kc2 * 16384u;
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + (((seg) ^ (r & 7)) << 4)), "r"(pk[0]),
                             "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + (((seg + 1) ^ (r & 7)) << 4)), "r"(pk[4]),
                             "r"(pk[5]), "r"(pk[6]), "r"(pk[7]) : "memory");
            }
            float sum_lo, sum_hi;
            unpack2(sum2, sum_lo, sum_hi);
            const float sum = sum_lo + sum_hi;
            fence_proxy_async();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready);
            // ---- O / sum ---------------------------------------------------------------------------------
            ok = mbar_wait(o_full, ph, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) fail(abort_flag, 68); break; }
            tc_fence_after_sync();
            const float inv = 1.0f / sum;
            __nv_bfloat16* orow = p.o + ((long long)b * p.T + row) * p.D + h * p.dk;
#pragma unroll 1
            for (int c = 0; c < p.dk; c += CW) {
                uint32_t acc[CW];
                tmem_ld_x16(taddr + c, acc);
                tmem_ld_wait_on(acc);
                uint32_t pk[8];
#pragma unroll
                for (int j2 = 0; j2 < 8; ++j2) {
                    __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(acc[2 * j2]) * inv,
                                                              __uint_as_float(acc[2 * j2 + 1]) * inv);
                    pk[j2] = *reinterpret_cast<uint32_t*>(&hh);
                }
                if (row < p.T) {
                    *reinterpret_cast<uint4*>(orow + c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    *reinterpret_cast<uint4*>(orow + c + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(t_empty);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, ncols);
    }
}

// One warp per query row; scores in shared memory.  float32 (and the fallback for shapes the
// tensor-core kernel does not take).
template <typename T>
__global__ void attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                      T* __restrict__ o, int Tn, int H, int dk, float scale) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    float* prob = sm + warp * (Tn + dk);
    float* qrow = prob + Tn;
    const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
    const long long D = (long long)H * dk;
    const T* kb = k + (long long)b * Tn * D + h * dk;
    const T* vb = v + (long long)b * Tn * D + h * dk;
    for (int row = blockIdx.x * nw + warp; row < Tn; row += gridDim.x * nw) {
        const T* qr = q + ((long long)b * Tn + row) * D + h * dk;
        for (int c = lane; c < dk; c += 32) qrow[c] = to_f32(qr[c]) * scale;
        __syncwarp();
        float m = -3.402823466e38f;
        for (int j = lane; j < Tn; j += 32) {
            const T* kr = kb + (long long)j * D;
            float s = 0.f;
            for (int c = 0; c < dk; ++c) s = fmaf(qrow[c], to_f32(kr[c]), s);
            prob[j] = s;
            m = fmaxf(m, s);
        }
        for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        float sum = 0.f;
        for (int j = lane; j < Tn; j += 32) {
            const float e = expf(prob[j] - m);
            prob[j] = e;
            sum += e;
        }
        for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        __syncwarp();
        const float inv = 1.0f / sum;
        T* orow = o + ((long long)b * Tn + row) * D + h * dk;
        for (int c = lane; c < dk; c += 32) {
            float acc = 0.f;
            for (int j = 0; j < Tn; ++j) acc = fmaf(prob[j], to_f32(vb[(long long)j * D + c]), acc);
            orow[c] = from_f32<T>(acc * inv);
        }
        __syncwarp();
    }
}

int pow2_at_least(int v, int lo) {
    int r = lo;
    while (r < v) r <<= 1;
    return r;
}

bool attention_tc_ok(int dtype, const void* q, const void* k, const void* v, const void* o, int Tn, int D, int H) {
    const int dk = D / H;
    return dtype == CONVNN_BF16 && !force_simt() && Tn <= 256 && dk % 16 == 0 && dk <= 128 && aligned16(q) &&
           aligned16(k) && aligned16(v) && aligned16(o);
}

int launch_attention_tc(const void* q, const void* k, const void* v, void* o, int B, int Tn, int D, int H,
                        cudaStream_t st) {
    AttnParams p{};
    p.o = static_cast<__nv_bfloat16*>(o);
    p.T = Tn; p.H = H; p.dk = D / H; p.D = D;
    p.KCH = p.dk % 64 == 0 ? 64 : (p.dk % 32 == 0 ? 32 : 16);
    p.KC = p.dk / p.KCH;
    p.BN = (Tn + 15) / 16 * 16;
    p.BNpad = pow2_at_least(p.BN > p.dk ? p.BN : p.dk, 32);
    p.NKC2 = (p.BN + 63) / 64;
    p.n_row_tiles = (Tn + BM - 1) / BM;
    p.n_units = B * H * p.n_row_tiles;
    p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)p.dk));
    const int pitch = p.KCH * 2;
    const size_t qk_bytes = (size_t)p.KC * (BM + p.BN) * pitch, pp_bytes = (size_t)p.NKC2 * 16384;
    p.p_region_bytes = (uint32_t)(((qk_bytes > pp_bytes ? qk_bytes : pp_bytes) + 1023) & ~(size_t)1023);
    const size_t smem = 1024 + p.p_region_bytes + (size_t)p.NKC2 * p.dk * 128 + (((size_t)p.BN * p.dk * 2 + 15) & ~(size_t)15) +
                        7 * 8 + 16;
    if (smem > 227 * 1024) return set_error(CONVNN_E_UNSUPPORTED, "attention_tc: shape needs %zu bytes of shared memory", smem);

    CUtensorMap tmQ, tmK, tmV;
    const uint64_t dims[4] = {(uint64_t)p.dk, (uint64_t)H, (uint64_t)Tn, (uint64_t)B};
    const uint64_t str[3] = {(uint64_t)p.dk * 2, (uint64_t)D * 2, (uint64_t)Tn * D * 2};
    const uint32_t boxQ[4] = {(uint32_t)p.KCH, 1, (uint32_t)BM, 1};
    const uint32_t boxK[4] = {(uint32_t)p.KCH, 1, (uint32_t)p.BN, 1};
    const uint32_t boxV[4] = {(uint32_t)p.dk, 1, (uint32_t)p.BN, 1};
    if (!encode_tensor_map_bf16(&tmQ, q, 4, dims, str, boxQ, pitch)) return CONVNN_E_CUDA;
    if (!encode_tensor_map_bf16(&tmK, k, 4, dims, str, boxK, pitch)) return CONVNN_E_CUDA;
    if (!encode_tensor_map_bf16(&tmV, v, 4, dims, str, boxV, 0)) return CONVNN_E_CUDA;

    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int per_sm = smem <= 113 * 1024 && p.BNpad <= 256 ? 2 : 1;
    const int ctas = sms * per_sm;
    const int grid = p.n_units < ctas ? p.n_units : ctas;
    auto kern = attention_tc_kernel;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    kern<<<grid, NTHREADS, smem, st>>>(tmQ, tmK, tmV, p);
    CONVNN_CHECK_LAUNCH("attention_tc");
    return CONVNN_OK;
}

template <typename T>
int launch_attention_simt_t(const void* q, const void* k, const void* v, void* o, int B, int Tn, int D, int H,
                            cudaStream_t st) {
    const int dk = D / H, nw = 4;
    const size_t smem = (size_t)nw * (Tn + dk) * sizeof(float);
    if (smem > 200 * 1024)
        return set_error(CONVNN_E_UNSUPPORTED, "softmax attention over %d tokens is outside this build", Tn);
    auto kern = attention_simt_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    int gx = (Tn + nw - 1) / nw;
    if (gx > 64) gx = 64;
    kern<<<dim3(gx, B * H), nw * 32, smem, st>>>(static_cast<const T*>(q), static_cast<const T*>(k),
                                                 static_cast<const T*>(v), static_cast<T*>(o), Tn, H, dk,
                                                 (float)(1.0 / sqrt((double)dk)));
    CONVNN_CHECK_LAUNCH("attention_simt");
    return CONVNN_OK;
}

}  // namespace

// q, k, v, o: (B, T, H, d_k) = (B*T, D) row-major in `dtype`.
int launch_attention(int dtype, const void* q, const void* k, const void* v, void* o, int B, int Tn, int D, int H,
                     cudaStream_t st) {
    if (attention_tc_ok(dtype, q, k, v, o, Tn, D, H)) return launch_attention_tc(q, k, v, o, B, Tn, D, H, st);
    if (dtype == CONVNN_F32) return launch_attention_simt_t<float>(q, k, v, o, B, Tn, D, H, st);
    return launch_attention_simt_t<__nv_bfloat16>(q, k, v, o, B, Tn, D, H, st);
}

int read_attention_status(int* out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_attention_status, sizeof(int));
    if (e != cudaSuccess) return set_error(CONVNN_E_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    *out = v;
    return CONVNN_OK;
}

}  // namespace convnn
