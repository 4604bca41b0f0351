// Shared host/device helpers of the convnn_b200 library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/convnn_b200.h"

namespace convnn {

// ---- error reporting -------------------------------------------------------------
int set_error(int status, const char* fmt, ...);
void clear_error();

void count_launch();

#define CONVNN_CHECK_LAUNCH(what)                                                    \
    do {                                                                             \
        ::convnn::count_launch();                                                    \
        cudaError_t e__ = cudaGetLastError();                                        \
        if (e__ != cudaSuccess)                                                      \
            return ::convnn::set_error(CONVNN_E_CUDA, "%s: %s", what, cudaGetErrorString(e__)); \
    } while (0)

// ---- descriptor-derived quantities -------------------------------------------------
struct Dims {
    int B, T, S, D, H, K, dk, C, Cp;   // C = input channels per head, Cp = stored channels
    int nsel;                          // neighbours picked from the candidates: K or K-1
    size_t elt;                        // bytes per element of dtype
};

// Validates the descriptor the way the reference would fail (or this build refuses)
// and fills Dims.  Returns CONVNN_OK or a negative status with last_error set.
int validate(const convnn_desc* d, Dims* out);

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr int kMaxK = 32;              // register-resident sorted list per row

// ---- dtype helpers -----------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- kernel launchers (one translation unit each) ------------------------------------
// A operand addressing of the SIMT GEMM.
enum AMode : int {
    A_ROWS = 0,       // A[m, kk] = a[m * lda + kk]
    A_TOKENS = 1,     // m = (b, r): token = cand ? cand[r] : r; a[(b*T + token) * lda + kk]
    A_HEAD_QUIRK = 2  // m = (b, t'), kk = h*dk + c': a[((b*H + h) * T) * dk + c' * T + t']
};
// C placement of the SIMT GEMM.
enum CMode : int {
    C_ROWS = 0,       // c[m * ldc + n]
    C_HEADS = 1       // n = h*dk + c: c[m * H*Cp + h*Cp + c]
};

struct GemmParams {
    const void* a;
    const void* w;        // (N, Kd) row-major: C = A * W^T
    const void* bias;     // (N) in dtype or nullptr
    void* c;
    const int32_t* cand;  // A_TOKENS only
    long long lda, ldc;
    int M, N, Kd;
    int a_mode, c_mode;
    int rows_per_batch;   // A_TOKENS: rows per batch item (T or S); A_HEAD_QUIRK: T
    int T, H, dk, Cp;     // geometry for A_TOKENS / A_HEAD_QUIRK / C_HEADS
    int gelu;             // apply exact GELU after bias
    const void* residual; // (M, N) with row stride ldr, added after rounding to dtype; or nullptr
    long long ldr;
};

int launch_gemm_simt(int dtype, const GemmParams& p, cudaStream_t st);

int launch_head_fill_and_stats(const convnn_desc* d, const Dims& dm, void* t, int rows, float* stat,
                               cudaStream_t st);
int launch_sim_topk_simt_f32(const convnn_desc* d, const Dims& dm, const void* q, const void* k,
                             const float* qstat, const float* kstat, const int32_t* cand,
                             int32_t* idx, float* val, cudaStream_t st);
int launch_sim_topk_simt_bf16(const convnn_desc* d, const Dims& dm, const void* q, const void* k,
                              const float* qstat, const float* kstat, const int32_t* cand,
                              int32_t* idx, float* val, cudaStream_t st);
bool sim_topk_tc_supported(const convnn_desc* d, const Dims& dm, const void* q, const void* k);
int launch_sim_topk_tc(const convnn_desc* d, const Dims& dm, const void* q, const void* k, const float* qstat,
                       const float* kstat, const int32_t* cand, int32_t* idx, float* val, cudaStream_t st);
bool sim_topk_tc2_wanted(const convnn_desc* d, const Dims& dm);
int launch_sim_topk_tc2(const convnn_desc* d, const Dims& dm, const void* q, const void* k, const float* qstat,
                        const float* kstat, const int32_t* cand, int32_t* idx, float* val, cudaStream_t st);
int read_sim_topk_status(int* out);
int read_sim_topk2_status(int* out);
int try_launch_gather_conv_dw_stream(const convnn_desc* d, const Dims& dm, const void* v, const int32_t* idx,
                                     const float* val, const void* w_conv, void* o, cudaStream_t st);
int read_dw_stream_status(int* out);
int read_gemm_tc_status(int* out);
// bfloat16 tensor-core GEMM C = A W^T (+bias, +GELU); `parts` outputs share M and split N evenly.
bool gemm_tc_supported(const void* a, long long lda, const void* w, int Kd, int N, int parts, const void* const* c,
                       long long ldc);
struct GemmTcOpts {
    const void* bias = nullptr;       // (N) bf16
    const void* residual = nullptr;   // (M, N) bf16 with row stride ldr, added after rounding
    long long ldr = 0;
    int gelu = 0;
    float* stat[3] = {nullptr, nullptr, nullptr};   // per part: fused per-(row, head) statistic
    int stat_mode = 0, dk = 0, heads = 1, rows_per_batch = 1;
    // heads wider than a tile: room for gemm_tc_stat_pieces() x M x heads floats per part with a
    // statistic (the tiles' partial sums, combined by a second small kernel)
    float* stat_scratch = nullptr;
    // Pre-norm fold: `a` holds the rows BEFORE their LayerNorm, `w` is W * diag(gamma) and ln_wextra
    // the (N, 16) extra rows of fold_layernorm(); ln_moments = [ln_planes][gemm_tc_moment_stride(M)][2]
    // partial (sum, sum of squares) of the rows of a.  No bias / skip connection (the bias is folded).
    const float* ln_moments = nullptr;
    int ln_planes = 0;
    float ln_eps = 0.f;
    const void* ln_wextra = nullptr;
    // Row moments of the stored rows, [gemm_tc_moment_planes(N)][gemm_tc_moment_stride(M)][2]; needs a skip connection.
    float* moments_out = nullptr;
};
bool gemm_tc_prenorm_supported(int N, int Kd, int parts, bool has_stat, bool gelu);
int gemm_tc_moment_planes(int N);
long long gemm_tc_moment_stride(long long M);   // entries between the planes of a moments buffer
bool gemm_tc_can_fuse_stats(int part_cols, int dk);
// Column tiles a head is spread over when the statistic is fused: 1 = a tile holds whole heads,
// m >= 2 = each head spans m tiles (partial sums + combine), 0 = cannot be fused.
int gemm_tc_stat_pieces(int part_cols, int dk);
int launch_gemm_tc(const void* a, long long lda, const void* w, int M, int N, int Kd, int parts, void* const* c,
                   long long ldc, const GemmTcOpts& o, cudaStream_t st);
int launch_layernorm(int dtype, const void* x, long long ldx, const void* gamma, const void* beta, float eps, void* y,
                     long long ldy, long long rows, int D, const void* pe, const void* cls, int Np,
                     long long cls_rows, float* moments, cudaStream_t st);
// The encoder's MLP block (norm2 folded, GELU, both Linear layers, skip connection) as one kernel.
bool mlp_tc_supported(int D, int DM, int planes);
int mlp_tc_moment_planes();
int launch_mlp_tc(const void* x, long long ldx, const float* moments, int planes, float eps, const void* w1_folded,
                  const void* w1_extra, const void* w2, const void* b2, void* out, long long ldo, int M, int D, int DM,
                  float* moments_out, const void* w_o, const void* resid, long long ldr, cudaStream_t st);
int read_mlp_tc_status(int* out);
int launch_row_moments(const void* x, long long ldx, long long rows, int D, float* moments, cudaStream_t st);
int launch_fold_layernorm(const void* w, const void* bias, const void* gamma, const void* beta, int N, int K,
                          void* w_folded, void* w_extra, cudaStream_t st);
int launch_patchify(int dtype, const void* img, void* out, int B, int C, int Hh, int Ww, int P, cudaStream_t st);
int launch_patchify_u8(int dtype, const uint8_t* img, const float* mean, const float* inv_std, void* out, int B, int C,
                       int Hh, int Ww, int P, cudaStream_t st);
int launch_gather_rows(int dtype, const void* x, long long ldx, const int32_t* cand, void* xq, int B, int Tn, int S,
                       int D, cudaStream_t st);
int launch_merge_heads(int dtype, const void* o, void* y, int B, int Tn, int H, int dk, cudaStream_t st);
int launch_attention(int dtype, const void* q, const void* k, const void* v, void* o, int B, int Tn, int D, int H,
                     cudaStream_t st);
int read_attention_status(int* out);
int launch_conv1d_heads(int dtype, const void* y, const void* w, const void* bias, void* o, void* unfold, int B,
                        int Tn, int H, int dk, int ks, cudaStream_t st);
bool force_simt();   // debugging switch: environment variable CONVNN_B200_FORCE_SIMT=1
int launch_gather_conv_simt(const convnn_desc* d, const Dims& dm, const void* v, const int32_t* idx,
                            const float* val, const void* w_conv, const void* w_pw, void* o, void* scratch,
                            cudaStream_t st);

}  // namespace convnn
