/*
 * convnn_b200 — C ABI of the B200 (sm_100a) ConvNN-Attention forward path.
 *
 * The reference is eager PyTorch and has no native interface; each entry point below
 * replaces a span of `MultiHeadConvNNAttention.forward` (reference layers.py:261-321)
 * and is what a Python/ctypes (or C++) binding of that span binds to.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer owned by the caller.  The library allocates
 *     nothing, frees nothing and keeps no caller pointer after the call returns.
 *   - All work is enqueued on `stream` (a cudaStream_t passed as void*); no call
 *     synchronises the host, except convnn_b200_device_status().  The stage calls, the
 *     workspace forward and the encoder ops are re-entrant: host threads may call them
 *     at the same time on different streams with different buffers.
 *   - Process-wide state, all of it: a launch counter; per-device flags remembering that
 *     a device was checked to be sm_100; one device-side error latch per tensor-core
 *     kernel family (read by convnn_b200_device_status(), never cleared, first code
 *     wins); and, for convnn_b200_forward_noalloc() only, one fixed device array per GPU
 *     with its cached address (those calls are NOT re-entrant on one device: see there).
 *     cudaDeviceReset() invalidates the cached address and the latches' device copies;
 *     a process that resets a device must not call the library on it afterwards.
 *   - Return value: CONVNN_OK or a negative convnn_status; a human-readable reason for
 *     the last failure on the calling thread is in convnn_b200_last_error().
 *   - `dtype` is the storage type of activations and weights (float32 or bfloat16);
 *     accumulation, similarity values, softmax and statistics are always float32.
 *
 * Layouts (row-major, innermost last)
 *   x        (B, T, D)       row stride `ldx` elements (>= D; lets a caller pass the
 *                            channel slice x[:, :, :D] of a wider tensor, layers.py:648)
 *   cand     (S) int32       candidate token indices of the sampled modes, else NULL
 *   q        (B, S, H, Cp)   Cp = convnn_b200_head_channels(): d_k, or with the
 *   k, v     (B, T, H, Cp)   coordinate channel d_k+1 rounded up to a multiple of 8
 *                            (channel d_k holds the coordinate, the rest are zero)
 *   qstat    (B, H, S) f32   cosine: 1/max(|q|,1e-12); euclidean: |q|^2; matmul: unused
 *   kstat    (B, H, T) f32   same for k
 *   idx, val (B, H, T, K)    int32 neighbour token indices / float32 pre-softmax
 *                            values, best first (sampled modes: slot 0 = self, value 1)
 *   o        (B, H, T, d_k)  per-head Conv1d output, token-major
 *   out      (B, T, D)       row stride `ldo` elements
 *
 * Packed weights (all in `dtype`; the Python module packs and caches them)
 *   w_qkv    (3, D, D)       [W_k; W_v; W_q], each (out, in) as nn.Linear stores it
 *   w_conv   depthwise / depthwise-separable stage 0: (K, C) tap-major, from (C, 1, K)
 *            standard: (d_k, K, C) from (d_k, C, K), i.e. a (d_k, K*C) matrix
 *   w_pw     depthwise-separable stage 1: (d_k, C) from (d_k, C, 1); else NULL
 *   w_o      (D, D) (out, in)
 */
#ifndef CONVNN_B200_H
#define CONVNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CONVNN_B200_ABI_VERSION 1

enum convnn_dtype { CONVNN_F32 = 0, CONVNN_BF16 = 1 };
enum convnn_metric { CONVNN_COSINE = 0, CONVNN_MATMUL = 1, CONVNN_EUCLIDEAN = 2 };
enum convnn_conv { CONVNN_DEPTHWISE = 0, CONVNN_STANDARD = 1, CONVNN_DEPTHWISE_SEPARABLE = 2 };

enum convnn_status {
    CONVNN_OK = 0,
    CONVNN_E_INVALID = -1,      /* argument out of range / inconsistent descriptor     */
    CONVNN_E_UNSUPPORTED = -2,  /* legal in the reference but outside this build        */
    CONVNN_E_NULL = -3,         /* a required pointer is NULL                            */
    CONVNN_E_ALIGN = -4,        /* pointer or leading dimension not 16-byte aligned      */
    CONVNN_E_WORKSPACE = -5,    /* workspace smaller than convnn_b200_workspace_bytes()  */
    CONVNN_E_CUDA = -6,         /* launch failed (cudaGetLastError)                      */
    CONVNN_E_DEVICE = -7,       /* current device is not sm_100                          */
    CONVNN_E_TOPK_RANGE = -8,   /* K exceeds the candidate count (torch.topk would raise)*/
    CONVNN_E_SEQ_LENGTH = -9    /* H > 1 and T != seq_length (reference reshape raises)  */
};

/* Problem descriptor: the constructor arguments of the reference layer
 * (layers.py:133-146) plus the shapes of this call. */
typedef struct convnn_desc {
    int32_t B;           /* batch                                                        */
    int32_t T;           /* tokens per sequence                                          */
    int32_t S;           /* candidates: T for sampling 'all', len(cand) otherwise        */
    int32_t D;           /* d_hidden = H * d_k                                           */
    int32_t H;           /* num_heads                                                    */
    int32_t K;           /* neighbours per token (Conv1d kernel size and stride)         */
    int32_t dtype;       /* convnn_dtype                                                 */
    int32_t metric;      /* convnn_metric (magnitude_type)                               */
    int32_t sampled;     /* 0: sampling_type 'all'; 1: 'random' / 'spatial' via cand[]   */
    int32_t conv_type;   /* convnn_conv                                                  */
    int32_t softmax;     /* softmax_topk_val                                             */
    int32_t coord;       /* coordinate_encoding                                          */
    int32_t seq_length;  /* ctor seq_length; H > 1 requires T == seq_length              */
    int32_t reserved;    /* must be 0                                                    */
} convnn_desc;

/* No reference counterpart: ABI guard for bindings. */
int convnn_b200_abi_version(void);
const char* convnn_b200_status_string(int status);
const char* convnn_b200_last_error(void);
/* No reference counterpart: number of kernels this library has launched in the process so
 * far (a monotonically increasing statistic; the only process-wide state it keeps). */
uint64_t convnn_b200_launch_count(void);

/* No reference counterpart: reads the device-side error latch (synchronises the device).
 * 0 = no kernel gave up; otherwise the code of the first bounded wait that expired inside
 * a tensor-core kernel (similarity: 1 producer, 2/3 MMA issuer, 4 epilogue; GEMM: 11-16; pair
 * similarity: 21-26; streaming depthwise conv: 31).  A wait gives up after 250 ms.  Results of
 * a call that latched a code are undefined. */
int convnn_b200_device_status(int* code);

/* No reference counterpart: exercises the bounded wait every tensor-core kernel of this
 * library uses, without any copy or MMA in flight.  One thread of a one-CTA kernel waits on a
 * barrier that nothing ever completes, for at most `budget_us` microseconds (1 .. 100000),
 * then writes 41 to *status_dev (0 if the wait had, impossibly, succeeded) and the time it
 * waited, in nanoseconds, to *waited_ns_dev (both DEVICE pointers), and returns.  The kernel
 * neither traps nor touches the error latch; the context stays usable. */
int convnn_b200_selftest_wait_timeout(uint32_t budget_us, int* status_dev, uint64_t* waited_ns_dev,
                                      void* stream);

/* Channels per head as stored in q/k/v (Cp above). Negative status on a bad descriptor. */
int convnn_b200_head_channels(const convnn_desc* d);

/* Bytes of scratch convnn_b200_forward() needs for this descriptor (q, k, v, qstat,
 * kstat, idx, val, o, stage scratch).  Replaces the temporaries the reference allocates implicitly
 * along layers.py:264-313. 0 on a bad descriptor. */
size_t convnn_b200_workspace_bytes(const convnn_desc* d);

/* Bytes of the optional `scratch` argument of the stages: room for the gathered candidate
 * rows (B, S, D) and, behind them, the partial row statistics of heads wider than a GEMM
 * tile, the GEMM operand of the standard (B, H, T, K*C) / separable (B, H, T, C)
 * conv, and the head-merged activations (B, T, D).  With scratch == NULL the stages still
 * work but leave the tensor cores for the cases that need it (sampled queries; standard and
 * separable conv; H > 1 output projection).  No reference counterpart. */
size_t convnn_b200_stage_scratch_bytes(const convnn_desc* d);

/* K/V/Q projections, head split and (optional) coordinate channel, plus the per-row
 * statistics the similarity needs.  Replaces layers.py:264-265, 269-270, 274-276,
 * 285-287, 298-300 and the norm terms of layers.py:328-329, 337-338. */
int convnn_b200_qkv_proj(const convnn_desc* d, const void* x, int64_t ldx, const void* w_qkv,
                         const int32_t* cand, void* q, void* k, void* v,
                         float* qstat, float* kstat, void* scratch, void* stream);

/* Similarity (cosine / matmul / euclidean), sampled-mode self mask and sorted top-K
 * without materialising the T x S matrix.  Replaces layers.py:278/289/302 (323-340),
 * 291-292, 304-305 and the torch.topk + index mapping of layers.py:344, 363-376, 391,
 * 410-423.  Exact ties keep the lower candidate column. */
int convnn_b200_sim_topk(const convnn_desc* d, const void* q, const void* k,
                         const float* qstat, const float* kstat, const int32_t* cand,
                         int32_t* idx, float* val, void* stream);

/* Softmax (or raw / reciprocal) weights over the K values, neighbour gather of V and the
 * K-tap stride-K Conv1d.  Replaces layers.py:345-357, 378-386, 394-405, 425-436 and
 * self.conv (layers.py:313, 187-228). */
int convnn_b200_gather_conv(const convnn_desc* d, const void* v, const int32_t* idx,
                            const float* val, const void* w_conv, const void* w_pw,
                            void* o, void* scratch, void* stream);

/* Head merge (including the reference's flat reinterpretation for H > 1) and the W_o
 * projection.  Replaces layers.py:317, 320 (247-259).  With `residual` != NULL (rows of D
 * elements, stride ldr) the caller's skip connection `x + attention(...)` (vit.py:264) is
 * folded into the store: out = residual + round(proj). */
int convnn_b200_out_proj(const convnn_desc* d, const void* o, const void* w_o,
                         const void* residual, int64_t ldr,
                         void* out, int64_t ldo, void* scratch, void* stream);

/* The whole layer forward: the four calls above chained on `stream` with their
 * intermediates placed in `workspace`.  Replaces MultiHeadConvNNAttention.forward
 * (layers.py:261-321), eval mode. */
int convnn_b200_forward(const convnn_desc* d, const void* x, int64_t ldx, const void* w_qkv,
                        const void* w_conv, const void* w_pw, const void* w_o,
                        const int32_t* cand, const void* residual, int64_t ldr,
                        void* out, int64_t ldo,
                        void* workspace, size_t workspace_bytes, void* stream);

/* No counterpart in the reference (which allocates its temporaries freely through PyTorch).
 * The same forward as convnn_b200_forward for callers that cannot provide a workspace because
 * they must not allocate device memory where they call from: a serving loop in which
 * cudaMalloc would stall the device, a plugin whose host application owns the allocator, or
 * a GPU whose memory is handed out in full once start-up is over.  The intermediates
 * live in a fixed array inside the library's device image: convnn_b200_noalloc_capacity()
 * bytes (32 MiB) per GPU.  A descriptor whose convnn_b200_workspace_bytes() exceeds the
 * capacity is refused with CONVNN_E_WORKSPACE.
 *   - The array is part of a CUDA module, and the CUDA runtime loads modules lazily by
 *     default (CUDA_MODULE_LOADING=LAZY): the GPU reserves the 32 MiB when the module is
 *     first touched, not when the shared library is loaded.  convnn_b200_noalloc_capacity()
 *     touches it: it resolves (and caches) the array's device address for the CURRENT
 *     device.  Call it once per device at start-up, with that device current, before
 *     memory is handed out and outside any stream capture; from then on
 *     convnn_b200_forward_noalloc() neither allocates nor frees anything and makes no
 *     address lookup.  Without that warm-up the first forward on a device does the lookup
 *     itself: it may then fail with CONVNN_E_CUDA on a GPU with no memory left, and must not
 *     run inside a capture.  The array is held until the process exits.
 *   - All calls on a device share the one array and it keeps the previous call's contents.
 *     Every intermediate is written before it is read, so nothing has to be cleared, but two
 *     calls that overlap on the GPU (different streams, graph branches, host threads) race
 *     on it: keep calls on one device stream-ordered. */
size_t convnn_b200_noalloc_capacity(void);
int convnn_b200_forward_noalloc(const convnn_desc* d, const void* x, int64_t ldx, const void* w_qkv,
                                const void* w_conv, const void* w_pw, const void* w_o,
                                const int32_t* cand, const void* residual, int64_t ldr,
                                void* out, int64_t ldo, void* stream);

/* ---- callers of the hot path: the rest of the reference's TransformerEncoder / ViT ----
 * dtype is a convnn_dtype; all pointers are device pointers in that type. */

/* y = LayerNorm(x) over the last dimension, affine (nn.LayerNorm: vit.py:247-248 as used at
 * vit.py:262, 267).  rows x D, strides ldx / ldy elements, statistics in fp32. */
int convnn_b200_layernorm(int dtype, const void* x, int64_t ldx, const void* gamma, const void* beta,
                          float eps, void* y, int64_t ldy, int64_t rows, int32_t D, void* stream);

/* out = [GELU](a * w^T + bias) [+ residual]: nn.Linear with its activation and the skip
 * connection folded in (vit.py:253-258 with 269; vit.py:71; and, on unfolded patches,
 * the Conv2d patch projection vit.py:99, 105).  a (M, K) stride lda; w (N, K) as nn.Linear
 * stores it; bias (N) or NULL; residual (M, N) stride ldr or NULL, added after rounding. */
int convnn_b200_linear(int dtype, const void* a, int64_t lda, const void* w, const void* bias,
                       const void* residual, int64_t ldr, void* out, int64_t ldo,
                       int64_t M, int32_t N, int32_t K, int32_t gelu, void* stream);

/* Unfold non-overlapping P x P patches: img (B, C, Hh, Ww) -> out (B * Hh/P * Ww/P, C*P*P),
 * the im2col of Conv2d(kernel = stride = P) (vit.py:99, 105-107). */
int convnn_b200_patchify(int dtype, const void* img, void* out, int32_t B, int32_t C, int32_t Hh,
                         int32_t Ww, int32_t P, void* stream);

/* The same unfold for images that are still 8-bit, with the loader's ToTensor + Normalize
 * (reference dataset.py:22-23, 73-74, 84-85) applied on the way: out = (img / 255 - mean[c]) *
 * inv_std[c] in `dtype`.  img (B, C, Hh, Ww) uint8, mean / inv_std (C) float32, all DEVICE
 * pointers.  Lets a caller ship a quarter of the bytes of float32 images over PCIe. */
int convnn_b200_patchify_u8(int dtype, const uint8_t* img, const float* mean, const float* inv_std, void* out,
                            int32_t B, int32_t C, int32_t Hh, int32_t Ww, int32_t P, void* stream);

/* Embedding tail: out[b, 0] = cls + pe[0]; out[b, 1 + n] = LayerNorm(proj[b, n]) + pe[1 + n]
 * (PatchEmbedding.norm, class token and positional table: vit.py:108, 126-135).
 * proj (B, Np, D), cls (D), pe (Np + 1, D), out (B, Np + 1, D), all contiguous. */
int convnn_b200_embed_tokens(int dtype, const void* proj, const void* gamma, const void* beta, float eps,
                             const void* cls, const void* pe, void* out, int32_t B, int32_t Np,
                             int32_t D, void* stream);

/* ---- LayerNorm folded into the GEMM that consumes it (bfloat16 only) ----
 * No reference counterpart as functions: together they compute exactly what vit.py:262-269 does
 * (norm1 -> attention, norm2 -> mlp) without writing or re-reading the normalised rows.  With
 * W' = W diag(gamma), c[n] = sum_k W'[n,k], b'[n] = sum_k W[n,k] beta[k] + bias[n]:
 *     LayerNorm(x) W^T + bias = rstd (x W'^T - mean c + sigma b'),   sigma = 1 / rstd,
 * so the consumer GEMM reads the rows x themselves plus their moments (sum x, sum x^2), and the
 * GEMM that produced x (always one with a skip connection in the encoder) emits those moments from
 * its epilogue.  `moments` buffers are float32 [planes][convnn_b200_moment_stride(M)][2], 16-byte
 * aligned: partial sums that the consumer adds up over the planes (it fetches them by TMA, hence
 * the even plane stride).  Rounding differs from the unfused order only in where the bfloat16 rounding
 * of the normalised activations happens (here the weights W' are rounded instead). */

/* Planes a GEMM with N output columns writes into `moments_out` (2 per 256-column tile), and the
 * entries (of two floats) from one plane of an M-row moments buffer to the next. */
int convnn_b200_moment_planes(int32_t N);
int64_t convnn_b200_moment_stride(int64_t M);
/* 1 if convnn_b200_prenorm_linear / _forward take this shape (the folded W tile must stay resident
 * in shared memory: small K), else 0 and the caller keeps LayerNorm + linear / forward. */
int convnn_b200_prenorm_linear_supported(int32_t N, int32_t K, int32_t gelu);
int convnn_b200_prenorm_forward_supported(const convnn_desc* d);
/* moments[r] = (sum, sum of squares) of row r of x (rows x D bfloat16, stride ldx): one plane, for
 * rows that no GEMM of this library produced (the embedding's output). */
int convnn_b200_row_moments(const void* x, int64_t ldx, int64_t rows, int32_t D, float* moments, void* stream);
/* Prepares the operands of the folded GEMM from nn.Linear(K -> N) weights w (N, K), bias (N) or
 * NULL and the LayerNorm's gamma, beta (K): w_folded (N, K) and w_extra (N, 16), all bfloat16. */
int convnn_b200_fold_layernorm(const void* w, const void* bias, const void* gamma, const void* beta, int32_t N,
                               int32_t K, void* w_folded, void* w_extra, void* stream);
/* out = [GELU](LayerNorm(a) w^T + bias) from the un-normalised rows a (M, K) and their moments
 * (vit.py:267 with 253-255).  CONVNN_E_UNSUPPORTED where _supported() says 0. */
int convnn_b200_prenorm_linear(const void* a, int64_t lda, const float* moments, int32_t planes, float eps,
                               const void* w_folded, const void* w_extra, void* out, int64_t ldo, int64_t M,
                               int32_t N, int32_t K, int32_t gelu, void* stream);
/* convnn_b200_linear with a skip connection (residual != NULL) that also writes the moments of
 * the rows it stores: moments_out = float32 [convnn_b200_moment_planes(N)][convnn_b200_moment_stride(M)][2]. */
int convnn_b200_linear_moments(const void* a, int64_t lda, const void* w, const void* bias, const void* residual,
                               int64_t ldr, void* out, int64_t ldo, int64_t M, int32_t N, int32_t K,
                               float* moments_out, void* stream);
/* convnn_b200_forward on rows x that have NOT been normalised yet (norm1 folded into the K/V/Q
 * projection; sampling 'all' only), optionally emitting the moments of residual + layer(x) for the
 * next folded GEMM (moments_out may be NULL; it needs residual != NULL).  With w_o == NULL
 * (num_heads = 1 only) the call stops before the output projection and writes the layer's
 * head-merged pre-projection rows (B, T, D) contiguously to `out`, for convnn_b200_outproj_mlp. */
int convnn_b200_prenorm_forward(const convnn_desc* d, const void* x, int64_t ldx, const float* moments,
                                int32_t planes, float eps, const void* w_qkv_folded, const void* w_qkv_extra,
                                const void* w_conv, const void* w_pw, const void* w_o, const void* residual,
                                int64_t ldr, void* out, int64_t ldo, float* moments_out, void* workspace,
                                size_t workspace_bytes, void* stream);

/* The whole MLP block of the encoder as one kernel (vit.py:267-269 with 253-258):
 *     out = x + (GELU(LayerNorm(x) w1^T + b1) w2^T + b2)
 * from the un-normalised rows x (M, D) and their moments; the hidden activations (M, d_mlp) stay in
 * shared memory / TMEM.  w1_folded (d_mlp, D) and w1_extra (d_mlp, 16) come from
 * convnn_b200_fold_layernorm(w1, b1, gamma, beta); w2 (D, d_mlp) and b2 (D) or NULL as nn.Linear
 * stores them.  moments_out (or NULL): float32 [convnn_b200_prenorm_mlp_moment_planes()]
 * [convnn_b200_moment_stride(M)][2], the moments of the rows of out as partial sums.  bfloat16;
 * D in {64, 128, 192}, d_mlp a multiple of 128, at most 16 planes of incoming moments
 * (CONVNN_E_UNSUPPORTED otherwise: use prenorm_linear + linear_moments).  out may not alias x. */
int convnn_b200_prenorm_mlp_supported(int32_t D, int32_t DM, int32_t planes);
int convnn_b200_prenorm_mlp_moment_planes(void);
int convnn_b200_prenorm_mlp(const void* x, int64_t ldx, const float* moments, int32_t planes, float eps,
                            const void* w1_folded, const void* w1_extra, const void* w2, const void* b2, void* out,
                            int64_t ldo, int64_t M, int32_t D, int32_t DM, float* moments_out, void* stream);

/* The output projection of the attention layer, its skip connection and the whole MLP block in one
 * kernel (layers.py:320 with vit.py:264, then vit.py:267-269):
 *     x1 = x + o w_o^T,     out = x1 + (GELU(LayerNorm(x1) w1^T + b1) w2^T + b2)
 * o (M, D) is the head-merged output of convnn_b200_gather_conv (num_heads = 1: the per-head layout IS
 * (M, D)), w_o (D, D) bias-free, x (M, D) the rows that entered the attention layer.  The moments
 * of x1 are computed inside.  Shapes as convnn_b200_prenorm_mlp (ask
 * convnn_b200_prenorm_mlp_supported(D, DM, 1)); moments_out as there.  out may alias neither o nor x. */
int convnn_b200_outproj_mlp(const void* o, int64_t ld_o, const void* w_o, const void* x, int64_t ldx, float eps,
                            const void* w1_folded, const void* w1_extra, const void* w2, const void* b2, void* out,
                            int64_t ldo, int64_t M, int32_t D, int32_t DM, float* moments_out, void* stream);

/* convnn_b200_embed_tokens that also writes the moments (sum, sum of squares) of every row it
 * stores: moments_out = float32 [convnn_b200_moment_stride(B * (Np + 1))][2], one plane, for the first
 * folded GEMM behind the embedding (instead of a convnn_b200_row_moments pass).  moments_out may be NULL. */
int convnn_b200_embed_tokens_moments(int dtype, const void* proj, const void* gamma, const void* beta, float eps,
                                     const void* cls, const void* pe, void* out, int32_t B, int32_t Np, int32_t D,
                                     float* moments_out, void* stream);

/* ---- the other halves of the reference's branching wrappers (layers.py:574-577, 648-651) ---- */

/* MultiHeadAttention.forward (layers.py:105-130), eval mode, no mask: q, k, v projections with the
 * packed bias-free weight w_qkv = (3, D, D) [W_q; W_k; W_v], softmax(q k^T / sqrt(d_k)) v per head,
 * then the bias-free W_o.  x (B, T, D) row stride ldx (a channel slice of a wider tensor goes in
 * as it is, layers.py:649), out (B, T, D) row stride ldo (written straight into the concat buffer).
 * workspace: convnn_b200_attention_workspace_bytes() bytes for q, k, v and the per-head output. */
size_t convnn_b200_attention_workspace_bytes(int dtype, int32_t B, int32_t T, int32_t D);
int convnn_b200_softmax_attention(int dtype, const void* x, int64_t ldx, const void* w_qkv, const void* w_o,
                                  void* out, int64_t ldo, int32_t B, int32_t T, int32_t D, int32_t H,
                                  void* workspace, size_t workspace_bytes, void* stream);

/* MultiHeadConv1dAttention.forward (layers.py:477-500): y = x W_x^T + b_x, per-head
 * Conv1d(d_k, d_k, kernel_size, padding='same') with bias over the tokens, the reference's flat
 * head reinterpretation (applied for every H, with seq_length = T), then W_o with bias.
 * w_conv is packed (d_k out, kernel_size, d_k in) from the module's (d_k, d_k, kernel_size). */
size_t convnn_b200_conv1d_attention_workspace_bytes(int dtype, int32_t B, int32_t T, int32_t D, int32_t kernel_size);
int convnn_b200_conv1d_attention(int dtype, const void* x, int64_t ldx, const void* w_x, const void* b_x,
                                 const void* w_conv, const void* b_conv, const void* w_o, const void* b_o,
                                 void* out, int64_t ldo, int32_t B, int32_t T, int32_t D, int32_t H,
                                 int32_t kernel_size, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CONVNN_B200_H */
