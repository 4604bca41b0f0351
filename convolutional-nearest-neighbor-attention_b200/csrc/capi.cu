// extern "C" surface of libconvnn_b200: argument validation, workspace carving and the
// chaining of the stage kernels on the caller's stream.
#include <atomic>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace convnn {

static thread_local char g_err[512] = "";

int set_error(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}
void clear_error() { g_err[0] = 0; }

bool force_simt() {
    static const bool v = [] {
        const char* e = getenv("CONVNN_B200_FORCE_SIMT");
        return e && e[0] == '1';
    }();
    return v;
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int validate(const convnn_desc* d, Dims* out) {
    if (!d) return set_error(CONVNN_E_NULL, "descriptor is NULL");
    if (d->B < 1 || d->T < 1 || d->S < 1 || d->D < 1 || d->H < 1 || d->K < 1)
        return set_error(CONVNN_E_INVALID, "B, T, S, D, H, K must be positive (got %d %d %d %d %d %d)", d->B, d->T,
                         d->S, d->D, d->H, d->K);
    if (d->D % d->H != 0) return set_error(CONVNN_E_INVALID, "d_hidden must be divisible by num_heads");
    if (d->dtype != CONVNN_F32 && d->dtype != CONVNN_BF16) return set_error(CONVNN_E_INVALID, "unknown dtype %d", d->dtype);
    if (d->metric < 0 || d->metric > 2) return set_error(CONVNN_E_INVALID, "unknown metric %d", d->metric);
    if (d->conv_type < 0 || d->conv_type > 2) return set_error(CONVNN_E_INVALID, "unknown conv_type %d", d->conv_type);
    if (d->reserved != 0) return set_error(CONVNN_E_INVALID, "reserved field must be 0");
    if (!d->sampled && d->S != d->T)
        return set_error(CONVNN_E_INVALID, "sampling 'all' needs S == T (got S=%d, T=%d)", d->S, d->T);
    if (d->coord && d->conv_type == CONVNN_DEPTHWISE)
        return set_error(CONVNN_E_INVALID, "coordinate_encoding with a depthwise conv is rejected by the reference "
                                           "(out_channels not divisible by groups)");
    const int nsel = d->sampled ? d->K - 1 : d->K;
    if (nsel > d->S) return set_error(CONVNN_E_TOPK_RANGE, "selected index k out of range");
    if (d->K > kMaxK) return set_error(CONVNN_E_UNSUPPORTED, "K=%d exceeds this build's limit of %d", d->K, kMaxK);
    if (d->H > 1 && d->T != d->seq_length)
        return set_error(CONVNN_E_SEQ_LENGTH, "shape '[%d, -1, %d, %d]' is invalid for input of size %lld", d->B,
                         d->D / d->H, d->seq_length, (long long)d->B * d->T * d->D);
    if ((long long)d->B * d->T * d->D >= (1ll << 31) || (long long)d->B * d->H * d->T * d->K >= (1ll << 31))
        return set_error(CONVNN_E_UNSUPPORTED, "tensor exceeds 2^31 elements");
    if (out) {
        out->B = d->B; out->T = d->T; out->S = d->S; out->D = d->D; out->H = d->H; out->K = d->K;
        out->dk = d->D / d->H;
        out->C = out->dk + (d->coord ? 1 : 0);
        out->Cp = d->coord ? ((out->dk + 1 + 7) / 8) * 8 : out->dk;
        out->nsel = nsel;
        out->elt = d->dtype == CONVNN_F32 ? 4 : 2;
    }
    return CONVNN_OK;
}

namespace {

int check_device() {
    static std::atomic<int> ok_mask[64];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) {
        cudaGetLastError();
        return set_error(CONVNN_E_DEVICE, "no CUDA device is current");
    }
    if (dev < 64 && ok_mask[dev].load(std::memory_order_relaxed) == 1) return CONVNN_OK;
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10)
        return set_error(CONVNN_E_DEVICE, "device %d is compute capability %d.x; this library is built for sm_100a only", dev, major);
    if (dev < 64) ok_mask[dev].store(1, std::memory_order_relaxed);
    return CONVNN_OK;
}

struct Workspace {
    char *q, *k, *v, *o, *scratch;
    float *qstat, *kstat, *val;
    int32_t* idx;
    size_t total;
};

size_t up256(size_t n) { return (n + 255) & ~(size_t)255; }

// Gathered candidate rows of x (B, S, D) for the query projection, later reused for the conv's
// GEMM operand and for the head-merged (B, T, D) operand of the output projection.
size_t stage_scratch(const Dims& dm, int conv_type) {
    size_t n = (size_t)dm.B * (dm.T > dm.S ? dm.T : dm.S) * dm.D;
    if (conv_type == CONVNN_STANDARD) {          // weighted neighbour block (B, H, T, K*C) of the tensor-core conv
        const size_t m = (size_t)dm.B * dm.H * dm.T * dm.K * dm.C;
        if (m > n) n = m;
    } else if (conv_type == CONVNN_DEPTHWISE_SEPARABLE) {
        const size_t m = (size_t)dm.B * dm.H * dm.T * dm.C;
        if (m > n) n = m;
    }
    return n * dm.elt;
}

Workspace carve(const Dims& dm, int conv_type, void* base) {
    Workspace w;
    char* p = static_cast<char*>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) { char* r = p ? p + off : nullptr; off += up256(bytes); return r; };
    w.q = take((size_t)dm.B * dm.S * dm.H * dm.Cp * dm.elt);
    w.k = take((size_t)dm.B * dm.T * dm.H * dm.Cp * dm.elt);
    w.v = take((size_t)dm.B * dm.T * dm.H * dm.Cp * dm.elt);
    w.o = take((size_t)dm.B * dm.H * dm.T * dm.dk * dm.elt);
    w.qstat = reinterpret_cast<float*>(take((size_t)dm.B * dm.H * dm.S * 4));
    w.kstat = reinterpret_cast<float*>(take((size_t)dm.B * dm.H * dm.T * 4));
    w.val = reinterpret_cast<float*>(take((size_t)dm.B * dm.H * dm.T * dm.K * 4));
    w.idx = reinterpret_cast<int32_t*>(take((size_t)dm.B * dm.H * dm.T * dm.K * 4));
    w.scratch = take(stage_scratch(dm, conv_type));
    w.total = off;
    return w;
}

}  // namespace

int check_device_is_sm100() { return check_device(); }

}  // namespace convnn

using namespace convnn;

#define REQUIRE_PTR(p)                                                               \
    do {                                                                             \
        if (!(p)) return set_error(CONVNN_E_NULL, "%s: argument '%s' is NULL", __func__, #p); \
    } while (0)

extern "C" {

int convnn_b200_abi_version(void) { return CONVNN_B200_ABI_VERSION; }

const char* convnn_b200_status_string(int s) {
    switch (s) {
        case CONVNN_OK: return "ok";
        case CONVNN_E_INVALID: return "invalid argument";
        case CONVNN_E_UNSUPPORTED: return "unsupported configuration";
        case CONVNN_E_NULL: return "null pointer";
        case CONVNN_E_ALIGN: return "misaligned pointer or leading dimension";
        case CONVNN_E_WORKSPACE: return "workspace too small";
        case CONVNN_E_CUDA: return "CUDA launch failure";
        case CONVNN_E_DEVICE: return "not an sm_100 device";
        case CONVNN_E_TOPK_RANGE: return "selected index k out of range";
        case CONVNN_E_SEQ_LENGTH: return "T != seq_length with num_heads > 1";
        default: return "unknown status";
    }
}

const char* convnn_b200_last_error(void) { return g_err; }

int convnn_b200_device_status(int* code) {
    if (!code) return set_error(CONVNN_E_NULL, "convnn_b200_device_status: argument 'code' is NULL");
    int a = 0, b = 0, c = 0, rc;
    if ((rc = read_sim_topk_status(&a))) return rc;
    if ((rc = read_gemm_tc_status(&b))) return rc;
    if ((rc = read_sim_topk2_status(&c))) return rc;
    if (!c && (rc = read_dw_stream_status(&c))) return rc;
    if (!c && (rc = read_attention_status(&c))) return rc;
    if (!c && (rc = read_mlp_tc_status(&c))) return rc;
    *code = a ? a : (b ? b : c);
    return CONVNN_OK;
}

uint64_t convnn_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int convnn_b200_head_channels(const convnn_desc* d) {
    Dims dm;
    int rc = validate(d, &dm);
    return rc != CONVNN_OK ? rc : dm.Cp;
}

size_t convnn_b200_stage_scratch_bytes(const convnn_desc* d) {
    Dims dm;
    if (validate(d, &dm) != CONVNN_OK) return 0;
    return stage_scratch(dm, d->conv_type);
}

size_t convnn_b200_workspace_bytes(const convnn_desc* d) {
    Dims dm;
    if (validate(d, &dm) != CONVNN_OK) return 0;
    return carve(dm, d->conv_type, nullptr).total;
}

}  // extern "C"

namespace {
// Pre-norm fold of the layer's first GEMM: x holds the rows before norm1, w_qkv the folded weight.
struct PreNorm {
    const float* moments;
    int planes;
    float eps;
    const void* w_extra;
};

bool qkv_fold_supported(const convnn_desc* d, const Dims& dm) {
    if (d->dtype != CONVNN_BF16 || d->coord || d->sampled || force_simt()) return false;
    const bool stats = d->metric != CONVNN_MATMUL;
    if (stats && gemm_tc_stat_pieces(dm.D, dm.dk) != 1) return false;
    return gemm_tc_prenorm_supported(3 * dm.D, dm.D, 3, stats, false);
}

int qkv_proj_impl(const convnn_desc* d, const void* x, int64_t ldx, const void* w_qkv,
                  const int32_t* cand, void* q, void* k, void* v, float* qstat, float* kstat,
                  void* scratch, void* stream, const PreNorm* pn) {
    Dims dm;
    int rc = validate(d, &dm);
    if (rc) return rc;
    REQUIRE_PTR(x); REQUIRE_PTR(w_qkv); REQUIRE_PTR(q); REQUIRE_PTR(k); REQUIRE_PTR(v);
    if (d->sampled) REQUIRE_PTR(cand);
    if (d->metric != CONVNN_MATMUL) { REQUIRE_PTR(qstat); REQUIRE_PTR(kstat); }
    if (ldx < dm.D) return set_error(CONVNN_E_INVALID, "ldx=%lld is smaller than D=%d", (long long)ldx, dm.D);
    if ((rc = check_device())) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t wsz = (size_t)dm.D * dm.D * dm.elt;
    const bool stats = d->metric != CONVNN_MATMUL;
    // bfloat16 without the coordinate channel: (B, rows, H, d_k) is plain (B*rows, D), so the
    // projections are ordinary GEMMs for the tensor cores
    if (d->dtype == CONVNN_BF16 && !d->coord && !force_simt()) {
        const char* wb = static_cast<const char*>(w_qkv);
        void* kvq[3] = {k, v, q};
        // Fused statistics: always when a tile holds whole heads; for heads that span several
        // tiles the partial sums need room in `scratch` behind the gathered candidate rows
        // (pieces x B x H x (T + S) floats).
        const int pieces = stats ? gemm_tc_stat_pieces(dm.D, dm.dk) : 0;
        const size_t gathered = d->sampled ? up256((size_t)dm.B * dm.S * dm.D * dm.elt) : 0;
        const size_t part_k = up256((size_t)pieces * dm.B * dm.H * dm.T * 4);
        const size_t part_q = up256((size_t)pieces * dm.B * dm.H * dm.S * 4);
        const size_t scratch_min = (size_t)dm.B * (dm.T > dm.S ? dm.T : dm.S) * dm.D * dm.elt;   // what every caller provides
        const bool fuse = pieces == 1 || (pieces > 1 && scratch && gathered + part_k + part_q <= scratch_min);
        float* sc_k = pieces > 1 && fuse ? reinterpret_cast<float*>(static_cast<char*>(scratch) + gathered) : nullptr;
        float* sc_q = sc_k ? reinterpret_cast<float*>(static_cast<char*>(scratch) + gathered + part_k) : nullptr;
        GemmTcOpts o;
        o.stat_mode = d->metric; o.dk = dm.dk; o.heads = dm.H;
        bool done = false;
        if (pn) {
            if (!qkv_fold_supported(d, dm) || !gemm_tc_supported(x, ldx, w_qkv, dm.D, 3 * dm.D, 3, kvq, dm.D))
                return set_error(CONVNN_E_UNSUPPORTED, "prenorm_forward: this descriptor takes the unfused path "
                                                       "(see convnn_b200_prenorm_forward_supported)");
            o.ln_moments = pn->moments; o.ln_planes = pn->planes; o.ln_eps = pn->eps; o.ln_wextra = pn->w_extra;
        }
        if (!d->sampled && gemm_tc_supported(x, ldx, w_qkv, dm.D, 3 * dm.D, 3, kvq, dm.D)) {
            if (fuse) { o.stat[0] = kstat; o.stat[2] = qstat; o.rows_per_batch = dm.T; o.stat_scratch = sc_k; }
            if ((rc = launch_gemm_tc(x, ldx, w_qkv, dm.B * dm.T, 3 * dm.D, dm.D, 3, kvq, dm.D, o, st))) return rc;
            done = true;
        } else if (d->sampled && scratch && gemm_tc_supported(x, ldx, w_qkv, dm.D, 2 * dm.D, 2, kvq, dm.D) &&
                   gemm_tc_supported(scratch, dm.D, wb + 2 * wsz, dm.D, dm.D, 1, &kvq[2], dm.D)) {
            if (fuse) { o.stat[0] = kstat; o.rows_per_batch = dm.T; o.stat_scratch = sc_k; }
            if ((rc = launch_gemm_tc(x, ldx, w_qkv, dm.B * dm.T, 2 * dm.D, dm.D, 2, kvq, dm.D, o, st))) return rc;
            if ((rc = launch_gather_rows(d->dtype, x, ldx, cand, scratch, dm.B, dm.T, dm.S, dm.D, st))) return rc;
            GemmTcOpts oq;
            oq.stat_mode = d->metric; oq.dk = dm.dk; oq.heads = dm.H;
            if (fuse) { oq.stat[0] = qstat; oq.rows_per_batch = dm.S; oq.stat_scratch = sc_q; }
            if ((rc = launch_gemm_tc(scratch, dm.D, wb + 2 * wsz, dm.B * dm.S, dm.D, dm.D, 1, &kvq[2], dm.D, oq, st)))
                return rc;
            done = true;
        }
        if (done) {
            if (fuse || !stats) return CONVNN_OK;
            if ((rc = launch_head_fill_and_stats(d, dm, q, dm.S, qstat, st))) return rc;
            return launch_head_fill_and_stats(d, dm, k, dm.T, kstat, st);
        }
    }
    if (pn) return set_error(CONVNN_E_UNSUPPORTED, "prenorm_forward: this descriptor takes the unfused path");
    GemmParams p{};
    p.a = x; p.lda = ldx; p.bias = nullptr; p.N = dm.D; p.Kd = dm.D;
    p.a_mode = A_TOKENS; p.c_mode = C_HEADS; p.T = dm.T; p.H = dm.H; p.dk = dm.dk; p.Cp = dm.Cp; p.gelu = 0;
    // keys and values: every token
    p.cand = nullptr; p.rows_per_batch = dm.T; p.M = dm.B * dm.T;
    p.w = static_cast<const char*>(w_qkv); p.c = k;
    if ((rc = launch_gemm_simt(d->dtype, p, st))) return rc;
    p.w = static_cast<const char*>(w_qkv) + wsz; p.c = v;
    if ((rc = launch_gemm_simt(d->dtype, p, st))) return rc;
    // queries: candidate tokens only
    p.cand = d->sampled ? cand : nullptr; p.rows_per_batch = dm.S; p.M = dm.B * dm.S;
    p.w = static_cast<const char*>(w_qkv) + 2 * wsz; p.c = q;
    if ((rc = launch_gemm_simt(d->dtype, p, st))) return rc;
    if ((rc = launch_head_fill_and_stats(d, dm, q, dm.S, stats ? qstat : nullptr, st))) return rc;
    if ((rc = launch_head_fill_and_stats(d, dm, k, dm.T, stats ? kstat : nullptr, st))) return rc;
    if ((rc = launch_head_fill_and_stats(d, dm, v, dm.T, nullptr, st))) return rc;
    return CONVNN_OK;
}
}  // namespace

extern "C" {

int convnn_b200_qkv_proj(const convnn_desc* d, const void* x, int64_t ldx, const void* w_qkv,
                         const int32_t* cand, void* q, void* k, void* v, float* qstat, float* kstat,
                         void* scratch, void* stream) {
    return qkv_proj_impl(d, x, ldx, w_qkv, cand, q, k, v, qstat, kstat, scratch, stream, nullptr);
}

int convnn_b200_sim_topk(const convnn_desc* d, const void* q, const void* k, const float* qstat,
                         const float* kstat, const int32_t* cand, int32_t* idx, float* val, void* stream) {
    Dims dm;
    int rc = validate(d, &dm);
    if (rc) return rc;
    REQUIRE_PTR(q); REQUIRE_PTR(k); REQUIRE_PTR(idx); REQUIRE_PTR(val);
    if (d->sampled) REQUIRE_PTR(cand);
    if (d->metric != CONVNN_MATMUL) { REQUIRE_PTR(qstat); REQUIRE_PTR(kstat); }
    if ((rc = check_device())) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!force_simt() && sim_topk_tc_supported(d, dm, q, k))
        return launch_sim_topk_tc(d, dm, q, k, qstat, kstat, cand, idx, val, st);
    if (d->dtype == CONVNN_F32) return launch_sim_topk_simt_f32(d, dm, q, k, qstat, kstat, cand, idx, val, st);
    return launch_sim_topk_simt_bf16(d, dm, q, k, qstat, kstat, cand, idx, val, st);
}

int convnn_b200_gather_conv(const convnn_desc* d, const void* v, const int32_t* idx, const float* val,
                            const void* w_conv, const void* w_pw, void* o, void* scratch, void* stream) {
    Dims dm;
    int rc = validate(d, &dm);
    if (rc) return rc;
    REQUIRE_PTR(v); REQUIRE_PTR(idx); REQUIRE_PTR(val); REQUIRE_PTR(w_conv); REQUIRE_PTR(o);
    if (d->conv_type == CONVNN_DEPTHWISE_SEPARABLE) REQUIRE_PTR(w_pw);
    if ((rc = check_device())) return rc;
    return launch_gather_conv_simt(d, dm, v, idx, val, w_conv, w_pw, o, scratch, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

namespace {
int out_proj_impl(const convnn_desc* d, const void* o, const void* w_o, const void* residual, int64_t ldr,
                  void* out, int64_t ldo, void* scratch, void* stream, float* moments_out) {
    Dims dm;
    int rc = validate(d, &dm);
    if (rc) return rc;
    REQUIRE_PTR(o); REQUIRE_PTR(w_o); REQUIRE_PTR(out);
    if (residual && ldr < dm.D) return set_error(CONVNN_E_INVALID, "ldr=%lld is smaller than D=%d", (long long)ldr, dm.D);
    if (ldo < dm.D) return set_error(CONVNN_E_INVALID, "ldo=%lld is smaller than D=%d", (long long)ldo, dm.D);
    if ((rc = check_device())) return rc;
    if (d->dtype == CONVNN_BF16 && !force_simt()) {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        void* cs[1] = {out};
        GemmTcOpts go;
        go.residual = residual; go.ldr = ldr; go.moments_out = moments_out;
        const bool res_ok = !residual || (ldr % 8 == 0 && aligned16(residual));
        if (res_ok && dm.H == 1 && gemm_tc_supported(o, dm.D, w_o, dm.D, dm.D, 1, cs, ldo))
            return launch_gemm_tc(o, dm.D, w_o, dm.B * dm.T, dm.D, dm.D, 1, cs, ldo, go, st);
        if (res_ok && dm.H > 1 && scratch && gemm_tc_supported(scratch, dm.D, w_o, dm.D, dm.D, 1, cs, ldo)) {
            if ((rc = launch_merge_heads(d->dtype, o, scratch, dm.B, dm.T, dm.H, dm.dk, st))) return rc;
            return launch_gemm_tc(scratch, dm.D, w_o, dm.B * dm.T, dm.D, dm.D, 1, cs, ldo, go, st);
        }
    }
    if (moments_out) return set_error(CONVNN_E_UNSUPPORTED, "out_proj: row moments need the tensor-core path");
    GemmParams p{};
    p.a = o; p.w = w_o; p.bias = nullptr; p.c = out; p.cand = nullptr;
    p.lda = dm.D; p.ldc = ldo; p.M = dm.B * dm.T; p.N = dm.D; p.Kd = dm.D;
    p.a_mode = dm.H == 1 ? A_ROWS : A_HEAD_QUIRK; p.c_mode = C_ROWS;
    p.rows_per_batch = dm.T; p.T = dm.T; p.H = dm.H; p.dk = dm.dk; p.Cp = dm.Cp; p.gelu = 0;
    p.residual = residual; p.ldr = ldr;
    return launch_gemm_simt(d->dtype, p, static_cast<cudaStream_t>(stream));
}
}  // namespace

extern "C" {

int convnn_b200_out_proj(const convnn_desc* d, const void* o, const void* w_o, const void* residual, int64_t ldr,
                         void* out, int64_t ldo, void* scratch, void* stream) {
    return out_proj_impl(d, o, w_o, residual, ldr, out, ldo, scratch, stream, nullptr);
}

int convnn_b200_forward(const convnn_desc* d, const void* x, int64_t ldx, const void* w_qkv,
                        const void* w_conv, const void* w_pw, const void* w_o, const int32_t* cand,
                        const void* residual, int64_t ldr, void* out, int64_t ldo, void* workspace,
                        size_t workspace_bytes, void* stream) {
    Dims dm;
    int rc = validate(d, &dm);
    if (rc) return rc;
    REQUIRE_PTR(workspace);
    if (!aligned16(workspace)) return set_error(CONVNN_E_ALIGN, "workspace must be 16-byte aligned");
    Workspace w = carve(dm, d->conv_type, workspace);
    if (workspace_bytes < w.total)
        return set_error(CONVNN_E_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes, w.total);
    if ((rc = convnn_b200_qkv_proj(d, x, ldx, w_qkv, cand, w.q, w.k, w.v, w.qstat, w.kstat, w.scratch, stream))) return rc;
    if ((rc = convnn_b200_sim_topk(d, w.q, w.k, w.qstat, w.kstat, cand, w.idx, w.val, stream))) return rc;
    if ((rc = convnn_b200_gather_conv(d, w.v, w.idx, w.val, w_conv, w_pw, w.o, w.scratch, stream))) return rc;
    return convnn_b200_out_proj(d, w.o, w_o, residual, ldr, out, ldo, w.scratch, stream);
}

int convnn_b200_layernorm(int dtype, const void* x, int64_t ldx, const void* gamma, const void* beta, float eps,
                          void* y, int64_t ldy, int64_t rows, int32_t D, void* stream) {
    if (dtype != CONVNN_F32 && dtype != CONVNN_BF16) return set_error(CONVNN_E_INVALID, "unknown dtype %d", dtype);
    REQUIRE_PTR(x); REQUIRE_PTR(gamma); REQUIRE_PTR(beta); REQUIRE_PTR(y);
    if (rows < 0 || D < 1 || ldx < D || ldy < D) return set_error(CONVNN_E_INVALID, "layernorm: bad shape");
    int rc = check_device();
    if (rc) return rc;
    if (rows == 0) return CONVNN_OK;
    return launch_layernorm(dtype, x, ldx, gamma, beta, eps, y, ldy, rows, D, nullptr, nullptr, 0, 0, nullptr,
                            static_cast<cudaStream_t>(stream));
}

int convnn_b200_embed_tokens_moments(int dtype, const void* proj, const void* gamma, const void* beta, float eps,
                                     const void* cls, const void* pe, void* out, int32_t B, int32_t Np, int32_t D,
                                     float* moments_out, void* stream) {
    if (dtype != CONVNN_F32 && dtype != CONVNN_BF16) return set_error(CONVNN_E_INVALID, "unknown dtype %d", dtype);
    REQUIRE_PTR(proj); REQUIRE_PTR(gamma); REQUIRE_PTR(beta); REQUIRE_PTR(cls); REQUIRE_PTR(pe); REQUIRE_PTR(out);
    if (B < 1 || Np < 1 || D < 1) return set_error(CONVNN_E_INVALID, "embed_tokens: bad shape");
    if (moments_out && (reinterpret_cast<uintptr_t>(moments_out) & 7u))
        return set_error(CONVNN_E_ALIGN, "embed_tokens: moments_out must be 8-byte aligned");
    int rc = check_device();
    if (rc) return rc;
    return launch_layernorm(dtype, proj, D, gamma, beta, eps, out, D, (long long)B * Np, D, pe, cls, Np, B, moments_out,
                            static_cast<cudaStream_t>(stream));
}

int convnn_b200_embed_tokens(int dtype, const void* proj, const void* gamma, const void* beta, float eps,
                             const void* cls, const void* pe, void* out, int32_t B, int32_t Np, int32_t D,
                             void* stream) {
    return convnn_b200_embed_tokens_moments(dtype, proj, gamma, beta, eps, cls, pe, out, B, Np, D, nullptr, stream);
}

int convnn_b200_patchify(int dtype, const void* img, void* out, int32_t B, int32_t C, int32_t Hh, int32_t Ww,
                         int32_t P, void* stream) {
    if (dtype != CONVNN_F32 && dtype != CONVNN_BF16) return set_error(CONVNN_E_INVALID, "unknown dtype %d", dtype);
    REQUIRE_PTR(img); REQUIRE_PTR(out);
    if (B < 1 || C < 1 || Hh < 1 || Ww < 1 || P < 1) return set_error(CONVNN_E_INVALID, "patchify: bad shape");
    int rc = check_device();
    if (rc) return rc;
    return launch_patchify(dtype, img, out, B, C, Hh, Ww, P, static_cast<cudaStream_t>(stream));
}

int convnn_b200_patchify_u8(int dtype, const uint8_t* img, const float* mean, const float* inv_std, void* out, int32_t B,
                            int32_t C, int32_t Hh, int32_t Ww, int32_t P, void* stream) {
    if (dtype != CONVNN_F32 && dtype != CONVNN_BF16) return set_error(CONVNN_E_INVALID, "unknown dtype %d", dtype);
    REQUIRE_PTR(img); REQUIRE_PTR(mean); REQUIRE_PTR(inv_std); REQUIRE_PTR(out);
    if (B < 1 || C < 1 || Hh < 1 || Ww < 1 || P < 1) return set_error(CONVNN_E_INVALID, "patchify: bad shape");
    int rc = check_device();
    if (rc) return rc;
    return launch_patchify_u8(dtype, img, mean, inv_std, out, B, C, Hh, Ww, P, static_cast<cudaStream_t>(stream));
}

int convnn_b200_linear(int dtype, const void* a, int64_t lda, const void* w, const void* bias, const void* residual,
                       int64_t ldr, void* out, int64_t ldo, int64_t M, int32_t N, int32_t K, int32_t gelu,
                       void* stream) {
    if (dtype != CONVNN_F32 && dtype != CONVNN_BF16) return set_error(CONVNN_E_INVALID, "unknown dtype %d", dtype);
    REQUIRE_PTR(a); REQUIRE_PTR(w); REQUIRE_PTR(out);
    if (M < 0 || N < 1 || K < 1 || lda < K || ldo < N || (residual && ldr < N) || M >= (1ll << 31))
        return set_error(CONVNN_E_INVALID, "linear: bad shape (M=%lld N=%d K=%d)", (long long)M, N, K);
    int rc = check_device();
    if (rc) return rc;
    if (M == 0) return CONVNN_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == CONVNN_BF16 && !force_simt()) {
        void* cs[1] = {out};
        const bool extra_ok = (!bias || aligned16(bias)) && (!residual || (aligned16(residual) && ldr % 8 == 0));
        if (extra_ok && gemm_tc_supported(a, lda, w, K, N, 1, cs, ldo)) {
            GemmTcOpts o;
            o.bias = bias; o.residual = residual; o.ldr = ldr; o.gelu = gelu;
            return launch_gemm_tc(a, lda, w, (int)M, N, K, 1, cs, ldo, o, st);
        }
    }
    GemmParams p{};
    p.a = a; p.w = w; p.bias = bias; p.c = out; p.cand = nullptr;
    p.lda = lda; p.ldc = ldo; p.M = (int)M; p.N = N; p.Kd = K;
    p.a_mode = A_ROWS; p.c_mode = C_ROWS; p.rows_per_batch = 1; p.T = 1; p.H = 1; p.dk = N; p.Cp = N;
    p.gelu = gelu; p.residual = residual; p.ldr = ldr;
    return launch_gemm_simt(dtype, p, st);
}

// ---- LayerNorm folded into the GEMM that consumes it ----------------------------------------------

int convnn_b200_moment_planes(int32_t N) { return N < 1 ? 0 : gemm_tc_moment_planes(N); }
int64_t convnn_b200_moment_stride(int64_t M) { return M < 0 ? 0 : gemm_tc_moment_stride(M); }

int convnn_b200_prenorm_linear_supported(int32_t N, int32_t K, int32_t gelu) {
    return (N >= 1 && K >= 1 && !force_simt() && gemm_tc_prenorm_supported(N, K, 1, false, gelu != 0)) ? 1 : 0;
}

int convnn_b200_prenorm_forward_supported(const convnn_desc* d) {
    Dims dm;
    if (validate(d, &dm) != CONVNN_OK) return 0;
    return qkv_fold_supported(d, dm) ? 1 : 0;
}

int convnn_b200_row_moments(const void* x, int64_t ldx, int64_t rows, int32_t D, float* moments, void* stream) {
    REQUIRE_PTR(x); REQUIRE_PTR(moments);
    if (rows < 0 || D < 1 || ldx < D) return set_error(CONVNN_E_INVALID, "row_moments: bad shape");
    int rc = check_device();
    if (rc) return rc;
    if (rows == 0) return CONVNN_OK;
    return launch_row_moments(x, ldx, rows, D, moments, static_cast<cudaStream_t>(stream));
}

int convnn_b200_fold_layernorm(const void* w, const void* bias, const void* gamma, const void* beta, int32_t N,
                               int32_t K, void* w_folded, void* w_extra, void* stream) {
    REQUIRE_PTR(w); REQUIRE_PTR(gamma); REQUIRE_PTR(beta); REQUIRE_PTR(w_folded); REQUIRE_PTR(w_extra);
    if (N < 1 || K < 1) return set_error(CONVNN_E_INVALID, "fold_layernorm: bad shape");
    int rc = check_device();
    if (rc) return rc;
    return launch_fold_layernorm(w, bias, gamma, beta, N, K, w_folded, w_extra, static_cast<cudaStream_t>(stream));
}

int convnn_b200_prenorm_linear(const void* a, int64_t lda, const float* moments, int32_t planes, float eps,
                               const void* w_folded, const void* w_extra, void* out, int64_t ldo, int64_t M,
                               int32_t N, int32_t K, int32_t gelu, void* stream) {
    REQUIRE_PTR(a); REQUIRE_PTR(moments); REQUIRE_PTR(w_folded); REQUIRE_PTR(w_extra); REQUIRE_PTR(out);
    if (M < 0 || N < 1 || K < 1 || lda < K || ldo < N || planes < 1 || M >= (1ll << 31))
        return set_error(CONVNN_E_INVALID, "prenorm_linear: bad shape (M=%lld N=%d K=%d planes=%d)", (long long)M, N, K, planes);
    int rc = check_device();
    if (rc) return rc;
    if (M == 0) return CONVNN_OK;
    void* cs[1] = {out};
    if (force_simt() || !gemm_tc_supported(a, lda, w_folded, K, N, 1, cs, ldo) ||
        !gemm_tc_prenorm_supported(N, K, 1, false, gelu != 0))
        return set_error(CONVNN_E_UNSUPPORTED, "prenorm_linear: N=%d K=%d takes the unfused path "
                                               "(see convnn_b200_prenorm_linear_supported)", N, K);
    GemmTcOpts o;
    o.gelu = gelu;
    o.ln_moments = moments; o.ln_planes = planes; o.ln_eps = eps; o.ln_wextra = w_extra;
    return launch_gemm_tc(a, lda, w_folded, (int)M, N, K, 1, cs, ldo, o, static_cast<cudaStream_t>(stream));
}

int convnn_b200_linear_moments(const void* a, int64_t lda, const void* w, const void* bias, const void* residual,
                               int64_t ldr, void* out, int64_t ldo, int64_t M, int32_t N, int32_t K,
                               float* moments_out, void* stream) {
    REQUIRE_PTR(a); REQUIRE_PTR(w); REQUIRE_PTR(residual); REQUIRE_PTR(out); REQUIRE_PTR(moments_out);
    if (M < 0 || N < 1 || K < 1 || lda < K || ldo < N || ldr < N || M >= (1ll << 31))
        return set_error(CONVNN_E_INVALID, "linear_moments: bad shape (M=%lld N=%d K=%d)", (long long)M, N, K);
    int rc = check_device();
    if (rc) return rc;
    if (M == 0) return CONVNN_OK;
    void* cs[1] = {out};
    const bool extra_ok = (!bias || aligned16(bias)) && aligned16(residual) && ldr % 8 == 0 &&
                          (reinterpret_cast<uintptr_t>(moments_out) & 7u) == 0;
    if (force_simt() || !extra_ok || !gemm_tc_supported(a, lda, w, K, N, 1, cs, ldo))
        return set_error(CONVNN_E_UNSUPPORTED, "linear_moments: needs the bfloat16 tensor-core path");
    GemmTcOpts o;
    o.bias = bias; o.residual = residual; o.ldr = ldr; o.moments_out = moments_out;
    return launch_gemm_tc(a, lda, w, (int)M, N, K, 1, cs, ldo, o, static_cast<cudaStream_t>(stream));
}

int convnn_b200_prenorm_forward(const convnn_desc* d, const void* x, int64_t ldx, const float* moments,
                                int32_t planes, float eps, const void* w_qkv_folded, const void* w_qkv_extra,
                                const void* w_conv, const void* w_pw, const void* w_o, const void* residual,
                                int64_t ldr, void* out, int64_t ldo, float* moments_out, void* workspace,
                                size_t workspace_bytes, void* stream) {
    Dims dm;
    int rc = validate(d, &dm);
    if (rc) return rc;
    REQUIRE_PTR(workspace); REQUIRE_PTR(moments); REQUIRE_PTR(w_qkv_extra);
    if (planes < 1) return set_error(CONVNN_E_INVALID, "prenorm_forward: planes must be positive");
    if (moments_out && !residual)
        return set_error(CONVNN_E_UNSUPPORTED, "prenorm_forward: row moments come with the skip connection");
    if (!aligned16(workspace)) return set_error(CONVNN_E_ALIGN, "workspace must be 16-byte aligned");
    Workspace w = carve(dm, d->conv_type, workspace);
    if (workspace_bytes < w.total)
        return set_error(CONVNN_E_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes, w.total);
    if (!w_o && (dm.H != 1 || ldo != dm.D || residual || moments_out))
        return set_error(CONVNN_E_INVALID, "prenorm_forward: without w_o the layer's pre-projection output is written to a "
                                           "contiguous `out` (num_heads = 1, ldo = D, no residual, no moments)");
    const PreNorm pn{moments, planes, eps, w_qkv_extra};
    if ((rc = qkv_proj_impl(d, x, ldx, w_qkv_folded, nullptr, w.q, w.k, w.v, w.qstat, w.kstat, w.scratch, stream, &pn))) return rc;
    if ((rc = convnn_b200_sim_topk(d, w.q, w.k, w.qstat, w.kstat, nullptr, w.idx, w.val, stream))) return rc;
    if (!w_o)      // the caller fuses the output projection into what follows (convnn_b200_outproj_mlp)
        return convnn_b200_gather_conv(d, w.v, w.idx, w.val, w_conv, w_pw, out, w.scratch, stream);
    if ((rc = convnn_b200_gather_conv(d, w.v, w.idx, w.val, w_conv, w_pw, w.o, w.scratch, stream))) return rc;
    return out_proj_impl(d, w.o, w_o, residual, ldr, out, ldo, w.scratch, stream, moments_out);
}

int convnn_b200_prenorm_mlp_supported(int32_t D, int32_t DM, int32_t planes) {
    return (!force_simt() && mlp_tc_supported(D, DM, planes)) ? 1 : 0;
}

int convnn_b200_prenorm_mlp_moment_planes(void) { return mlp_tc_moment_planes(); }

int convnn_b200_prenorm_mlp(const void* x, int64_t ldx, const float* moments, int32_t planes, float eps,
                            const void* w1_folded, const void* w1_extra, const void* w2, const void* b2, void* out,
                            int64_t ldo, int64_t M, int32_t D, int32_t DM, float* moments_out, void* stream) {
    REQUIRE_PTR(x); REQUIRE_PTR(moments); REQUIRE_PTR(w1_folded); REQUIRE_PTR(w1_extra); REQUIRE_PTR(w2); REQUIRE_PTR(out);
    if (M < 0 || D < 1 || DM < 1 || ldx < D || ldo < D || planes < 1 || M >= (1ll << 31))
        return set_error(CONVNN_E_INVALID, "prenorm_mlp: bad shape (M=%lld D=%d d_mlp=%d planes=%d)", (long long)M, D, DM, planes);
    int rc = check_device();
    if (rc) return rc;
    if (M == 0) return CONVNN_OK;
    if (force_simt()) return set_error(CONVNN_E_UNSUPPORTED, "prenorm_mlp: needs the tensor-core path");
    return launch_mlp_tc(x, ldx, moments, planes, eps, w1_folded, w1_extra, w2, b2, out, ldo, (int)M, D, DM, moments_out,
                         nullptr, nullptr, 0, static_cast<cudaStream_t>(stream));
}

int convnn_b200_outproj_mlp(const void* o, int64_t ld_o, const void* w_o, const void* x, int64_t ldx, float eps,
                            const void* w1_folded, const void* w1_extra, const void* w2, const void* b2, void* out,
                            int64_t ldo, int64_t M, int32_t D, int32_t DM, float* moments_out, void* stream) {
    REQUIRE_PTR(o); REQUIRE_PTR(w_o); REQUIRE_PTR(x); REQUIRE_PTR(w1_folded); REQUIRE_PTR(w1_extra); REQUIRE_PTR(w2);
    REQUIRE_PTR(out);
    if (M < 0 || D < 1 || DM < 1 || ld_o < D || ldx < D || ldo < D || M >= (1ll << 31))
        return set_error(CONVNN_E_INVALID, "outproj_mlp: bad shape (M=%lld D=%d d_mlp=%d)", (long long)M, D, DM);
    int rc = check_device();
    if (rc) return rc;
    if (M == 0) return CONVNN_OK;
    if (force_simt()) return set_error(CONVNN_E_UNSUPPORTED, "outproj_mlp: needs the tensor-core path");
    return launch_mlp_tc(o, ld_o, nullptr, 1, eps, w1_folded, w1_extra, w2, b2, out, ldo, (int)M, D, DM, moments_out, w_o, x,
                         ldx, static_cast<cudaStream_t>(stream));
}

// ---- the other halves of the branching wrappers ------------------------------------------------

static int branch_args_ok(const char* who, int dtype, int32_t B, int32_t T, int32_t D, int32_t H, int64_t ldx, int64_t ldo) {
    if (dtype != CONVNN_F32 && dtype != CONVNN_BF16) return set_error(CONVNN_E_INVALID, "%s: unknown dtype %d", who, dtype);
    if (B < 1 || T < 1 || D < 1 || H < 1 || D % H != 0)
        return set_error(CONVNN_E_INVALID, "%s: bad shape (B=%d T=%d D=%d H=%d)", who, B, T, D, H);
    if (ldx < D || ldo < D) return set_error(CONVNN_E_INVALID, "%s: a leading dimension is smaller than D=%d", who, D);
    if ((long long)B * T * D >= (1ll << 31)) return set_error(CONVNN_E_UNSUPPORTED, "%s: tensor exceeds 2^31 elements", who);
    return CONVNN_OK;
}

size_t convnn_b200_attention_workspace_bytes(int dtype, int32_t B, int32_t T, int32_t D) {
    if ((dtype != CONVNN_F32 && dtype != CONVNN_BF16) || B < 1 || T < 1 || D < 1) return 0;
    return 4 * up256((size_t)B * T * D * (dtype == CONVNN_F32 ? 4 : 2));
}

int convnn_b200_softmax_attention(int dtype, const void* x, int64_t ldx, const void* w_qkv, const void* w_o, void* out,
                                  int64_t ldo, int32_t B, int32_t T, int32_t D, int32_t H, void* workspace,
                                  size_t workspace_bytes, void* stream) {
    int rc = branch_args_ok("softmax_attention", dtype, B, T, D, H, ldx, ldo);
    if (rc) return rc;
    REQUIRE_PTR(x); REQUIRE_PTR(w_qkv); REQUIRE_PTR(w_o); REQUIRE_PTR(out); REQUIRE_PTR(workspace);
    if (!aligned16(workspace)) return set_error(CONVNN_E_ALIGN, "workspace must be 16-byte aligned");
    const size_t need = convnn_b200_attention_workspace_bytes(dtype, B, T, D);
    if (workspace_bytes < need)
        return set_error(CONVNN_E_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes, need);
    if ((rc = check_device())) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t elt = dtype == CONVNN_F32 ? 4 : 2, part = up256((size_t)B * T * D * elt);
    char* ws = static_cast<char*>(workspace);
    void* qkv[3] = {ws, ws + part, ws + 2 * part};
    void* o = ws + 3 * part;
    const long long M = (long long)B * T;
    // q, k, v: one launch over the packed weight where the tensor-core GEMM takes the shape
    if (dtype == CONVNN_BF16 && !force_simt() && gemm_tc_supported(x, ldx, w_qkv, D, 3 * D, 3, qkv, D)) {
        GemmTcOpts go;
        if ((rc = launch_gemm_tc(x, ldx, w_qkv, (int)M, 3 * D, D, 3, qkv, D, go, st))) return rc;
    } else {
        for (int i = 0; i < 3; ++i)
            if ((rc = convnn_b200_linear(dtype, x, ldx, static_cast<const char*>(w_qkv) + (size_t)i * D * D * elt, nullptr,
                                         nullptr, 0, qkv[i], D, M, D, D, 0, stream)))
                return rc;
    }
    if ((rc = launch_attention(dtype, qkv[0], qkv[1], qkv[2], o, B, T, D, H, st))) return rc;
    return convnn_b200_linear(dtype, o, D, w_o, nullptr, nullptr, 0, out, ldo, M, D, D, 0, stream);
}

size_t convnn_b200_conv1d_attention_workspace_bytes(int dtype, int32_t B, int32_t T, int32_t D, int32_t kernel_size) {
    if ((dtype != CONVNN_F32 && dtype != CONVNN_BF16) || B < 1 || T < 1 || D < 1 || kernel_size < 1) return 0;
    const size_t elt = dtype == CONVNN_F32 ? 4 : 2, part = up256((size_t)B * T * D * elt);
    return 3 * part + up256((size_t)B * T * D * kernel_size * elt);
}

int convnn_b200_conv1d_attention(int dtype, const void* x, int64_t ldx, const void* w_x, const void* b_x,
                                 const void* w_conv, const void* b_conv, const void* w_o, const void* b_o, void* out,
                                 int64_t ldo, int32_t B, int32_t T, int32_t D, int32_t H, int32_t kernel_size,
                                 void* workspace, size_t workspace_bytes, void* stream) {
    int rc = branch_args_ok("conv1d_attention", dtype, B, T, D, H, ldx, ldo);
    if (rc) return rc;
    if (kernel_size < 1) return set_error(CONVNN_E_INVALID, "conv1d_attention: kernel_size must be positive");
    REQUIRE_PTR(x); REQUIRE_PTR(w_x); REQUIRE_PTR(w_conv); REQUIRE_PTR(w_o); REQUIRE_PTR(out); REQUIRE_PTR(workspace);
    if (!aligned16(workspace)) return set_error(CONVNN_E_ALIGN, "workspace must be 16-byte aligned");
    const size_t need = convnn_b200_conv1d_attention_workspace_bytes(dtype, B, T, D, kernel_size);
    if (workspace_bytes < need)
        return set_error(CONVNN_E_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes, need);
    if ((rc = check_device())) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t elt = dtype == CONVNN_F32 ? 4 : 2, part = up256((size_t)B * T * D * elt);
    char* ws = static_cast<char*>(workspace);
    void *y = ws, *o = ws + part, *merged = ws + 2 * part, *unfold = ws + 3 * part;
    const long long M = (long long)B * T;
    if ((rc = convnn_b200_linear(dtype, x, ldx, w_x, b_x, nullptr, 0, y, D, M, D, D, 0, stream))) return rc;
    if ((rc = launch_conv1d_heads(dtype, y, w_conv, b_conv, o, unfold, B, T, H, D / H, kernel_size, st))) return rc;
    // the reference reads the per-head (T, d_k) block back as (d_k, T) for every H (layers.py:487-489, 499)
    if ((rc = launch_merge_heads(dtype, o, merged, B, T, H, D / H, st))) return rc;
    return convnn_b200_linear(dtype, merged, D, w_o, b_o, nullptr, 0, out, ldo, M, D, D, 0, stream);
}

}  // extern "C"
