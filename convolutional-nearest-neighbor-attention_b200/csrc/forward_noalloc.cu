// convnn_b200_forward_noalloc: the whole-layer forward for callers that cannot hand the
// library a workspace because they are not allowed to allocate device memory at the point
// of the call -- a latency-critical serving loop where cudaMalloc would synchronise the
// device, plugins of a host runtime that owns the allocator and exposes no allocation hook,
// and processes on a GPU whose memory has been fully handed out up front.  Instead of a caller-provided workspace, the layer's
// intermediates (q, k, v, statistics, neighbour lists, conv output, stage scratch) live in
// one fixed array that is part of the library's device image.
#include <mutex>

#include "common.cuh"

namespace convnn {
namespace {

// The array belongs to this translation unit's CUDA module.  The runtime loads modules lazily by
// default, so a GPU reserves these bytes when the module is first touched on it -- by the address
// lookup below -- and keeps them until the process exits.
constexpr size_t kStaticWorkspaceBytes = 32u << 20;
static __device__ __align__(256) unsigned char g_static_workspace[kStaticWorkspaceBytes];

// In host code `g_static_workspace` is only a handle for the runtime, not a device address;
// the address a kernel can use has to be asked for, per device, with that device current.
std::mutex g_ws_mutex;
void* g_ws_ptr[64] = {nullptr};

int static_workspace(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return set_error(CONVNN_E_DEVICE, "forward_noalloc: no usable current device");
    }
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    if (!g_ws_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_workspace);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return set_error(CONVNN_E_CUDA, "forward_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        }
        g_ws_ptr[dev] = p;
    }
    *out = g_ws_ptr[dev];
    return CONVNN_OK;
}

}  // namespace

// capi.cu: the current device must be an sm_100 part (cached per device).
int check_device_is_sm100();
}  // namespace convnn

extern "C" {

// Also the warm-up: resolving the address here, at start-up, is what makes the GPU reserve the
// array, so that no later forward has to (see the header).  The capacity is returned whether or
// not the lookup worked; a failed lookup is reported by the first forward.
size_t convnn_b200_noalloc_capacity(void) {
    if (convnn::check_device_is_sm100() == CONVNN_OK) {
        void* ws = nullptr;
        (void)convnn::static_workspace(&ws);
    }
    return convnn::kStaticWorkspaceBytes;
}

int convnn_b200_forward_noalloc(const convnn_desc* d, const void* x, int64_t ldx, const void* w_qkv,
                                const void* w_conv, const void* w_pw, const void* w_o, const int32_t* cand,
                                const void* residual, int64_t ldr, void* out, int64_t ldo, void* stream) {
    const size_t need = convnn_b200_workspace_bytes(d);
    if (need == 0) return convnn_b200_head_channels(d) < 0 ? convnn_b200_head_channels(d) : CONVNN_E_INVALID;
    if (need > convnn::kStaticWorkspaceBytes)
        return convnn::set_error(CONVNN_E_WORKSPACE,
                                 "forward_noalloc: this shape needs %zu bytes of intermediates but the built-in "
                                 "workspace holds %zu; use convnn_b200_forward with a caller-provided workspace",
                                 need, convnn::kStaticWorkspaceBytes);
    void* ws = nullptr;
    int rc = convnn::check_device_is_sm100();         // a foreign GPU is a device error, not a CUDA error
    if (rc) return rc;
    rc = convnn::static_workspace(&ws);
    if (rc) return rc;
    return convnn_b200_forward(d, x, ldx, w_qkv, w_conv, w_pw, w_o, cand, residual, ldr, out, ldo, ws,
                               convnn::kStaticWorkspaceBytes, stream);
}

}  // extern "C"
