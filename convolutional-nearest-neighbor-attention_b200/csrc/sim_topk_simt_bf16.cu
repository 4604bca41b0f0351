// bfloat16 instantiations of the SIMT similarity + top-K kernel.
#include "sim_topk_simt.cuh"

namespace convnn {
int launch_sim_topk_simt_bf16(const convnn_desc* d, const Dims& dm, const void* q, const void* k,
                              const float* qstat, const float* kstat, const int32_t* cand, int32_t* idx,
                              float* val, cudaStream_t st) {
    return simt_topk::dispatch<__nv_bfloat16>(d, dm, q, k, qstat, kstat, cand, idx, val, st);
}
}  // namespace convnn
