// float32 instantiations of the SIMT similarity + top-K kernel.
#include "sim_topk_simt.cuh"

namespace convnn {
int launch_sim_topk_simt_f32(const convnn_desc* d, const Dims& dm, const void* q, const void* k,
                             const float* qstat, const float* kstat, const int32_t* cand, int32_t* idx,
                             float* val, cudaStream_t st) {
    return simt_topk::dispatch<float>(d, dm, q, k, qstat, kstat, cand, idx, val, st);
}
}  // namespace convnn
