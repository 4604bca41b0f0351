// Host-side construction of TMA tensor maps.  cuTensorMapEncodeTiled is a pure host
// function of the driver; it is resolved at run time through the CUDA runtime so the
// library does not link against libcuda.
#include <mutex>

#include "common.cuh"
#include "sm100.cuh"

namespace convnn {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn resolve_encode() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    });
    return fn;
}
}  // namespace

static bool encode_tensor_map(CUtensorMap* out, CUtensorMapDataType type, const void* base, int rank, const uint64_t* dims,
                              const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes) {
    EncodeTiledFn fn = resolve_encode();
    if (!fn) {
        set_error(CONVNN_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
        return false;
    }
    cuuint64_t gdims[5], gstr[4];
    cuuint32_t gbox[5], estr[5];
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        estr[i] = 1;
        if (i + 1 < rank) gstr[i] = strides_bytes[i];
    }
    CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle_bytes == 64  ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle_bytes == 32  ? CU_TENSOR_MAP_SWIZZLE_32B
                                                 : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = fn(out, type, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstr,
                    gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error(CONVNN_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu %llu ..., box %u %u ...)",
                  (int)r, rank, (unsigned long long)dims[0], (unsigned long long)dims[1], box[0], box[1]);
        return false;
    }
    return true;
}

bool encode_tensor_map_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                            const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes) {
    return encode_tensor_map(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides_bytes, box, swizzle_bytes);
}

// float32 elements, no swizzle (the row moments of the pre-norm fold)
bool encode_tensor_map_f32(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box) {
    return encode_tensor_map(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides_bytes, box, 0);
}

}  // namespace convnn
