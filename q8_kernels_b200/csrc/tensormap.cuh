// Host-side construction of TMA tensor maps for byte matrices.  The driver's
// encode function is resolved through the runtime, so the library has no
// link-time dependency on libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace q8k {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Tensor map over a byte tensor of `rank` dims (dims[0] innermost, contiguous;
// strides_bytes[i] is the byte stride of dims[i+1]) loaded in boxes of box[].
// Out-of-range elements of a box read as zero.
inline int make_byte_tensor_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                                const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes,
                                const char* what) {
    EncodeTiledFn encode = get_encode_tiled();
    Q8K_REQUIRE(encode != nullptr, Q8K_ERR_CUDA, "%s: cuTensorMapEncodeTiled is not available from this driver", what);
    cuuint64_t gdim[5];
    cuuint64_t gstride[5];
    cuuint32_t bdim[5];
    cuuint32_t estride[5];
    for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bdim[i] = box[i]; estride[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) gstride[i] = strides_bytes[i];
    const CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : swizzle_bytes == 64  ? CU_TENSOR_MAP_SWIZZLE_64B
                                : swizzle_bytes == 32  ? CU_TENSOR_MAP_SWIZZLE_32B
                                                       : CU_TENSOR_MAP_SWIZZLE_NONE;
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, (cuuint32_t)rank, const_cast<void*>(base), gdim,
                              gstride, bdim, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    Q8K_REQUIRE(r == CUDA_SUCCESS, Q8K_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, (int)r);
    return Q8K_OK;
}

}  // namespace q8k
