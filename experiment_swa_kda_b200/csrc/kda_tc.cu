// Tensor-core lane (K = V = 128, bf16 operands, fp32 accumulation and state): host-side TMA tensor maps shared by
// the tcgen05 kernels.
//
// The driver entry point cuTensorMapEncodeTiled is fetched through the runtime, so the library links against
// nothing but libcudart and libcuda's loader stub.

#include "common.cuh"
#include "simt_ws.cuh"
#include "tc_common.cuh"
#include "tc_ws.cuh"

namespace kda {
namespace tc {

// ---------------------------------------------------------------------------------------------
// host: tensor maps
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = (EncodeFn)p;
    }
    return fn;
}

// 2-D bf16 row-major tensor [rows][cols]; box = box_cols x box_rows; 128-byte swizzle (box_cols must be 64).
int make_map_bf16(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows) {
    EncodeFn enc = encode_fn();
    if (!enc) return KDA_ERR_CUDA;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t es[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_ERROR_INVALID_CONTEXT) {
        // a host thread that has made no runtime call yet (e.g. an autograd worker) has no context bound:
        // bind the current device's primary context and try once more
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess && cudaFree(nullptr) == cudaSuccess)
            r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS && getenv("KDA_B200_VERBOSE"))
        fprintf(stderr, "libkda_b200: cuTensorMapEncodeTiled failed (%d): ptr %p rows %llu cols %llu box %u x %u\n", (int)r, ptr,
                (unsigned long long)rows, (unsigned long long)cols, box_cols, box_rows);
    return r == CUDA_SUCCESS ? KDA_OK : KDA_ERR_CUDA;
}

}  // namespace tc
}  // namespace kda
