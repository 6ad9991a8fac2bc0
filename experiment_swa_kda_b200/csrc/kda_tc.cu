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

// ---------------------------------------------------------------------------------------------
// self-test of the bounded wait every tensor-core-lane kernel relies on: one warp waits, with a short limit, on a
// barrier that nothing ever arrives at.  The wait must give up, record its code in the status word and let the kernel
// return normally (no trap, no unbounded spin), which is how a lost TMA completion or UMMA commit would surface.
// ---------------------------------------------------------------------------------------------
constexpr int kSelftestWaitCode = 99;

__global__ void bounded_wait_selftest_kernel(int* status, uint32_t limit, int* returned) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    const bool ok = mbar_wait(&bar, 0, status, kSelftestWaitCode, limit);
    if (threadIdx.x == 0) *returned = ok ? 1 : 2;      // 2: the wait ran out and the thread carried on
}

}  // namespace tc
}  // namespace kda

extern "C" int kda_selftest_bounded_wait(int32_t* device_words, uint32_t poll_limit, void* stream) {
    if (!device_words) return KDA_ERR_NULL;
    if (poll_limit == 0 || poll_limit > 1000000u) return KDA_ERR_BAD_SHAPE;      // keep the self-test short
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemsetAsync(device_words, 0, 2 * sizeof(int32_t), st) != cudaSuccess) return KDA_ERR_CUDA;
    KDA_LAUNCH("bounded_wait_selftest_kernel", st,
               kda::tc::bounded_wait_selftest_kernel<<<1, 32, 0, st>>>(device_words, poll_limit, device_words + 1));
    return kda::launch_status();
}
