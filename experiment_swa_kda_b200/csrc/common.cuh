// Shared device/host helpers for the KDA kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "../../include/kda_b200.h"

namespace kda {

constexpr int kChunk = 64;   // tokens per chunk
constexpr int kLD = 68;      // padded leading dimension (floats) of a 64x64 shared-memory tile

__device__ __forceinline__ float ld_io(const void* p, size_t i, int bf16) {
    return bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i])
                : reinterpret_cast<const float*>(p)[i];
}
__device__ __forceinline__ void st_io(void* p, size_t i, int bf16, float x) {
    if (bf16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(x);
    else reinterpret_cast<float*>(p)[i] = x;
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Launch accounting (implemented in kda_api.cu): every kernel launch of the library goes through
// KDA_LAUNCH, which counts it and, when profiling is enabled, brackets it with CUDA events on the
// launching stream so a caller can read per-kernel device time.
namespace prof {
void begin(const char* name, cudaStream_t st);
void end(cudaStream_t st);
}  // namespace prof
#define KDA_LAUNCH(name, st, ...)      \
    do {                               \
        ::kda::prof::begin(name, st);  \
        __VA_ARGS__;                   \
        ::kda::prof::end(st);          \
    } while (0)

// Host-side launch check: returns a KDA_ERR_* code instead of throwing.
inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess && getenv("KDA_B200_VERBOSE")) fprintf(stderr, "libkda_b200: CUDA error: %s\n", cudaGetErrorString(e));
    return e == cudaSuccess ? KDA_OK : KDA_ERR_CUDA;
}

}  // namespace kda
