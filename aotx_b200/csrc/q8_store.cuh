// The parts of the common header that hold no inline PTX: block constants, the row stride and the
// typed store of a result.  Kernels on the ordinary cores include only this, so that they can
// also be compiled for the host by the tests' warp emulator (tests/simt_emu.cu).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define Q8_BLOCK 32u
#define Q8_BLOCK_BYTES 34u
#define Q8_TYPE_Q8_0 8u /* cuda/model/model.cuh:31 */

namespace q8 {

__host__ __device__ inline unsigned long long row_bytes(unsigned int k)
{
    return (unsigned long long)(k / Q8_BLOCK) * Q8_BLOCK_BYTES;
}

template <typename T>
__device__ __forceinline__ void store_out(T *y, size_t at, float v);

template <>
__device__ __forceinline__ void store_out<float>(float *y, size_t at, float v)
{
    y[at] = v;
}

template <>
__device__ __forceinline__ void store_out<__half>(__half *y, size_t at, float v)
{
    y[at] = __float2half_rn(v);
}

template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16 *y, size_t at, float v)
{
    y[at] = __float2bfloat16_rn(v);
}

} // namespace q8
