// Dequantisation and the product for every block type of the model file, on the ordinary cores.
// Q8_0 has its own kernels (q8_stream.cu, q8_simt.cu); the other eleven types the reference's
// kernels read (cuda/model/dequant.cu:26-70, cuda/model/gemv.cuh:147-195, cuda/model/gemm.cuh:199-239)
// go through the one decoder of q_blocks.cuh here, so that the entry points serve whatever type
// a model file holds.  These kernels are written for coverage and exactness first: a lane
// decodes a run of 32 weights into registers once and uses it for up to 8 rows of x.
#include "q8_launch.h"
#include "q8_store.cuh"
#include "q_blocks.cuh"

namespace q8 {

#define QG_WARPS 8u
#define QG_TAKE 8u

// out[r][c] = half(weight) for rows [first, first + rows): one thread per run of 32 weights.
__global__ void __launch_bounds__(256)
q_dequant_any_kernel(const unsigned char *__restrict__ w, uint32_t type, uint32_t k, uint32_t first_row,
                     uint32_t rows, __half *__restrict__ out)
{
    const unsigned long long stride = block_row_bytes(type, k);
    const uint32_t runs = k / 32u;
    const unsigned long long total = (unsigned long long)rows * runs;
    for (unsigned long long at = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; at < total;
         at += (unsigned long long)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(at / runs);
        const uint32_t run = (uint32_t)(at % runs);
        float values[32];
        decode_run(type, w + stride * (first_row + r), run, values);
        __half *dst = out + (size_t)r * k + (size_t)run * 32u;
#pragma unroll
        for (uint32_t i = 0; i < 32u; i += 2u) {
            *reinterpret_cast<__half2 *>(dst + i) = __floats2half2_rn(values[i], values[i + 1u]);
        }
    }
}

template <typename XT>
__device__ __forceinline__ float x_value(const XT *x);

template <>
__device__ __forceinline__ float x_value<__half>(const __half *x)
{
    return __half2float(*x);
}

template <>
__device__ __forceinline__ float x_value<__nv_bfloat16>(const __nv_bfloat16 *x)
{
    return __bfloat162float(*x);
}

// eight activations from one 16-byte load
template <typename XT>
__device__ __forceinline__ void x_eight(const uint4 &packed, float *out);

template <>
__device__ __forceinline__ void x_eight<__half>(const uint4 &packed, float *out)
{
    const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 pair = __half22float2(*reinterpret_cast<const __half2 *>(&words[i]));
        out[2 * i] = pair.x;
        out[2 * i + 1] = pair.y;
    }
}

template <>
__device__ __forceinline__ void x_eight<__nv_bfloat16>(const uint4 &packed, float *out)
{
    const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(words[i] << 16);
        out[2 * i + 1] = __uint_as_float(words[i] & 0xFFFF0000u);
    }
}

// The rows of one warp for one block type.  TYPE is a constant here, so the decoder's switch
// folds to the one reader; the activations come as 16-byte loads when x allows it.
template <uint32_t TYPE, typename XT, typename YT>
__device__ __forceinline__ void gemv_rows(const unsigned char *__restrict__ w, uint32_t n, uint32_t k,
                                          const XT *__restrict__ x, uint32_t m, YT *__restrict__ y, bool wide_x)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = threadIdx.x >> 5;
    const unsigned long long stride = block_row_bytes(TYPE, k);
    const uint32_t runs = k / 32u;
    for (uint32_t j = blockIdx.x * QG_WARPS + warp; j < n; j += gridDim.x * QG_WARPS) {
        const unsigned char *row = w + stride * j;
        for (uint32_t m0 = 0; m0 < m; m0 += QG_TAKE) {
            const uint32_t take = m - m0 < QG_TAKE ? m - m0 : QG_TAKE;
            float acc[QG_TAKE];
#pragma unroll
            for (uint32_t t = 0; t < QG_TAKE; ++t) {
                acc[t] = 0.0f;
            }
            for (uint32_t run = lane; run < runs; run += 32u) {
                float values[32];
                decode_run(TYPE, row, run, values);
#pragma unroll
                for (uint32_t t = 0; t < QG_TAKE; ++t) {
                    if (t < take) {
                        const XT *xr = x + (size_t)(m0 + t) * k + (size_t)run * 32u;
                        float sum = acc[t];
                        if (wide_x) {
                            const uint4 *wide = reinterpret_cast<const uint4 *>(xr);
#pragma unroll
                            for (uint32_t q = 0; q < 4u; ++q) {
                                float eight[8];
                                x_eight<XT>(wide[q], eight);
#pragma unroll
                                for (uint32_t i = 0; i < 8u; ++i) {
                                    sum = fmaf(values[8u * q + i], eight[i], sum);
                                }
                            }
                        } else {
#pragma unroll
                            for (uint32_t i = 0; i < 32u; ++i) {
                                sum = fmaf(values[i], x_value<XT>(xr + i), sum);
                            }
                        }
                        acc[t] = sum;
                    }
                }
            }
#pragma unroll
            for (uint32_t step = 16u; step > 0u; step >>= 1) {
#pragma unroll
                for (uint32_t t = 0; t < QG_TAKE; ++t) {
                    acc[t] += __shfl_down_sync(0xFFFFFFFFu, acc[t], step);
                }
            }
            if (lane == 0u) {
#pragma unroll
                for (uint32_t t = 0; t < QG_TAKE; ++t) {
                    if (t < take) {
                        store_out<YT>(y, (size_t)(m0 + t) * n + j, acc[t]);
                    }
                }
            }
        }
    }
}

// One warp, one row of w, up to 8 rows of x: lanes take runs of 32 weights 32 apart, keep the
// float value of a weight (no rounding to half, like the reference's memory-bound kernel,
// cuda/model/matrix.cuh:493-670), and add their parts with a shuffle tree.
template <typename XT, typename YT>
__global__ void __launch_bounds__(QG_WARPS * 32u)
q_gemv_any_kernel(const unsigned char *__restrict__ w, uint32_t type, uint32_t n, uint32_t k,
                  const XT *__restrict__ x, uint32_t m_max, const unsigned int *m_dev, YT *__restrict__ y,
                  uint32_t wide_x)
{
    uint32_t m = m_max;
    if (m_dev != nullptr) {
        const uint32_t live = *m_dev;
        m = live < m_max ? live : m_max;
    }
    const bool wide = wide_x != 0u;
    switch (type) {
    case kTypeF32: gemv_rows<kTypeF32, XT, YT>(w, n, k, x, m, y, wide); break;
    case kTypeF16: gemv_rows<kTypeF16, XT, YT>(w, n, k, x, m, y, wide); break;
    case kTypeQ4_0: gemv_rows<kTypeQ4_0, XT, YT>(w, n, k, x, m, y, wide); break;
    case kTypeQ4_1: gemv_rows<kTypeQ4_1, XT, YT>(w, n, k, x, m, y, wide); break;
    case kTypeQ5_0: gemv_rows<kTypeQ5_0, XT, YT>(w, n, k, x, m, y, wide); break;
    case kTypeQ5_1: gemv_rows<kTypeQ5_1, XT, YT>(w, n, k, x, m, y, wide); break;
    case kTypeQ8_0: gemv_rows<kTypeQ8_0, XT, YT>(w, n, k, x, m, y, wide); break;
    case kTypeQ2_K: gemv_rows<kTypeQ2_K, XT, YT>(w, n, k, x, m, y, wide); break;
    case kTypeQ3_K: gemv_rows<kTypeQ3_K, XT, YT>(w, n, k, x, m, y, wide); break;
    case kTypeQ4_K: gemv_rows<kTypeQ4_K, XT, YT>(w, n, k, x, m, y, wide); break;
    case kTypeQ5_K: gemv_rows<kTypeQ5_K, XT, YT>(w, n, k, x, m, y, wide); break;
    case kTypeQ6_K: gemv_rows<kTypeQ6_K, XT, YT>(w, n, k, x, m, y, wide); break;
    default: break; // a type without a layout writes nothing
    }
}

bool block_type_known(unsigned int type)
{
    uint32_t weights = 0, bytes = 0;
    return block_shape(type, &weights, &bytes);
}

unsigned int block_type_run(unsigned int type)
{
    return block_run(type);
}

cudaError_t launch_dequant_any(cudaStream_t stream, const void *w, unsigned int type, unsigned int k,
                               unsigned int first_row, unsigned int rows, void *out)
{
    if (rows == 0u) {
        return cudaSuccess;
    }
    const unsigned long long total = (unsigned long long)rows * (k / 32u);
    unsigned long long want = (total + 255ull) / 256ull;
    const unsigned int grid = want < 148ull * 16ull ? (unsigned int)want : 148u * 16u;
    return launch_kernel(q_dequant_any_kernel, grid, 256, 0, stream, static_cast<const unsigned char *>(w), type, k,
                         first_row, rows, static_cast<__half *>(out));
}

template <typename XT, typename YT>
static cudaError_t launch_gemv_any_typed(cudaStream_t stream, const void *w, unsigned int type, unsigned int n,
                                         unsigned int k, const void *x, unsigned int m,
                                         const unsigned int *m_dev, void *y)
{
    const unsigned int want = (n + QG_WARPS - 1u) / QG_WARPS;
    const unsigned int grid = want < 148u * 8u ? want : 148u * 8u;
    // rows of x are k * 2 bytes, a multiple of 64: 16-byte loads need only an aligned base
    const uint32_t wide_x = (reinterpret_cast<uintptr_t>(x) & 15u) == 0u ? 1u : 0u;
    return launch_kernel(q_gemv_any_kernel<XT, YT>, grid, QG_WARPS * 32u, 0, stream,
                         static_cast<const unsigned char *>(w), type, n, k, static_cast<const XT *>(x), m, m_dev,
                         static_cast<YT *>(y), wide_x);
}

cudaError_t launch_gemv_any(cudaStream_t stream, const void *w, unsigned int type, unsigned int n,
                            unsigned int k, const void *x, int x_bf16, unsigned int m,
                            const unsigned int *m_dev, void *y, int y_dtype)
{
    if (n == 0u || m == 0u) {
        return cudaSuccess;
    }
#define QG_CASE(XT, YD, YT)                                                                       \
    if (y_dtype == (YD)) {                                                                       \
        return launch_gemv_any_typed<XT, YT>(stream, w, type, n, k, x, m, m_dev, y);             \
    }
    if (x_bf16) {
        QG_CASE(__nv_bfloat16, 0, float)
        QG_CASE(__nv_bfloat16, 1, __half)
        QG_CASE(__nv_bfloat16, 2, __nv_bfloat16)
    } else {
        QG_CASE(__half, 0, float)
        QG_CASE(__half, 1, __half)
        QG_CASE(__half, 2, __nv_bfloat16)
    }
#undef QG_CASE
    return cudaErrorInvalidValue;
}


} // namespace q8
