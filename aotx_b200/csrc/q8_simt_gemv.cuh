// The any-shape Q8_0 product on the ordinary cores (plain and with the fused stores).  No inline
// PTX here, so the tests' warp emulator can run these kernels on the host (tests/simt_emu.cu).
#pragma once

#include "q8_launch.h"
#include "q8_store.cuh"

namespace q8 {

// ---------------------------------------------------------------------------------------
// Two activations from one 32-bit word.
// ---------------------------------------------------------------------------------------
template <typename XT>
__device__ __forceinline__ float2 unpack2(uint32_t word);

template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t word)
{
    return __half22float2(*reinterpret_cast<__half2 *>(&word));
}

template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t word)
{
    return make_float2(__uint_as_float(word << 16), __uint_as_float(word & 0xFFFF0000u));
}

#define Q8_SIMT_TAKE 8u
#define Q8_SIMT_WARPS 8u

// One warp, one row of w, up to 8 rows of x: the lanes take blocks 32 apart, keep the product
// of a weight and its scale in float like the reference's memory-bound kernel
// (cuda/model/matrix.cuh:498-512), and add their parts with a shuffle tree.
template <typename XT>
__device__ __forceinline__ void simt_row(const unsigned char *__restrict__ row, unsigned int k,
                                         const XT *__restrict__ x, size_t x_stride, unsigned int take,
                                         float *acc)
{
    unsigned int lane = threadIdx.x & 31u;
    unsigned int blocks = k / Q8_BLOCK;
#pragma unroll
    for (unsigned int t = 0; t < Q8_SIMT_TAKE; ++t) {
        acc[t] = 0.0f;
    }
    for (unsigned int b = lane; b < blocks; b += 32u) {
        const unsigned char *one = row + (size_t)b * Q8_BLOCK_BYTES;
        float d = __half2float(*reinterpret_cast<const __half *>(one));
        const unsigned short *src = reinterpret_cast<const unsigned short *>(one + 2u);
#pragma unroll 4
        for (unsigned int i = 0; i < 16u; ++i) {
            unsigned int v = src[i];
            float w0 = (float)(int)(signed char)(v & 0xFFu) * d;
            float w1 = (float)(int)(signed char)(v >> 8) * d;
#pragma unroll
            for (unsigned int t = 0; t < Q8_SIMT_TAKE; ++t) {
                if (t < take) {
                    const uint32_t *xr = reinterpret_cast<const uint32_t *>(x + (size_t)t * x_stride
                                                                            + (size_t)b * Q8_BLOCK);
                    float2 xv = unpack2<XT>(xr[i]);
                    acc[t] = fmaf(w0, xv.x, acc[t]);
                    acc[t] = fmaf(w1, xv.y, acc[t]);
                }
            }
        }
    }
#pragma unroll
    for (unsigned int step = 16u; step > 0u; step >>= 1) {
#pragma unroll
        for (unsigned int t = 0; t < Q8_SIMT_TAKE; ++t) {
            acc[t] += __shfl_down_sync(0xFFFFFFFFu, acc[t], step);
        }
    }
}

// y[i][j] = sum_c x[i][c] * w[j][c] for i < m, j < n; nothing else is written.  The batch m is
// the smaller of `m_max` and the device word `m_dev` when that is given.
template <typename XT, typename YT>
__global__ void __launch_bounds__(Q8_SIMT_WARPS * 32u)
q8_gemv_simt_kernel(const unsigned char *__restrict__ w, unsigned int n, unsigned int k,
                    const XT *__restrict__ x, unsigned int m_max, const unsigned int *m_dev,
                    YT *__restrict__ y)
{
    unsigned int m = m_max;
    if (m_dev != nullptr) {
        unsigned int live = *m_dev;
        m = live < m_max ? live : m_max;
    }
    unsigned int lane = threadIdx.x & 31u;
    unsigned int warp = threadIdx.x >> 5;
    unsigned long long stride = row_bytes(k);
    for (unsigned int j = blockIdx.x * Q8_SIMT_WARPS + warp; j < n; j += gridDim.x * Q8_SIMT_WARPS) {
        const unsigned char *row = w + stride * j;
        for (unsigned int m0 = 0; m0 < m; m0 += Q8_SIMT_TAKE) {
            unsigned int take = m - m0 < Q8_SIMT_TAKE ? m - m0 : Q8_SIMT_TAKE;
            float acc[Q8_SIMT_TAKE];
            simt_row<XT>(row, k, x + (size_t)m0 * k, k, take, acc);
            if (lane == 0u) {
#pragma unroll
                for (unsigned int t = 0; t < Q8_SIMT_TAKE; ++t) {
                    if (t < take) {
                        store_out<YT>(y, (size_t)(m0 + t) * n + j, acc[t]);
                    }
                }
            }
        }
    }
}

// The same product with one of the two fused stores (q8_launch.h): the sum is added to the
// float that y holds, or the sums of rows 2p and 2p+1 of w (gate and up of column p) leave as
// silu(gate) * up in column p of a y that is n / 2 wide (arithmetic of
// cuda/model/norm.cu:78-105).  One warp takes one output column.
template <typename XT, typename YT>
__global__ void __launch_bounds__(Q8_SIMT_WARPS * 32u)
q8_gemv_simt_fused_kernel(const unsigned char *__restrict__ w, unsigned int n, unsigned int k,
                          const XT *__restrict__ x, unsigned int m_max, const unsigned int *m_dev,
                          YT *__restrict__ y, unsigned int epilogue)
{
    unsigned int m = m_max;
    if (m_dev != nullptr) {
        unsigned int live = *m_dev;
        m = live < m_max ? live : m_max;
    }
    const unsigned int lane = threadIdx.x & 31u;
    const unsigned int warp = threadIdx.x >> 5;
    const unsigned long long stride = row_bytes(k);
    const bool swiglu = epilogue == kEpilogueSwiglu;
    const unsigned int columns = swiglu ? n / 2u : n;
    for (unsigned int p = blockIdx.x * Q8_SIMT_WARPS + warp; p < columns; p += gridDim.x * Q8_SIMT_WARPS) {
        const unsigned char *row = w + stride * (swiglu ? 2ull * p : (unsigned long long)p);
        for (unsigned int m0 = 0; m0 < m; m0 += Q8_SIMT_TAKE) {
            const unsigned int take = m - m0 < Q8_SIMT_TAKE ? m - m0 : Q8_SIMT_TAKE;
            float first[Q8_SIMT_TAKE];
            float second[Q8_SIMT_TAKE];
            simt_row<XT>(row, k, x + (size_t)m0 * k, k, take, first);
            if (swiglu) {
                simt_row<XT>(row + stride, k, x + (size_t)m0 * k, k, take, second);
            }
            if (lane == 0u) {
#pragma unroll
                for (unsigned int t = 0; t < Q8_SIMT_TAKE; ++t) {
                    if (t < take) {
                        const size_t at = (size_t)(m0 + t) * columns + p;
                        if (swiglu) {
                            const float unit = first[t] / (1.0f + expf(-first[t]));
                            store_out<YT>(y, at, unit * second[t]);
                        } else {
                            float *sum = reinterpret_cast<float *>(y) + at;
                            *sum = *sum + first[t];
                        }
                    }
                }
            }
        }
    }
}

} // namespace q8
