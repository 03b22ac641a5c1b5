// Shared definitions of the Q8_0 kernels: the block layout, the exact dequantisation, and
// thin wrappers over the sm_100a PTX instructions the kernels issue (mbarrier, bulk tensor
// copies, tcgen05 tensor memory and MMA).
//
// Layout (reference: cuda/model/matrix.cuh:6-7,26,77-82; ptx/gemv_q8.ptx:12-13): a weight
// tensor w[n][k] is rows of k/32 blocks; one block is 34 bytes = little-endian binary16
// scale d followed by 32 signed bytes q.  The dequantised weight is half(float(q)*float(d)),
// one rounding (cuda/model/matrix.cuh:413-422).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "q8_store.cuh"


// Bits of the device status word that kernels raise instead of hanging.
#define Q8_DEV_BARRIER_TIMEOUT 1u /* a wait on a shared-memory barrier ran out */
#define Q8_DEV_FLAG_TIMEOUT 2u    /* a wait on another block's partial sum ran out */

// The single instructions behind inline PTX.  A build for the tests' host emulation
// (-DQ8_HOST_EMULATION) takes host stand-ins of the same names from its own include path.
#ifdef Q8_HOST_EMULATION
#include "q8_ptx_emu.cuh"
#else
#include "q8_ptx.cuh"
#endif

namespace q8 {

// ---------------------------------------------------------------------------------------
// Exact dequantisation of packed bytes.
//
// A signed byte q becomes the half 1024 + (q + 128) by placing (q ^ 0x80) under the
// exponent byte 0x64; taking 1152 away is exact, and one half multiply by the scale gives
// half(q * d) with a single rounding to nearest even, subnormal results kept - the same
// value as rounding the (exact) float product.
// ---------------------------------------------------------------------------------------

// Two weights from the low (HIGH = 0) or high (HIGH = 1) half of a word whose bytes were
// already xor-ed with 0x80; d2 holds the scale in both halves.
template <int HIGH>
__device__ __forceinline__ uint32_t dequant_pair(uint32_t flipped, __half2 d2)
{
    uint32_t magic = prmt(flipped, 0x64646464u, HIGH ? 0x4342u : 0x4140u);
    __half2 v = *reinterpret_cast<__half2 *>(&magic);
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480)); // 1152.0
    v = __hmul2(__hsub2(v, bias), d2);
    return *reinterpret_cast<uint32_t *>(&v);
}

// The same two weights as bfloat16: float(q) * float(d) is exact in float, so the pack is the
// single rounding bfloat16(q * d).  Used where the activations are bfloat16, because one MMA
// takes both operands in one 16-bit format.
template <int HIGH>
__device__ __forceinline__ uint32_t dequant_pair_bf16(uint32_t flipped, float d)
{
    uint32_t magic = prmt(flipped, 0x64646464u, HIGH ? 0x4342u : 0x4140u);
    __half2 v = *reinterpret_cast<__half2 *>(&magic);
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480)); // 1152.0
    float2 q = __half22float2(__hsub2(v, bias));
    return cvt_bf16x2_rn(q.y * d, q.x * d);
}

// Two bfloat16 values in one word become two binary16 values (same rule as below).
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t w)
{
    const float lo = __uint_as_float(w << 16);
    const float hi = __uint_as_float(w & 0xFFFF0000u);
    return cvt_f16x2_rn_sat(hi, lo);
}

// Eight bfloat16 values in shared memory become eight binary16 values in place.  Every
// bfloat16 of magnitude between 2^-14 and 65504 converts exactly; larger ones saturate to the
// largest half, smaller ones round to the half subnormals.
__device__ __forceinline__ void bf16_chunk_to_f16_inplace(uint32_t addr)
{
    uint32_t w[4];
    ld_shared_v4(addr, w[0], w[1], w[2], w[3]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float lo = __uint_as_float(w[i] << 16);
        float hi = __uint_as_float(w[i] & 0xFFFF0000u);
        w[i] = cvt_f16x2_rn_sat(hi, lo);
    }
    st_shared_v4(addr, w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ __half dequant_one(int q, __half d)
{
    return __float2half_rn((float)q * __half2float(d));
}

// ---------------------------------------------------------------------------------------
// Shared-memory barriers.
// ---------------------------------------------------------------------------------------

// Every wait is bounded.  When the bound runs out the waiter raises `*abort_flag` (shared)
// and the device status word, and the caller leaves its loop; the kernel then runs to its
// end with a wrong result rather than holding the GPU.
#define Q8_WAIT_CYCLES 4000000000ll /* about two seconds of SM clock */

// Out of line on purpose: a kernel has dozens of waits, and a short launch fetches its code cold
// at its start and again at its end, so the call sites have to stay small.
static __device__ __noinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                              unsigned int *status)
{
    // The common case: the phase completes within a few thousand polls; no clock is read.
#pragma unroll 1
    for (uint32_t spin = 0; spin < 4096u; ++spin) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
    }
    const long long begin = clock64();
#pragma unroll 1
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if ((spin & 255u) == 0u) {
            if (*abort_flag != 0u) {
                return false;
            }
            if (clock64() - begin > Q8_WAIT_CYCLES) {
                break;
            }
        }
    }
    *abort_flag = 1u;
    if (status != nullptr) {
        atomicOr(status, Q8_DEV_BARRIER_TIMEOUT);
    }
    return false;
}


// The same wait for the hot loops (the converters, which hold a row of raw bytes in registers
// across it): the polls are inline, so that no call - and with it no save and restore of the
// live registers through local memory - lies on the path that is taken every time.
__device__ __forceinline__ bool mbar_wait_hot(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                              unsigned int *status)
{
#pragma unroll 1
    for (uint32_t spin = 0; spin < 64u; ++spin) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
    }
    return mbar_wait(bar, parity, abort_flag, status);
}

// ---------------------------------------------------------------------------------------
// Bulk tensor copies (TMA), global -> shared, no multicast.
// ---------------------------------------------------------------------------------------

// ---------------------------------------------------------------------------------------
// Tensor memory and the fifth-generation tensor core.
// ---------------------------------------------------------------------------------------

// Shared-memory operand descriptor, K-major rows of 128 bytes with the 128-byte swizzle:
// rows 128 bytes apart, groups of 8 rows 1024 bytes apart, 16-byte chunk c of row r stored
// at chunk c ^ (r & 7).  The buffer starts on a 1024-byte boundary.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr)
{
    uint64_t desc = 0;
    desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);       // start address, 16-byte units
    desc |= (uint64_t)1u << 16;                            // leading byte offset (unused here)
    desc |= (uint64_t)(1024u >> 4) << 32;                  // stride between 8-row groups
    desc |= (uint64_t)1u << 46;                            // descriptor version of sm_100
    desc |= (uint64_t)2u << 61;                            // 128-byte swizzle
    return desc;
}

// Instruction descriptor of kind::f16: float accumulator, both operands K-major.
// a_bf16 / b_bf16 select bfloat16 instead of binary16 for that operand.
__host__ __device__ inline uint32_t umma_idesc(unsigned int m, unsigned int n, unsigned int a_bf16,
                                               unsigned int b_bf16)
{
    uint32_t d = 0;
    d |= 1u << 4;               // accumulator format: float
    d |= (a_bf16 & 1u) << 7;    // A format
    d |= (b_bf16 & 1u) << 10;   // B format
    d |= (n >> 3) << 17;        // N, in units of 8
    d |= (m >> 4) << 24;        // M, in units of 16
    return d;
}

} // namespace q8
