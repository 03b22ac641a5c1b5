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

namespace q8 {

// ---------------------------------------------------------------------------------------
// Exact dequantisation of packed bytes.
//
// A signed byte q becomes the half 1024 + (q + 128) by placing (q ^ 0x80) under the
// exponent byte 0x64; taking 1152 away is exact, and one half multiply by the scale gives
// half(q * d) with a single rounding to nearest even, subnormal results kept - the same
// value as rounding the (exact) float product.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t out;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(a), "r"(b), "r"(sel));
    return out;
}

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
    uint32_t out;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(q.y * d), "f"(q.x * d));
    return out;
}

// Eight bfloat16 values in shared memory become eight binary16 values in place.  Every
// bfloat16 of magnitude between 2^-14 and 65504 converts exactly; larger ones saturate to the
// largest half, smaller ones round to the half subnormals.
__device__ __forceinline__ void bf16_chunk_to_f16_inplace(uint32_t addr)
{
    uint32_t w[4];
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                 : "r"(addr)
                 : "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float lo = __uint_as_float(w[i] << 16);
        float hi = __uint_as_float(w[i] & 0xFFFF0000u);
        asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(w[i]) : "f"(hi), "f"(lo));
    }
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3])
                 : "memory");
}

__device__ __forceinline__ __half dequant_one(int q, __half d)
{
    return __float2half_rn((float)q * __half2float(d));
}

// ---------------------------------------------------------------------------------------
// Shared-memory barriers.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}

// Every wait is bounded.  When the bound runs out the waiter raises `*abort_flag` (shared)
// and the device status word, and the caller leaves its loop; the kernel then runs to its
// end with a wrong result rather than holding the GPU.
#define Q8_WAIT_CYCLES 4000000000ll /* about two seconds of SM clock */

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          unsigned int *status)
{
    // The common case: the phase completes within a few thousand polls; no clock is read.
    for (uint32_t spin = 0; spin < 4096u; ++spin) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
    }
    const long long begin = clock64();
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

__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------
// Bulk tensor copies (TMA), global -> shared, no multicast.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void *tmap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tmap) : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, uint32_t bar, int c0, int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)tmap), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

// Ask L2 to fetch [addr, addr + bytes) from device memory; nothing waits for it.  Address and
// size are multiples of 16.
__device__ __forceinline__ void l2_prefetch_bulk(const void *addr, uint32_t bytes)
{
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(addr), "r"(bytes) : "memory");
}

// ---------------------------------------------------------------------------------------
// Tensor memory and the fifth-generation tensor core.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t columns)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result),
                 "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem], one 128 x N x 16 step, 16-bit operands, float sums.
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The same with A read from tensor memory: lane = row of A, 8 columns hold the 16 halves of a
// row, lower k in the lower half of a column.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrive on a barrier when every MMA this thread issued before has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// 32 lanes x 32 columns of 32-bit values: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t *v)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
          "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
          "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
          "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t *v)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
          "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

// 32 lanes x 32 columns: thread t of the warp writes lane (base lane + t).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t *v)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_wait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

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

// Programmatic dependent launch: let the next kernel on the stream start its blocks early,
// and wait (in that next kernel) until everything before it on the stream has finished and
// its memory is visible.  Both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void grid_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const unsigned int *p)
{
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_gpu(unsigned int *p, uint32_t v)
{
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

} // namespace q8
