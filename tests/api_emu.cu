// The whole library on the host: every source of the product library compiled as host code
// around the stand-ins of tests/q8_ptx_emu.cuh, so that the C ABI of include/aotx_q8_b200.h can be
// called on a machine without a GPU.  "Device" memory is host memory (a pointer is a pointer),
// a stream is ignored, a launch runs the grid's blocks as host threads before it returns, and
// the device has AOTX_EMULATED_SMS multiprocessors (six unless set), so that grids stay small.
// What this adds to tests/stream_emu.cu, which calls the kernels with arguments the test driver
// fills in: here the library's own host code fills them in - argument checks and return codes,
// the choice of kernel, tensor maps, grids, scratch sets, workspaces, and
// product, the order of the launches of the routed-expert step.
//
// Built as a shared library by tests/test_api_emu.py.
#include "stream_emu.cu"

#include <cstdlib>

// ---- the rest of what the ordinary-core kernels use ------------------------------------------
namespace emu {

inline float shfl_down(float value, unsigned int delta)
{
    const unsigned int lane = thread_index.x % 32u;
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    warp->slot[lane] = bits;
    warp->barrier.wait();
    if (lane + delta < 32u) {
        bits = warp->slot[lane + delta];
    }
    warp->barrier.wait();
    std::memcpy(&value, &bits, 4);
    return value;
}

// one rounding each, never contracted into a fused multiply-add
inline float fmul_rn(float a, float b)
{
    volatile float product = a * b;
    return product;
}

inline float fadd_rn(float a, float b)
{
    volatile float sum = a + b;
    return sum;
}

} // namespace emu

#define __shfl_down_sync(mask, value, delta) emu::shfl_down((value), (delta))
#define __int_as_float(bits) emu::uint_as_float((uint32_t)(bits))
#define __fmul_rn(a, b) emu::fmul_rn((a), (b))
#define __fadd_rn(a, b) emu::fadd_rn((a), (b))

namespace q8 {
static float emulated_dynamic_shared[4 * 16384]; // the router kernel's dynamic shared memory
} // namespace q8

// ---- the CUDA runtime calls of the library's host code, as host calls ---------------------------
static inline int emulated_sms()
{
    const char *env = std::getenv("AOTX_EMULATED_SMS");
    const int sms = env != nullptr ? std::atoi(env) : 6;
    return sms > 0 ? sms : 6;
}

static inline cudaError_t emulated_attribute(int *value, cudaDeviceAttr attribute)
{
    *value = attribute == cudaDevAttrMultiProcessorCount ? emulated_sms()
             : (attribute == cudaDevAttrComputeCapabilityMajor ? 10 : 0);
    return cudaSuccess;
}

static inline cudaError_t emulated_malloc(void **out, size_t bytes)
{
    *out = std::malloc(bytes == 0 ? 1 : bytes);
    return *out != nullptr ? cudaSuccess : cudaErrorMemoryAllocation;
}

#define cudaGetDevice(out) (*(out) = 0, cudaSuccess)
#define cudaSetDevice(device) cudaSuccess
#define cudaDeviceGetAttribute(value, attribute, device) emulated_attribute((value), (attribute))
#define cudaDeviceSynchronize() cudaSuccess
#define cudaMalloc(out, bytes) emulated_malloc((void **)(out), (bytes))
#define cudaFree(p) (std::free(p), cudaSuccess)
#define cudaMemset(p, value, bytes) (std::memset((p), (value), (bytes)), cudaSuccess)
#define cudaMemsetAsync(p, value, bytes, stream) (std::memset((p), (value), (bytes)), cudaSuccess)
#define cudaMemcpy(dst, src, bytes, kind) (std::memcpy((dst), (src), (bytes)), cudaSuccess)
#define cudaGetSymbolAddress(out, symbol) (*(out) = (void *)&(symbol), cudaSuccess)
#undef __align__
#define __align__(n) __attribute__((aligned(n)))

#include "q8_simt.cu"
#include "q_generic.cu"
#include "q8_static.cu"
#include "q8_peers.cu"
#include "q8_api.cu"

// Status bits the emulation itself raised since the last call of this function (work in flight at
// a block's end 0x200, tensor memory kept 0x400, a use the hardware does not define 0x800).
extern "C" unsigned int api_emu_status()
{
    const unsigned int status = emulated_status;
    emulated_status = 0;
    return status;
}

// Copies and tensor-core work complete at once (0) or later on engine threads (1).
extern "C" void api_emu_mode(int asynchronous, unsigned int max_delay_us)
{
    set_mode(asynchronous, max_delay_us);
}

