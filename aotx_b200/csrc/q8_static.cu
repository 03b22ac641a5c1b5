// The product for callers that cannot allocate device memory.
//
// aotx_q8_matmul_static runs the same kernels as aotx_q8_matmul but takes its scratch (the
// slots through which blocks that share a weight tile hand partial sums to the tile's owner,
// and their flags) from a fixed array inside this library instead of a context that
// aotx_q8_init would have to cudaMalloc.  It is meant for code that runs where allocation is
// not an option: inside a memory plan that is already frozen, in a process that must not grow
// its device footprint after start-up, or in a plug-in that is handed a stream and buffers and
// nothing else.
//
// The array is part of the loaded module: every GPU that loads the library holds it (about
// 5.3 MB) until the process exits.  Its size fixes the limit of this entry point: at most
// Q8_STATIC_MAX_ROWS rows of x per call.  All calls share it, it keeps whatever the last call
// left, and two calls that overlap on the GPU would race on it: issue them on one stream, or
// order them yourself.
#include "../../include/aotx_q8_b200.h"

#include <cuda_runtime.h>

#include <mutex>

#include "q8_common.cuh"
#include "q8_launch.h"

#define Q8_STATIC_MAX_ROWS 64u
#define Q8_STATIC_BLOCKS 160u                                     /* at least the SM count */
#define Q8_STATIC_TILE_FLOATS (128u * Q8_STATIC_MAX_ROWS)         /* one 128 x 64 float tile per block */
#define Q8_STATIC_PARTIAL_BYTES (Q8_STATIC_BLOCKS * Q8_STATIC_TILE_FLOATS * 4u)
#define Q8_STATIC_FLAG_WORDS (Q8_STATIC_BLOCKS * 4u + 4u)         /* flags, then the status word */
#define Q8_STATIC_BYTES (Q8_STATIC_PARTIAL_BYTES + Q8_STATIC_FLAG_WORDS * 4u)
#define Q8_STATIC_DEVICES 64

// Device memory owned by the module.  In host code this name is only a handle for
// cudaGetSymbolAddress; the address the kernels get is looked up below, once per device.
static __device__ __align__(256) unsigned char q8_static_scratch[Q8_STATIC_BYTES];

namespace {

struct StaticDevice {
    bool ready;
    unsigned int sm_count;
    unsigned char *base;
};

StaticDevice g_static[Q8_STATIC_DEVICES];
std::mutex g_static_mutex; // first calls from several host threads set a device up once

// Set-up for the current device: the device address of the array and the SM count.  Runs on
// the first call on each device (not inside a stream capture: the look-up is not a stream
// operation, but it may initialise the module on that device).
cudaError_t static_device(StaticDevice **out)
{
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) {
        return err;
    }
    if (device < 0 || device >= Q8_STATIC_DEVICES) {
        return cudaErrorInvalidDevice;
    }
    StaticDevice *slot = &g_static[device];
    std::lock_guard<std::mutex> guard(g_static_mutex);
    if (!slot->ready) {
        void *address = nullptr;
        err = cudaGetSymbolAddress(&address, q8_static_scratch);
        if (err != cudaSuccess) {
            return err;
        }
        int sms = 0;
        err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (err != cudaSuccess) {
            return err;
        }
        int major = 0;
        err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (err != cudaSuccess) {
            return err;
        }
        if (major != 10) {
            return cudaErrorNotSupported;
        }
        slot->base = static_cast<unsigned char *>(address);
        slot->sm_count = (unsigned int)sms;
        slot->ready = true;
    }
    *out = slot;
    return cudaSuccess;
}

bool is_aligned(const void *p, uintptr_t to)
{
    return (reinterpret_cast<uintptr_t>(p) & (to - 1u)) == 0u;
}

} // namespace

extern "C" int aotx_q8_matmul_static(void *stream, const void *w, uint32_t type, uint32_t n, uint32_t k,
                                     const void *x, int x_dtype, uint32_t m, const uint32_t *m_dev, void *y,
                                     int y_dtype)
{
    if (type != AOTX_Q8_TYPE_Q8_0 && !q8::block_type_known(type)) {
        return AOTX_Q8_ERR_TYPE;
    }
    if ((x_dtype != AOTX_Q8_F16 && x_dtype != AOTX_Q8_BF16) || y_dtype < AOTX_Q8_F32 || y_dtype > AOTX_Q8_BF16
        || k == 0u || (k % 32u) != 0u) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (m > Q8_STATIC_MAX_ROWS) {
        /* the fixed scratch holds tiles of at most 64 rows of x */
        return AOTX_Q8_ERR_WORKSPACE;
    }
    if (n == 0u || m == 0u) {
        return AOTX_Q8_OK;
    }
    if (type != AOTX_Q8_TYPE_Q8_0) {
        /* the other block types run on the ordinary cores and use no scratch */
        if (w == nullptr || x == nullptr || y == nullptr || (k % q8::block_type_run(type)) != 0u
            || !is_aligned(x, 4u) || !is_aligned(y, y_dtype == AOTX_Q8_F32 ? 4u : 2u)
            || (m_dev != nullptr && !is_aligned(m_dev, 4u))) {
            return AOTX_Q8_ERR_ARGUMENT;
        }
        cudaError_t err = q8::launch_gemv_any((cudaStream_t)stream, w, type, n, k, x, x_dtype == AOTX_Q8_BF16, m,
                                              m_dev, y, y_dtype);
        return err == cudaSuccess ? AOTX_Q8_OK : AOTX_Q8_ERR_CUDA;
    }
    if (w == nullptr || x == nullptr || y == nullptr || !is_aligned(w, 2u) || !is_aligned(x, 4u)
        || !is_aligned(y, y_dtype == AOTX_Q8_F32 ? 4u : 2u) || (m_dev != nullptr && !is_aligned(m_dev, 4u))) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    StaticDevice *dev = nullptr;
    if (static_device(&dev) != cudaSuccess) {
        return AOTX_Q8_ERR_CUDA;
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (!q8::umma_supports(w, n, k, x, m)) {
        /* shapes outside the tensor-core kernel need no scratch at all */
        cudaError_t err = q8::launch_gemv_simt(s, w, n, k, x, x_dtype == AOTX_Q8_BF16, m, m_dev, y, y_dtype);
        return err == cudaSuccess ? AOTX_Q8_OK : AOTX_Q8_ERR_CUDA;
    }
    q8::UmmaScratch scratch = {};
    scratch.partial = reinterpret_cast<float *>(dev->base);
    scratch.flags = reinterpret_cast<unsigned int *>(dev->base + Q8_STATIC_PARTIAL_BYTES);
    scratch.status = scratch.flags + Q8_STATIC_BLOCKS * 4u;
    scratch.blocks = Q8_STATIC_BLOCKS;
    scratch.tile_floats = Q8_STATIC_TILE_FLOATS;
    /* The flags must be zero when a launch starts, and the array keeps what the last call (or
     * a call that was cut short) left behind. */
    cudaError_t err = cudaMemsetAsync(scratch.flags, 0, Q8_STATIC_BLOCKS * 4u * sizeof(unsigned int), s);
    if (err == cudaSuccess) {
        err = q8::launch_umma(s, scratch, dev->sm_count, w, n, k, x, x_dtype == AOTX_Q8_BF16, m, m_dev, y,
                              y_dtype, 0u, false);
    }
    return err == cudaSuccess ? AOTX_Q8_OK : AOTX_Q8_ERR_CUDA;
}

extern "C" int aotx_q8_static_status(uint32_t *status, int clear)
{
    if (status == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    *status = 0u;
    StaticDevice *dev = nullptr;
    if (static_device(&dev) != cudaSuccess) {
        return AOTX_Q8_ERR_CUDA;
    }
    unsigned int *flags = reinterpret_cast<unsigned int *>(dev->base + Q8_STATIC_PARTIAL_BYTES);
    unsigned int *word = flags + Q8_STATIC_BLOCKS * 4u;
    cudaError_t err = cudaDeviceSynchronize();
    if (err == cudaSuccess) {
        err = cudaMemcpy(status, word, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    }
    if (err == cudaSuccess && clear && *status != 0u) {
        /* a launch that was cut short may have left hand-over flags raised: nothing runs now,
         * so they go back to zero together with the word */
        err = cudaMemset(flags, 0, (Q8_STATIC_BLOCKS * 4u + 1u) * sizeof(unsigned int));
    }
    if (err != cudaSuccess) {
        return AOTX_Q8_ERR_CUDA;
    }
    return *status == 0u ? AOTX_Q8_OK : AOTX_Q8_ERR_DEVICE;
}
