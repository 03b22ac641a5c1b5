// Dry run of aotx_b200/csrc/gguf_upload.cu on a machine without a GPU: the CUDA runtime calls it
// makes become host calls ("device" memory is whatever the caller passes, pinned memory is the
// heap, events are inert, copies happen at once).  Forced in front of the source with
// `-include`, so the macros below must come after the runtime's own declarations.  It checks the
// loader's host logic - pieces, offsets, the two-buffer turn, the strided row copy - not a GPU.
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

static inline cudaError_t dry_host_alloc(void **out, size_t bytes)
{
    *out = std::malloc(bytes == 0 ? 1 : bytes);
    return *out != nullptr ? cudaSuccess : cudaErrorMemoryAllocation;
}

static inline cudaError_t dry_copy_2d(void *dst, size_t dpitch, const void *src, size_t spitch, size_t width,
                                      size_t height)
{
    for (size_t r = 0; r < height; ++r) {
        std::memcpy(static_cast<unsigned char *>(dst) + r * dpitch,
                    static_cast<const unsigned char *>(src) + r * spitch, width);
    }
    return cudaSuccess;
}

#define cudaGetDevice(out) (*(out) = 0, cudaSuccess)
#define cudaSetDevice(device) cudaSuccess
#define cudaMallocHost(out, bytes) dry_host_alloc((void **)(out), (bytes))
#define cudaFreeHost(p) (std::free(p), cudaSuccess)
#define cudaEventCreateWithFlags(out, flags) (*(out) = reinterpret_cast<cudaEvent_t>(1), cudaSuccess)
#define cudaEventSynchronize(event) cudaSuccess
#define cudaEventRecord(event, stream) cudaSuccess
#define cudaEventDestroy(event) cudaSuccess
#define cudaMemcpyAsync(dst, src, bytes, kind, stream) (std::memcpy((dst), (src), (bytes)), cudaSuccess)
#define cudaMemcpy2DAsync(dst, dpitch, src, spitch, width, height, kind, stream) \
    dry_copy_2d((dst), (dpitch), (src), (spitch), (width), (height))
