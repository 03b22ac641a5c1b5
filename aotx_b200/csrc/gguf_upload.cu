// Upload of tensor bytes from a GGUF file to device memory: two pinned buffers, the read of one
// piece overlapping the copy of the piece before it, and the read of one piece split over host
// threads (aotx_gguf_read_threads: a page-cache or NVMe read on one thread runs well below what
// the link to a B200 takes).  Interface and the reference code it stands in for: include/aotx_gguf_b200.h.
#include "../../include/aotx_gguf_b200.h"

#include <cuda_runtime.h>

#include <new>
#include <thread>

struct aotx_gguf_loader {
    int device;
    size_t piece;
    unsigned char *host[2];
    cudaEvent_t done[2];
    unsigned int turn;
    unsigned int threads;
    int last_cuda;
};

namespace {

const size_t kDefaultPiece = 64ull * 1024ull * 1024ull; /* cuda/boot/weights_host.cu:20 */

int cuda_fail(aotx_gguf_loader *loader, cudaError_t err)
{
    loader->last_cuda = (int)err;
    return AOTX_GGUF_ERR_CUDA;
}

// Makes `device` current for the life of the object and puts the caller's device back.
class DeviceScope {
public:
    explicit DeviceScope(int device) : restore_(false), previous_(0)
    {
        error_ = cudaGetDevice(&previous_);
        if (error_ == cudaSuccess && previous_ != device) {
            error_ = cudaSetDevice(device);
            restore_ = error_ == cudaSuccess;
        }
    }
    ~DeviceScope()
    {
        if (restore_) {
            cudaSetDevice(previous_);
        }
    }
    cudaError_t error() const { return error_; }

private:
    bool restore_;
    int previous_;
    cudaError_t error_;
};

} // namespace

extern "C" int aotx_gguf_loader_init(aotx_gguf_loader **out, int device, size_t piece_bytes)
{
    if (out == nullptr) {
        return AOTX_GGUF_ERR_READ;
    }
    *out = nullptr;
    aotx_gguf_loader *loader = new (std::nothrow) aotx_gguf_loader();
    if (loader == nullptr) {
        return AOTX_GGUF_ERR_READ;
    }
    loader->device = device;
    loader->piece = piece_bytes == 0 ? kDefaultPiece : piece_bytes;
    loader->turn = 0;
    loader->last_cuda = 0;
    unsigned int cores = std::thread::hardware_concurrency();
    loader->threads = cores == 0 ? 1u : (cores > 8u ? 8u : cores);
    DeviceScope scope(device);
    cudaError_t err = scope.error();
    for (int i = 0; i < 2 && err == cudaSuccess; ++i) {
        err = cudaMallocHost((void **)&loader->host[i], loader->piece);
        if (err == cudaSuccess) {
            err = cudaEventCreateWithFlags(&loader->done[i], cudaEventDisableTiming);
        }
    }
    if (err != cudaSuccess) {
        int code = cuda_fail(loader, err);
        aotx_gguf_loader_destroy(loader);
        return code;
    }
    *out = loader;
    return AOTX_GGUF_OK;
}

extern "C" int aotx_gguf_loader_destroy(aotx_gguf_loader *loader)
{
    if (loader == nullptr) {
        return AOTX_GGUF_OK;
    }
    DeviceScope scope(loader->device);
    for (int i = 0; i < 2; ++i) {
        if (loader->done[i] != nullptr) {
            cudaEventSynchronize(loader->done[i]); // a buffer may still be the source of a copy
            cudaEventDestroy(loader->done[i]);
        }
        if (loader->host[i] != nullptr) {
            cudaFreeHost(loader->host[i]);
        }
    }
    delete loader;
    return AOTX_GGUF_OK;
}

extern "C" int aotx_gguf_loader_last_cuda_error(const aotx_gguf_loader *loader)
{
    return loader == nullptr ? 0 : loader->last_cuda;
}

extern "C" int aotx_gguf_upload(aotx_gguf_loader *loader, const aotx_gguf *file, uint64_t offset, uint64_t bytes,
                                void *device_dst, void *stream)
{
    if (loader == nullptr || file == nullptr || (device_dst == nullptr && bytes > 0)) {
        return AOTX_GGUF_ERR_READ;
    }
    const uint64_t have = aotx_gguf_data_bytes(file);
    if (bytes > have || offset > have - bytes) {
        return AOTX_GGUF_ERR_FORMAT;
    }
    DeviceScope scope(loader->device);
    if (scope.error() != cudaSuccess) {
        return cuda_fail(loader, scope.error());
    }
    unsigned char *dst = static_cast<unsigned char *>(device_dst);
    for (uint64_t at = 0; at < bytes; at += loader->piece) {
        const uint64_t piece = bytes - at < loader->piece ? bytes - at : loader->piece;
        const unsigned int slot = loader->turn & 1u;
        // the buffer is free once the copy that last read from it has finished
        cudaError_t err = cudaEventSynchronize(loader->done[slot]);
        if (err != cudaSuccess) {
            return cuda_fail(loader, err);
        }
        int code = aotx_gguf_read_threads(file, offset + at, piece, loader->host[slot], loader->threads);
        if (code != 0) {
            return code;
        }
        err = cudaMemcpyAsync(dst + at, loader->host[slot], (size_t)piece, cudaMemcpyHostToDevice,
                              (cudaStream_t)stream);
        if (err == cudaSuccess) {
            err = cudaEventRecord(loader->done[slot], (cudaStream_t)stream);
        }
        if (err != cudaSuccess) {
            return cuda_fail(loader, err);
        }
        loader->turn += 1u;
    }
    return AOTX_GGUF_OK;
}

extern "C" int aotx_gguf_upload_rows(aotx_gguf_loader *loader, const aotx_gguf *file, uint64_t offset,
                                     uint64_t row_bytes, uint64_t rows, void *device_dst, uint64_t dst_pitch,
                                     void *stream)
{
    if (loader == nullptr || file == nullptr || (device_dst == nullptr && rows > 0) || row_bytes == 0
        || dst_pitch < row_bytes) {
        return AOTX_GGUF_ERR_READ;
    }
    const uint64_t have = aotx_gguf_data_bytes(file);
    if (rows > have / row_bytes || offset > have - rows * row_bytes) {
        return AOTX_GGUF_ERR_FORMAT;
    }
    const uint64_t per_piece = loader->piece / row_bytes; // whole rows per pinned buffer
    if (per_piece == 0) {
        return AOTX_GGUF_ERR_READ;
    }
    DeviceScope scope(loader->device);
    if (scope.error() != cudaSuccess) {
        return cuda_fail(loader, scope.error());
    }
    unsigned char *dst = static_cast<unsigned char *>(device_dst);
    for (uint64_t row = 0; row < rows; row += per_piece) {
        const uint64_t count = rows - row < per_piece ? rows - row : per_piece;
        const unsigned int slot = loader->turn & 1u;
        cudaError_t err = cudaEventSynchronize(loader->done[slot]);
        if (err != cudaSuccess) {
            return cuda_fail(loader, err);
        }
        int code = aotx_gguf_read_threads(file, offset + row * row_bytes, count * row_bytes, loader->host[slot],
                                          loader->threads);
        if (code != 0) {
            return code;
        }
        err = cudaMemcpy2DAsync(dst + row * dst_pitch, (size_t)dst_pitch, loader->host[slot], (size_t)row_bytes,
                                (size_t)row_bytes, (size_t)count, cudaMemcpyHostToDevice, (cudaStream_t)stream);
        if (err == cudaSuccess) {
            err = cudaEventRecord(loader->done[slot], (cudaStream_t)stream);
        }
        if (err != cudaSuccess) {
            return cuda_fail(loader, err);
        }
        loader->turn += 1u;
    }
    return AOTX_GGUF_OK;
}
