// Dry run of tests/seam_check.cu on a machine without a GPU: the few CUDA runtime calls the
// program makes become host calls (device memory = heap, a captured graph = the recorded call
// replayed), and the library's entry points become a plain host product.  Built with
// -DSEAM_DRY_RUN and without the product library.  It checks the PROGRAM - its fixtures, its
// host product, its measure, its guard rows, the loop over the batch word - not the kernels.
#pragma once

#include <cstdlib>
#include <cstring>

struct DryCall {
    bool set;
    const void *w;
    uint32_t n, k;
    const void *x;
    uint32_t m;
    const uint32_t *m_dev;
    float *y;
};

static bool dry_capturing = false;
static DryCall dry_call = {};

static void dry_run(const DryCall &c)
{
    const unsigned char *w = static_cast<const unsigned char *>(c.w);
    const __half *x = static_cast<const __half *>(c.x);
    uint32_t live = c.m;
    if (c.m_dev != nullptr && *c.m_dev < live) {
        live = *c.m_dev;
    }
    for (uint32_t i = 0; i < live; ++i) {
        for (uint32_t j = 0; j < c.n; ++j) {
            float sum = 0.0f;
            for (uint32_t b = 0; b < c.k / 32u; ++b) {
                const unsigned char *block = w + ((size_t)j * (c.k / 32u) + b) * 34u;
                __half d;
                std::memcpy(&d, block, 2);
                for (uint32_t t = 0; t < 32u; ++t) {
                    const float weight = __half2float(__float2half((float)(signed char)block[2u + t] * __half2float(d)));
                    sum += weight * __half2float(x[(size_t)i * c.k + b * 32u + t]);
                }
            }
            c.y[(size_t)i * c.n + j] = sum;
        }
    }
}

extern "C" int aotx_q8_init(aotx_q8_ctx **ctx, int)
{
    *ctx = reinterpret_cast<aotx_q8_ctx *>(std::malloc(1));
    return AOTX_Q8_OK;
}

extern "C" int aotx_q8_destroy(aotx_q8_ctx *ctx)
{
    std::free(ctx);
    return AOTX_Q8_OK;
}

extern "C" int aotx_q8_device_status(aotx_q8_ctx *, uint32_t *status, int)
{
    *status = 0;
    return AOTX_Q8_OK;
}

extern "C" int aotx_q8_matmul(aotx_q8_ctx *, void *, const void *w, uint32_t type, uint32_t n, uint32_t k,
                              const void *x, int x_dtype, uint32_t m, const uint32_t *m_dev, void *y, int y_dtype)
{
    if (type != AOTX_Q8_TYPE_Q8_0) {
        return AOTX_Q8_ERR_TYPE;
    }
    if (x_dtype != AOTX_Q8_F16 || y_dtype != AOTX_Q8_F32 || (k % 32u) != 0u) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    DryCall call = {true, w, n, k, x, m, m_dev, static_cast<float *>(y)};
    if (dry_capturing) {
        dry_call = call; // nothing runs inside a capture
    } else {
        dry_run(call);
    }
    return AOTX_Q8_OK;
}

extern "C" int aotx_q8_matmul_fused(aotx_q8_ctx *, void *, const void *, uint32_t, uint32_t, uint32_t, const void *,
                                    int, uint32_t, const uint32_t *, void *, int, int)
{
    return AOTX_Q8_ERR_UNSUPPORTED;
}

extern "C" int aotx_q8_dequant(aotx_q8_ctx *, void *, const void *, uint32_t, uint32_t, uint32_t, uint32_t, void *)
{
    return AOTX_Q8_ERR_UNSUPPORTED;
}

static cudaError_t dry_malloc(void **out, size_t bytes)
{
    *out = std::malloc(bytes == 0 ? 1 : bytes);
    return *out != nullptr ? cudaSuccess : cudaErrorMemoryAllocation;
}

static cudaError_t dry_begin()
{
    dry_capturing = true;
    dry_call.set = false;
    return cudaSuccess;
}

static cudaError_t dry_end(cudaGraph_t *graph)
{
    dry_capturing = false;
    *graph = reinterpret_cast<cudaGraph_t>(&dry_call);
    return dry_call.set ? cudaSuccess : cudaErrorInvalidValue;
}

static cudaError_t dry_replay()
{
    if (!dry_call.set) {
        return cudaErrorInvalidValue;
    }
    dry_run(dry_call);
    return cudaSuccess;
}

#define cudaMalloc(out, bytes) dry_malloc((void **)(out), (bytes))
#define cudaFree(p) (std::free(p), cudaSuccess)
#define cudaMemcpy(dst, src, bytes, kind) (std::memcpy((dst), (src), (bytes)), cudaSuccess)
#define cudaMemcpyAsync(dst, src, bytes, kind, stream) (std::memcpy((dst), (src), (bytes)), cudaSuccess)
#define cudaStreamCreate(out) (*(out) = nullptr, cudaSuccess)
#define cudaStreamSynchronize(stream) cudaSuccess
#define cudaStreamDestroy(stream) cudaSuccess
#define cudaStreamBeginCapture(stream, mode) dry_begin()
#define cudaStreamEndCapture(stream, graph) dry_end(graph)
#define cudaGraphInstantiate(exec, graph, flags) (*(exec) = reinterpret_cast<cudaGraphExec_t>(graph), cudaSuccess)
#define cudaGraphLaunch(exec, stream) dry_replay()
#define cudaGraphExecDestroy(exec) cudaSuccess
#define cudaGraphDestroy(graph) cudaSuccess
