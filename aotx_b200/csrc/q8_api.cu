// The C ABI of the Q8_0 path: argument checks, the per-device context and the choice of
// kernel family.  Declarations and the reference interfaces they replace are in
// include/aotx_q8_b200.h.
#include "../../include/aotx_q8_b200.h"

#include <cuda_runtime.h>
#include <new>

#include "q8_common.cuh"
#include "q8_launch.h"

struct aotx_q8_ctx {
    int device;
    unsigned int sm_count;
    int path;
    int last_cuda;
    int overlap;
    unsigned int launches;
    q8::UmmaScratch scratch;
};

namespace {

const unsigned int kMaxTokenTile = 256u;
const unsigned int kMaxExperts = 256u; /* cuda/model/kinds_data.h:36 */
const size_t kActivationCopyBytes = 8u << 20; /* 128 rows of x at a depth of 32768 */
const unsigned int kMaxRouteHidden = 10240u; /* the router keeps four rows of x as floats in 160 KB of shared memory */

int cuda_fail(aotx_q8_ctx *ctx, cudaError_t err)
{
    ctx->last_cuda = (int)err;
    return AOTX_Q8_ERR_CUDA;
}

bool dtype_16(int dtype)
{
    return dtype == AOTX_Q8_F16 || dtype == AOTX_Q8_BF16;
}

bool dtype_out(int dtype)
{
    return dtype == AOTX_Q8_F32 || dtype == AOTX_Q8_F16 || dtype == AOTX_Q8_BF16;
}

bool aligned(const void *p, uintptr_t to)
{
    return (reinterpret_cast<uintptr_t>(p) & (to - 1u)) == 0u;
}

} // namespace

extern "C" int aotx_q8_init(aotx_q8_ctx **out, int device)
{
    if (out == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    *out = nullptr;
    aotx_q8_ctx *ctx = new (std::nothrow) aotx_q8_ctx();
    if (ctx == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    ctx->device = device;
    ctx->path = AOTX_Q8_PATH_AUTO;
    ctx->last_cuda = 0;
    ctx->overlap = 1;
    ctx->launches = 0;
    cudaError_t err = cudaSetDevice(device);
    int sms = 0;
    if (err == cudaSuccess) {
        err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    }
    int major = 0;
    if (err == cudaSuccess) {
        err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    }
    if (err != cudaSuccess) {
        int code = cuda_fail(ctx, err);
        delete ctx;
        return code;
    }
    if (major != 10) {
        /* The kernels are sm_100a only; there is no other path. */
        delete ctx;
        return AOTX_Q8_ERR_UNSUPPORTED;
    }
    ctx->sm_count = (unsigned int)sms;
    ctx->scratch.blocks = 2u * ctx->sm_count; /* the decode kernel runs two blocks per SM */
    ctx->scratch.tile_floats = 128ull * kMaxTokenTile;
    size_t partial_bytes = 2u * (size_t)ctx->scratch.blocks * ctx->scratch.tile_floats * sizeof(float);
    size_t flag_bytes = 2u * (size_t)ctx->scratch.blocks * 4u * sizeof(unsigned int);
    err = cudaMalloc((void **)&ctx->scratch.partial, partial_bytes);
    if (err == cudaSuccess) {
        err = cudaMalloc((void **)&ctx->scratch.flags, flag_bytes + sizeof(unsigned int));
    }
    if (err == cudaSuccess) {
        err = cudaMemset(ctx->scratch.flags, 0, flag_bytes + sizeof(unsigned int));
    }
    if (err == cudaSuccess) {
        ctx->scratch.x16_bytes = kActivationCopyBytes;
        err = cudaMalloc(&ctx->scratch.x16, kActivationCopyBytes);
    }
    if (err != cudaSuccess) {
        int code = cuda_fail(ctx, err);
        cudaFree(ctx->scratch.partial);
        cudaFree(ctx->scratch.flags);
        cudaFree(ctx->scratch.x16);
        delete ctx;
        return code;
    }
    ctx->scratch.status = ctx->scratch.flags + 2u * (size_t)ctx->scratch.blocks * 4u;
    *out = ctx;
    return AOTX_Q8_OK;
}

extern "C" int aotx_q8_destroy(aotx_q8_ctx *ctx)
{
    if (ctx == nullptr) {
        return AOTX_Q8_OK;
    }
    cudaSetDevice(ctx->device);
    cudaFree(ctx->scratch.partial);
    cudaFree(ctx->scratch.flags);
    cudaFree(ctx->scratch.x16);
    delete ctx;
    return AOTX_Q8_OK;
}

extern "C" int aotx_q8_set_path(aotx_q8_ctx *ctx, int path)
{
    if (ctx == nullptr || path < AOTX_Q8_PATH_AUTO || path > AOTX_Q8_PATH_TENSOR) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    ctx->path = path;
    return AOTX_Q8_OK;
}

extern "C" int aotx_q8_set_overlap(aotx_q8_ctx *ctx, int enabled)
{
    if (ctx == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    ctx->overlap = enabled != 0;
    return AOTX_Q8_OK;
}

extern "C" int aotx_q8_last_cuda_error(const aotx_q8_ctx *ctx)
{
    return ctx == nullptr ? 0 : ctx->last_cuda;
}

extern "C" int aotx_q8_device_status(aotx_q8_ctx *ctx, uint32_t *status, int clear)
{
    if (ctx == nullptr || status == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    /* the context's device, whatever the caller's current one is; put back afterwards */
    int before = -1;
    cudaGetDevice(&before);
    if (before != ctx->device) {
        cudaSetDevice(ctx->device);
    }
    struct Back {
        int device, ours;
        ~Back()
        {
            if (device >= 0 && device != ours) {
                cudaSetDevice(device);
            }
        }
    } back = {before, ctx->device};
    cudaError_t err = cudaDeviceSynchronize();
    if (err == cudaSuccess) {
        err = cudaMemcpy(status, ctx->scratch.status, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    }
    if (err == cudaSuccess && clear) {
        // A launch whose wait ran out may have left hand-over flags raised (a partial sum that
        // was published and never taken); the next launch would misread them.  Nothing runs
        // now, so the flags of both sets go back to zero together with the status word, which
        // lies right behind them.
        const size_t words = *status != 0u ? 2u * (size_t)ctx->scratch.blocks * 4u + 1u : 1u;
        err = cudaMemset(ctx->scratch.status + 1 - words, 0, words * sizeof(uint32_t));
    }
    if (err != cudaSuccess) {
        return cuda_fail(ctx, err);
    }
    return *status == 0u ? AOTX_Q8_OK : AOTX_Q8_ERR_DEVICE;
}

extern "C" int aotx_q8_dequant(aotx_q8_ctx *ctx, void *stream, const void *w, uint32_t type, uint32_t k,
                               uint32_t first_row, uint32_t rows, void *out_f16)
{
    if (ctx == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (!q8::block_type_known(type)) {
        return AOTX_Q8_ERR_TYPE;
    }
    if (rows == 0u) {
        return AOTX_Q8_OK;
    }
    if (w == nullptr || out_f16 == nullptr || k == 0u || (k % q8::block_type_run(type)) != 0u || !aligned(w, 2u)
        || !aligned(out_f16, 4u)) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    cudaError_t err = type == AOTX_Q8_TYPE_Q8_0
        ? q8::launch_dequant((cudaStream_t)stream, w, k, first_row, rows, out_f16)
        : q8::launch_dequant_any((cudaStream_t)stream, w, type, k, first_row, rows, out_f16);
    return err == cudaSuccess ? AOTX_Q8_OK : cuda_fail(ctx, err);
}

extern "C" int aotx_q8_matmul(aotx_q8_ctx *ctx, void *stream, const void *w, uint32_t type, uint32_t n,
                              uint32_t k, const void *x, int x_dtype, uint32_t m, const uint32_t *m_dev,
                              void *y, int y_dtype)
{
    if (ctx == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (!q8::block_type_known(type)) {
        return AOTX_Q8_ERR_TYPE;
    }
    if (!dtype_16(x_dtype) || !dtype_out(y_dtype) || k == 0u || (k % q8::block_type_run(type)) != 0u) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (n == 0u || m == 0u) {
        return AOTX_Q8_OK;
    }
    if (w == nullptr || x == nullptr || y == nullptr || !aligned(w, 2u) || !aligned(x, 4u)
        || !aligned(y, y_dtype == AOTX_Q8_F32 ? 4u : 2u) || (m_dev != nullptr && !aligned(m_dev, 4u))) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (type != AOTX_Q8_TYPE_Q8_0) {
        /* the other block types of a model file: one decoder, general kernel */
        if (ctx->path == AOTX_Q8_PATH_TENSOR) {
            return AOTX_Q8_ERR_UNSUPPORTED;
        }
        cudaError_t any = q8::launch_gemv_any(s, w, type, n, k, x, x_dtype == AOTX_Q8_BF16, m, m_dev, y, y_dtype);
        return any == cudaSuccess ? AOTX_Q8_OK : cuda_fail(ctx, any);
    }
    /* One MMA takes both operands in one 16-bit format (binary16 weights against bfloat16
     * activations raise an illegal-instruction fault on sm_100a), so for bfloat16 activations
     * the streaming kernel turns the x tiles into binary16 in shared memory (values beyond the
     * binary16 range saturate). */
    bool tensor_ok = q8::umma_supports(w, n, k, x, m);
    if (ctx->path == AOTX_Q8_PATH_TENSOR && !tensor_ok) {
        return AOTX_Q8_ERR_UNSUPPORTED;
    }
    cudaError_t err;
    if (tensor_ok && ctx->path != AOTX_Q8_PATH_GENERAL) {
        err = q8::launch_umma(s, ctx->scratch, ctx->sm_count, w, n, k, x, x_dtype == AOTX_Q8_BF16, m,
                              m_dev, y, y_dtype, ctx->launches++, ctx->overlap != 0, nullptr, 0u);
    } else {
        err = q8::launch_gemv_simt(s, w, n, k, x, x_dtype == AOTX_Q8_BF16, m, m_dev, y, y_dtype);
    }
    return err == cudaSuccess ? AOTX_Q8_OK : cuda_fail(ctx, err);
}

extern "C" int aotx_q8_matmul_fused(aotx_q8_ctx *ctx, void *stream, const void *w, uint32_t type, uint32_t n,
                                    uint32_t k, const void *x, int x_dtype, uint32_t m, const uint32_t *m_dev,
                                    void *y, int y_dtype, int epilogue)
{
    if (ctx == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (epilogue == AOTX_Q8_EPILOGUE_STORE) {
        return aotx_q8_matmul(ctx, stream, w, type, n, k, x, x_dtype, m, m_dev, y, y_dtype);
    }
    if (type != AOTX_Q8_TYPE_Q8_0) {
        return AOTX_Q8_ERR_TYPE;
    }
    if (epilogue != AOTX_Q8_EPILOGUE_ADD && epilogue != AOTX_Q8_EPILOGUE_SWIGLU) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (!dtype_16(x_dtype) || !dtype_out(y_dtype) || k == 0u || (k % 32u) != 0u
        || (epilogue == AOTX_Q8_EPILOGUE_ADD && y_dtype != AOTX_Q8_F32)
        || (epilogue == AOTX_Q8_EPILOGUE_SWIGLU && (n & 1u) != 0u)) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (n == 0u || m == 0u) {
        return AOTX_Q8_OK;
    }
    if (w == nullptr || x == nullptr || y == nullptr || !aligned(w, 2u) || !aligned(x, 4u)
        || !aligned(y, y_dtype == AOTX_Q8_F32 ? 4u : 2u) || (m_dev != nullptr && !aligned(m_dev, 4u))) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    cudaStream_t s = (cudaStream_t)stream;
    bool tensor_ok = q8::umma_supports(w, n, k, x, m);
    if (ctx->path == AOTX_Q8_PATH_TENSOR && !tensor_ok) {
        return AOTX_Q8_ERR_UNSUPPORTED;
    }
    cudaError_t err;
    if (tensor_ok && ctx->path != AOTX_Q8_PATH_GENERAL) {
        err = q8::launch_umma(s, ctx->scratch, ctx->sm_count, w, n, k, x, x_dtype == AOTX_Q8_BF16, m, m_dev, y,
                              y_dtype, ctx->launches++, ctx->overlap != 0, nullptr, (unsigned int)epilogue);
    } else {
        err = q8::launch_gemv_simt(s, w, n, k, x, x_dtype == AOTX_Q8_BF16, m, m_dev, y, y_dtype,
                                   (unsigned int)epilogue);
    }
    return err == cudaSuccess ? AOTX_Q8_OK : cuda_fail(ctx, err);
}

extern "C" int aotx_q8_moe_route(aotx_q8_ctx *ctx, void *stream, const void *x_f16, const float *router,
                                 uint32_t tokens, const uint32_t *tokens_dev, uint32_t hidden,
                                 uint32_t experts, uint32_t used, float *prob, uint32_t *ids)
{
    if (ctx == nullptr || experts == 0u || experts > kMaxExperts || used == 0u || used > experts
        || hidden == 0u) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (tokens == 0u) {
        return AOTX_Q8_OK;
    }
    if (x_f16 == nullptr || router == nullptr || prob == nullptr || ids == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (hidden > kMaxRouteHidden) {
        return AOTX_Q8_ERR_UNSUPPORTED; /* four rows of x as floats must fit in shared memory */
    }
    cudaError_t err = q8::launch_route((cudaStream_t)stream, x_f16, router, tokens, tokens_dev, hidden,
                                       experts, used, prob, ids);
    return err == cudaSuccess ? AOTX_Q8_OK : cuda_fail(ctx, err);
}

extern "C" size_t aotx_q8_moe_workspace_bytes(uint32_t tokens, uint32_t used, uint32_t hidden, uint32_t ffn)
{
    return q8::moe_workspace_layout(tokens, used, hidden, ffn, kMaxExperts).bytes;
}

extern "C" int aotx_q8_moe_ffn(aotx_q8_ctx *ctx, void *stream, const void *w_gate, const void *w_up,
                               const void *w_down, uint32_t type, uint32_t experts, uint32_t hidden,
                               uint32_t ffn, const void *x_f16, const float *prob, const uint32_t *ids,
                               uint32_t tokens, const uint32_t *tokens_dev, uint32_t used, void *out,
                               int out_dtype, void *workspace, size_t workspace_bytes)
{
    if (ctx == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (type != AOTX_Q8_TYPE_Q8_0) {
        return AOTX_Q8_ERR_TYPE;
    }
    if (experts == 0u || experts > kMaxExperts || used == 0u || used > experts || hidden == 0u || ffn == 0u
        || (hidden % 32u) != 0u || (ffn % 32u) != 0u || !dtype_out(out_dtype)) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (tokens == 0u) {
        return AOTX_Q8_OK;
    }
    if (w_gate == nullptr || w_up == nullptr || w_down == nullptr || x_f16 == nullptr || prob == nullptr
        || ids == nullptr || out == nullptr || !aligned(x_f16, 4u)) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    q8::MoeWorkspace ws = q8::moe_workspace_layout(tokens, used, hidden, ffn, kMaxExperts);
    if (workspace == nullptr || !aligned(workspace, 256u) || workspace_bytes < ws.bytes) {
        return AOTX_Q8_ERR_WORKSPACE;
    }
    unsigned char *base = static_cast<unsigned char *>(workspace);
    float *proj = reinterpret_cast<float *>(base + ws.proj);
    cudaStream_t s = (cudaStream_t)stream;
    bool grouped = q8::moe_grouped_supports(w_gate, w_up, w_down, x_f16, hidden, ffn, experts);
    if (ctx->path == AOTX_Q8_PATH_TENSOR && !grouped) {
        return AOTX_Q8_ERR_UNSUPPORTED;
    }
    cudaError_t err;
    if (grouped && ctx->path != AOTX_Q8_PATH_GENERAL) {
        err = q8::launch_moe_grouped(s, ctx->scratch, ctx->sm_count, &ctx->launches, ctx->overlap != 0, w_gate,
                                     w_up, w_down, experts, hidden, ffn, x_f16, ids, tokens, tokens_dev, used,
                                     base, ws);
    } else {
        err = q8::launch_expert_pairs_simt(s, w_gate, w_up, w_down, hidden, ffn, x_f16, ids, experts, tokens,
                                           tokens_dev, used, base + ws.act, proj);
    }
    if (err == cudaSuccess) {
        err = q8::launch_expert_sum(s, proj, prob, ids, tokens, tokens_dev, hidden, experts, used, out,
                                    out_dtype);
    }
    return err == cudaSuccess ? AOTX_Q8_OK : cuda_fail(ctx, err);
}

extern "C" int aotx_q8_moe_ffn_fused(aotx_q8_ctx *ctx, void *stream, const void *w_gate_up, const void *w_down,
                                     uint32_t type, uint32_t experts, uint32_t hidden, uint32_t ffn,
                                     const void *x_f16, const float *prob, const uint32_t *ids, uint32_t tokens,
                                     const uint32_t *tokens_dev, uint32_t used, void *out, int out_dtype,
                                     void *workspace, size_t workspace_bytes)
{
    if (ctx == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (type != AOTX_Q8_TYPE_Q8_0) {
        return AOTX_Q8_ERR_TYPE;
    }
    if (experts == 0u || experts > kMaxExperts || used == 0u || used > experts || hidden == 0u || ffn == 0u
        || (hidden % 32u) != 0u || (ffn % 32u) != 0u || !dtype_out(out_dtype)) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (tokens == 0u) {
        return AOTX_Q8_OK;
    }
    if (w_gate_up == nullptr || w_down == nullptr || x_f16 == nullptr || prob == nullptr || ids == nullptr
        || out == nullptr || !aligned(x_f16, 4u)) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    q8::MoeWorkspace ws = q8::moe_workspace_layout(tokens, used, hidden, ffn, kMaxExperts);
    if (workspace == nullptr || !aligned(workspace, 256u) || workspace_bytes < ws.bytes) {
        return AOTX_Q8_ERR_WORKSPACE;
    }
    /* only the grouped tensor-core products take the interleaved tensor */
    if (ctx->path == AOTX_Q8_PATH_GENERAL
        || !q8::moe_grouped_supports(w_gate_up, w_gate_up, w_down, x_f16, hidden, ffn, experts)) {
        return AOTX_Q8_ERR_UNSUPPORTED;
    }
    unsigned char *base = static_cast<unsigned char *>(workspace);
    float *proj = reinterpret_cast<float *>(base + ws.proj);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t err = q8::launch_moe_grouped_fused(s, ctx->scratch, ctx->sm_count, &ctx->launches,
                                                   ctx->overlap != 0, w_gate_up, w_down, experts, hidden, ffn,
                                                   x_f16, ids, tokens, tokens_dev, used, base, ws);
    if (err == cudaSuccess) {
        err = q8::launch_expert_sum(s, proj, prob, ids, tokens, tokens_dev, hidden, experts, used, out,
                                    out_dtype);
    }
    return err == cudaSuccess ? AOTX_Q8_OK : cuda_fail(ctx, err);
}

extern "C" int aotx_q8_moe_combine(aotx_q8_ctx *ctx, void *stream, const float *proj, const float *prob,
                                   const uint32_t *ids, uint32_t tokens, const uint32_t *tokens_dev,
                                   uint32_t hidden, uint32_t experts, uint32_t used, void *out,
                                   int out_dtype)
{
    if (ctx == nullptr || experts == 0u || used == 0u || used > experts || hidden == 0u
        || !dtype_out(out_dtype)) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (tokens == 0u) {
        return AOTX_Q8_OK;
    }
    if (proj == nullptr || prob == nullptr || ids == nullptr || out == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    cudaError_t err = q8::launch_expert_sum((cudaStream_t)stream, proj, prob, ids, tokens, tokens_dev,
                                            hidden, experts, used, out, out_dtype);
    return err == cudaSuccess ? AOTX_Q8_OK : cuda_fail(ctx, err);
}

extern "C" int aotx_q8_matmul_peers(aotx_q8_ctx *ctx, void *stream, const void *w, uint32_t type, uint32_t n,
                                    uint32_t k, const void *x, int x_dtype, uint32_t m, const uint32_t *m_dev,
                                    void *const *y_peers, uint32_t peers, uint32_t ldy, uint32_t col0,
                                    int y_dtype)
{
    if (ctx == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (type != AOTX_Q8_TYPE_Q8_0) {
        return AOTX_Q8_ERR_TYPE;
    }
    if (!dtype_16(x_dtype) || !dtype_out(y_dtype) || k == 0u || (k % 32u) != 0u || peers == 0u || peers > 8u
        || y_peers == nullptr || (unsigned long long)col0 + n > ldy) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (n == 0u || m == 0u) {
        return AOTX_Q8_OK;
    }
    q8::PeerOut out;
    out.peers = peers;
    out.col0 = col0;
    out.ldy = ldy;
    for (uint32_t i = 0; i < 8u; ++i) {
        out.y_peer[i] = i < peers ? y_peers[i] : nullptr;
        if (i < peers && (y_peers[i] == nullptr || !aligned(y_peers[i], y_dtype == AOTX_Q8_F32 ? 4u : 2u))) {
            return AOTX_Q8_ERR_ARGUMENT;
        }
    }
    if (w == nullptr || x == nullptr || !q8::umma_supports(w, n, k, x, m)) {
        /* only the tensor-core kernels store into peers */
        return w == nullptr || x == nullptr ? AOTX_Q8_ERR_ARGUMENT : AOTX_Q8_ERR_UNSUPPORTED;
    }
    cudaError_t err = q8::launch_umma((cudaStream_t)stream, ctx->scratch, ctx->sm_count, w, n, k, x,
                                      x_dtype == AOTX_Q8_BF16, m, m_dev, out.y_peer[0], y_dtype, ctx->launches++,
                                      ctx->overlap != 0, &out);
    return err == cudaSuccess ? AOTX_Q8_OK : cuda_fail(ctx, err);
}

extern "C" int aotx_q8_peer_barrier(aotx_q8_ctx *ctx, void *stream, void *const *flag_arrays, uint32_t peers,
                                    uint32_t rank, uint32_t *step_word)
{
    if (ctx == nullptr || flag_arrays == nullptr || step_word == nullptr || peers == 0u || peers > 8u
        || rank >= peers || !aligned(step_word, 4u)) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    for (uint32_t i = 0; i < peers; ++i) {
        if (flag_arrays[i] == nullptr || !aligned(flag_arrays[i], 4u)) {
            return AOTX_Q8_ERR_ARGUMENT;
        }
    }
    cudaError_t err = q8::launch_peer_barrier((cudaStream_t)stream, flag_arrays, peers, rank, step_word,
                                              ctx->scratch.status, ctx->overlap != 0);
    return err == cudaSuccess ? AOTX_Q8_OK : cuda_fail(ctx, err);
}

extern "C" int aotx_q8_matmul_colsplit(aotx_q8_ctx *ctx, void *stream, const void *w, uint32_t type, uint32_t n,
                                       uint32_t k, const void *x, int x_dtype, uint32_t m, const uint32_t *m_dev,
                                       void *const *y_peers, void *const *flag_arrays, uint32_t peers,
                                       uint32_t rank, uint32_t ldy, uint32_t col0, int y_dtype,
                                       uint32_t *step_word)
{
    if (ctx == nullptr || flag_arrays == nullptr || step_word == nullptr || rank >= peers) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    int code = aotx_q8_matmul_peers(ctx, stream, w, type, n, k, x, x_dtype, m, m_dev, y_peers, peers, ldy, col0,
                                    y_dtype);
    if (code != AOTX_Q8_OK) {
        return code;
    }
    return aotx_q8_peer_barrier(ctx, stream, flag_arrays, peers, rank, step_word);
}

// The split of `total` experts over `parts` GPUs: the first total % parts hold one more.
static void expert_range(uint32_t total, uint32_t parts, uint32_t rank, uint32_t *first, uint32_t *last)
{
    const uint32_t share = total / parts;
    const uint32_t extra = total % parts;
    *first = rank * share + (rank < extra ? rank : extra);
    *last = *first + share + (rank < extra ? 1u : 0u);
}

extern "C" size_t aotx_q8_moe_ep_workspace_bytes(uint32_t tokens, uint32_t used, uint32_t hidden, uint32_t ffn,
                                                 uint32_t peers)
{
    if (peers == 0u || peers > 8u) {
        return 0u;
    }
    const size_t all = (size_t)tokens * peers;
    return q8::moe_workspace_layout((unsigned int)all, used, hidden, ffn, kMaxExperts).bytes
         + (all * used * sizeof(uint32_t) + 255u) / 256u * 256u;
}

extern "C" int aotx_q8_moe_ep(aotx_q8_ctx *ctx, void *stream, const void *w_gate, const void *w_up,
                              const void *w_down, uint32_t type, uint32_t experts_total, uint32_t hidden,
                              uint32_t ffn, const void *const *x_of_rank, const uint32_t *const *ids_of_rank,
                              const float *prob, uint32_t tokens, uint32_t used, float *const *proj_of_rank,
                              void *const *flag_arrays, uint32_t peers, uint32_t rank, uint32_t *step_word,
                              void *out, int out_dtype, void *workspace, size_t workspace_bytes)
{
    if (ctx == nullptr || peers == 0u || peers > 8u || rank >= peers || x_of_rank == nullptr
        || ids_of_rank == nullptr || proj_of_rank == nullptr || flag_arrays == nullptr || step_word == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (type != AOTX_Q8_TYPE_Q8_0) {
        return AOTX_Q8_ERR_TYPE;
    }
    uint32_t first = 0u, last = 0u;
    expert_range(experts_total, peers, rank, &first, &last);
    const uint32_t local = last - first;
    if (experts_total == 0u || local == 0u || local > kMaxExperts || used == 0u || used > experts_total
        || hidden == 0u || ffn == 0u || !dtype_out(out_dtype)
        || (unsigned long long)tokens * peers * used >= (1ull << 31)) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    if (tokens == 0u) {
        return AOTX_Q8_OK;
    }
    if (w_gate == nullptr || w_up == nullptr || w_down == nullptr || prob == nullptr || out == nullptr) {
        return AOTX_Q8_ERR_ARGUMENT;
    }
    for (uint32_t q = 0; q < peers; ++q) {
        if (x_of_rank[q] == nullptr || ids_of_rank[q] == nullptr || proj_of_rank[q] == nullptr
            || !aligned(x_of_rank[q], 16u) || !aligned(proj_of_rank[q], 16u)) {
            return AOTX_Q8_ERR_ARGUMENT;
        }
    }
    /* the expert-parallel step runs on the grouped tensor-core products only */
    if (ctx->path == AOTX_Q8_PATH_GENERAL
        || !q8::moe_grouped_supports(w_gate, w_up, w_down, x_of_rank[rank], hidden, ffn, local)) {
        return AOTX_Q8_ERR_UNSUPPORTED;
    }
    const uint32_t all = tokens * peers;
    q8::MoeWorkspace ws = q8::moe_workspace_layout(all, used, hidden, ffn, kMaxExperts);
    const size_t ids_bytes = ((size_t)all * used * sizeof(uint32_t) + 255u) / 256u * 256u;
    if (workspace == nullptr || !aligned(workspace, 256u) || workspace_bytes < ws.bytes + ids_bytes) {
        return AOTX_Q8_ERR_WORKSPACE;
    }
    unsigned char *base = static_cast<unsigned char *>(workspace);
    uint32_t *ids_all = reinterpret_cast<uint32_t *>(base + ws.bytes);
    cudaStream_t s = (cudaStream_t)stream;

    /* every GPU's x and selections of this step are in place, and every GPU is done with the
       projections of the step before */
    cudaError_t err = q8::launch_peer_barrier(s, flag_arrays, peers, rank, step_word, ctx->scratch.status);
    if (err == cudaSuccess) {
        err = q8::launch_collect_ids(s, ids_of_rank, peers, tokens * used, first, ids_all);
    }
    if (err == cudaSuccess) {
        q8::RowParts rows = {};
        for (uint32_t q = 0; q < peers; ++q) {
            rows.base[q] = x_of_rank[q];
        }
        rows.parts = peers;
        rows.rows_per_part = tokens;
        err = q8::launch_moe_grouped(s, ctx->scratch, ctx->sm_count, &ctx->launches, ctx->overlap != 0, w_gate,
                                     w_up, w_down, local, hidden, ffn, x_of_rank[rank], ids_all, all, nullptr, used,
                                     base, ws, &rows, proj_of_rank[rank]);
    }
    /* every GPU has written the projections of its experts */
    if (err == cudaSuccess) {
        err = q8::launch_peer_barrier(s, flag_arrays, peers, rank, step_word, ctx->scratch.status);
    }
    if (err == cudaSuccess) {
        q8::ProjParts from = {};
        for (uint32_t q = 0; q < peers; ++q) {
            from.base[q] = proj_of_rank[q];
        }
        from.parts = peers;
        from.share = experts_total / peers;
        from.extra = experts_total % peers;
        from.first_pair = rank * tokens * used;
        err = q8::launch_expert_sum_parts(s, from, prob, ids_of_rank[rank], tokens, nullptr, hidden, experts_total,
                                          used, out, out_dtype);
    }
    return err == cudaSuccess ? AOTX_Q8_OK : cuda_fail(ctx, err);
}
