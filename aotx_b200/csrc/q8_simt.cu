// General-shape kernels of the Q8_0 path on the ordinary cores: dequantisation, the
// any-shape product (depth any multiple of 32, any alignment the block layout allows), the
// expert router, the per-pair expert products and the ordered expert sum.
//
// The streaming tensor-core kernel in q8_umma.cu takes the shapes it supports (depth a
// multiple of 256, 16-byte aligned rows); the product here serves every other shape, so
// that the library covers the whole contract of the reference's kernels:
//   cuda/model/dequant.cu:9-70      -> q8_dequant_kernel
//   cuda/model/gemv.cuh:33-145      -> q8_gemv_simt_kernel
//   cuda/model/experts.cu:10-75     -> q8_route_kernel
//   cuda/model/expert_matrix.cu:8-27, cuda/model/norm.cu:92-105 -> q8_expert_feed_kernel / q8_expert_down_kernel
//   cuda/model/experts.cu:77-98     -> q8_expert_sum_kernel
#include "q8_common.cuh"
#include "q8_launch.h"
#include "q8_simt_gemv.cuh"

#include <math_constants.h>

namespace q8 {

// ---------------------------------------------------------------------------------------
// Dequantisation.  The rows [first, first + rows) are one contiguous run of 34-byte
// blocks, so the kernel walks blocks, not rows: one thread turns 8 weights of one block
// into 8 halves and stores them with one 16-byte store.
// ---------------------------------------------------------------------------------------
__global__ void q8_dequant_kernel(const unsigned char *__restrict__ w, unsigned long long blocks,
                                  __half *__restrict__ out, int wide_store)
{
    unsigned long long total = blocks * 4ull;
    unsigned long long step = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long at = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; at < total;
         at += step) {
        unsigned long long block = at >> 2;
        unsigned int part = (unsigned int)(at & 3ull);
        const unsigned char *one = w + block * Q8_BLOCK_BYTES;
        __half d = *reinterpret_cast<const __half *>(one);
        __half2 d2 = __half2half2(d);
        const unsigned short *src = reinterpret_cast<const unsigned short *>(one + 2u + part * 8u);
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t flipped = (uint32_t)src[i] ^ 0x8080u;
            packed[i] = dequant_pair<0>(flipped, d2);
        }
        __half *dst = out + block * Q8_BLOCK + part * 8u;
        if (wide_store) {
            *reinterpret_cast<uint4 *>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                *reinterpret_cast<__half2 *>(dst + 2 * i) = *reinterpret_cast<__half2 *>(&packed[i]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Expert router.  One block per token (stepping by the grid), 256 threads.  Logits are float
// dot products of the float router rows with the half activations, one warp per expert with
// lanes 32 apart and a shuffle tree; the softmax takes the maximum away; the rank of an
// expert is the count of experts with a larger probability, or an equal one and a lower
// index.  The sums run in the same order as the reference kernel's, so the probabilities
// are the same floats.
// ---------------------------------------------------------------------------------------
#define Q8_ROUTE_THREADS 256u
#define Q8_ROUTE_TOKENS 4u /* tokens that share one pass over the router rows */

// One block takes Q8_ROUTE_TOKENS tokens at a time: a warp reads a router row once and forms
// the dot product of every token of the group with it.  Each (token, expert) sum still adds
// the same products in the same order as one warp of the reference kernel does (lanes 32
// apart, then the shuffle tree), so the probabilities are the same floats.
__global__ void __launch_bounds__(Q8_ROUTE_THREADS)
q8_route_kernel(const __half *__restrict__ x, const float *__restrict__ router, unsigned int tokens_max,
                const unsigned int *tokens_dev, unsigned int hidden, unsigned int experts,
                unsigned int used, float *__restrict__ prob, unsigned int *__restrict__ ids)
{
    // the group's activations as float: [Q8_ROUTE_TOKENS][hidden]
#ifdef Q8_HOST_EMULATION
    float *route_x = emulated_dynamic_shared;
#else
    extern __shared__ float route_x[];
#endif
    __shared__ float probability[Q8_ROUTE_TOKENS][Q8_ROUTE_THREADS];
    __shared__ float reduce[Q8_ROUTE_THREADS];
    unsigned int tokens = tokens_max;
    if (tokens_dev != nullptr) {
        unsigned int live = *tokens_dev;
        tokens = live < tokens_max ? live : tokens_max;
    }
    unsigned int lane = threadIdx.x & 31u;
    unsigned int warp = threadIdx.x >> 5;
    unsigned int e = threadIdx.x;
    for (unsigned int t0 = blockIdx.x * Q8_ROUTE_TOKENS; t0 < tokens; t0 += gridDim.x * Q8_ROUTE_TOKENS) {
        unsigned int group = tokens - t0 < Q8_ROUTE_TOKENS ? tokens - t0 : Q8_ROUTE_TOKENS;
        for (unsigned int at = threadIdx.x; at < Q8_ROUTE_TOKENS * hidden; at += Q8_ROUTE_THREADS) {
            unsigned int g = at / hidden;
            route_x[at] = g < group ? __half2float(x[(size_t)(t0 + g) * hidden + (at - g * hidden)]) : 0.0f;
        }
        __syncthreads();
        for (unsigned int ex = warp; ex < experts; ex += Q8_ROUTE_THREADS / 32u) {
            const float *row = router + (size_t)ex * hidden;
            float dot[Q8_ROUTE_TOKENS];
#pragma unroll
            for (unsigned int g = 0; g < Q8_ROUTE_TOKENS; ++g) {
                dot[g] = 0.0f;
            }
#pragma unroll 8
            for (unsigned int d = lane; d < hidden; d += 32u) {
                float r = row[d];
#pragma unroll
                for (unsigned int g = 0; g < Q8_ROUTE_TOKENS; ++g) {
                    // the reference's own expression; both compile to one fused multiply-add
                    dot[g] += r * route_x[g * hidden + d];
                }
            }
#pragma unroll
            for (unsigned int g = 0; g < Q8_ROUTE_TOKENS; ++g) {
                for (unsigned int step = 16u; step != 0u; step >>= 1) {
                    dot[g] += __shfl_down_sync(0xFFFFFFFFu, dot[g], step);
                }
                if (lane == 0u) {
                    probability[g][ex] = dot[g];
                }
            }
        }
        __syncthreads();
        for (unsigned int g = 0; g < group; ++g) {
            unsigned int t = t0 + g;
            reduce[e] = e < experts ? probability[g][e] : -CUDART_INF_F;
            __syncthreads();
            for (unsigned int step = Q8_ROUTE_THREADS / 2u; step != 0u; step >>= 1) {
                if (e < step) {
                    reduce[e] = fmaxf(reduce[e], reduce[e + step]);
                }
                __syncthreads();
            }
            float value = e < experts ? expf(probability[g][e] - reduce[0]) : 0.0f;
            __syncthreads();
            reduce[e] = value;
            __syncthreads();
            for (unsigned int step = Q8_ROUTE_THREADS / 2u; step != 0u; step >>= 1) {
                if (e < step) {
                    reduce[e] += reduce[e + step];
                }
                __syncthreads();
            }
            if (e < experts) {
                value /= reduce[0];
                probability[g][e] = value;
                prob[(size_t)t * experts + e] = value;
            }
            __syncthreads();
            if (e < experts) {
                unsigned int rank = 0u;
                for (unsigned int other = 0u; other < experts; ++other) {
                    float candidate = probability[g][other];
                    rank += (candidate > value || (candidate == value && other < e)) ? 1u : 0u;
                }
                if (rank < used) {
                    ids[(size_t)t * used + rank] = e;
                }
            }
            __syncthreads();
        }
    }
}

// ---------------------------------------------------------------------------------------
// Per-pair expert products (pair = token t, rank r; index t * used + r).  These re-read an
// expert's slice for every pair, like the reference's per-token kernel; the grouped
// tensor-core kernels replace them for the shapes those support.
// ---------------------------------------------------------------------------------------

// act[pair][f] = half(silu(gate) * up), gate = x[t] . Wg[e][f], up = x[t] . Wu[e][f].
__global__ void __launch_bounds__(Q8_SIMT_WARPS * 32u)
q8_expert_feed_kernel(const unsigned char *__restrict__ w_gate, const unsigned char *__restrict__ w_up,
                      unsigned int hidden, unsigned int ffn, const __half *__restrict__ x,
                      const unsigned int *__restrict__ ids, unsigned int experts, unsigned int tokens_max,
                      const unsigned int *tokens_dev, unsigned int used, __half *__restrict__ act)
{
    unsigned int tokens = tokens_max;
    if (tokens_dev != nullptr) {
        unsigned int live = *tokens_dev;
        tokens = live < tokens_max ? live : tokens_max;
    }
    unsigned int lane = threadIdx.x & 31u;
    unsigned int warp = threadIdx.x >> 5;
    unsigned long long stride = row_bytes(hidden);
    unsigned int f = blockIdx.x * Q8_SIMT_WARPS + warp;
    if (f >= ffn) {
        return;
    }
    for (unsigned int pair = blockIdx.y; pair < tokens * used; pair += gridDim.y) {
        unsigned int t = pair / used;
        unsigned int expert = ids[pair];
        if (expert >= experts) {
            continue; // a selection outside the expert table: left out, as in the grouped path
        }
        const unsigned char *gate_row = w_gate + ((unsigned long long)expert * ffn + f) * stride;
        const unsigned char *up_row = w_up + ((unsigned long long)expert * ffn + f) * stride;
        float gate[Q8_SIMT_TAKE];
        float up[Q8_SIMT_TAKE];
        simt_row<__half>(gate_row, hidden, x + (size_t)t * hidden, hidden, 1u, gate);
        simt_row<__half>(up_row, hidden, x + (size_t)t * hidden, hidden, 1u, up);
        if (lane == 0u) {
            float unit = gate[0] / (1.0f + expf(-gate[0]));
            act[(size_t)pair * ffn + f] = __float2half_rn(unit * up[0]);
        }
    }
}

// proj[pair][d] = act[pair] . Wd[e][d]
__global__ void __launch_bounds__(Q8_SIMT_WARPS * 32u)
q8_expert_down_kernel(const unsigned char *__restrict__ w_down, unsigned int hidden, unsigned int ffn,
                      const __half *__restrict__ act, const unsigned int *__restrict__ ids,
                      unsigned int experts, unsigned int tokens_max, const unsigned int *tokens_dev,
                      unsigned int used, float *__restrict__ proj)
{
    unsigned int tokens = tokens_max;
    if (tokens_dev != nullptr) {
        unsigned int live = *tokens_dev;
        tokens = live < tokens_max ? live : tokens_max;
    }
    unsigned int lane = threadIdx.x & 31u;
    unsigned int warp = threadIdx.x >> 5;
    unsigned long long stride = row_bytes(ffn);
    unsigned int d = blockIdx.x * Q8_SIMT_WARPS + warp;
    if (d >= hidden) {
        return;
    }
    for (unsigned int pair = blockIdx.y; pair < tokens * used; pair += gridDim.y) {
        unsigned int expert = ids[pair];
        if (expert >= experts) {
            continue;
        }
        const unsigned char *row = w_down + ((unsigned long long)expert * hidden + d) * stride;
        float sum[Q8_SIMT_TAKE];
        simt_row<__half>(row, ffn, act + (size_t)pair * ffn, ffn, 1u, sum);
        if (lane == 0u) {
            proj[(size_t)pair * hidden + d] = sum[0];
        }
    }
}

// out[t][d] = the ordered sum over ranks: rank 0 gives fmul(proj, p); each later rank adds
// fmul(proj, p) with a separate rounding of the product and of the sum.  A thread carries
// WIDTH neighbouring columns (WIDTH = 4: one 16-byte load of proj per rank); every column's
// chain of roundings is the one written above whatever the width.  The loads of up to eight
// ranks go out together before the chain of additions starts.
//
// `from` says where a pair's projection lies: in one array [tokens][used][hidden], or - expert
// parallel - in the array of the GPU that holds the pair's expert (experts dealt to `parts`
// GPUs as shard_rows deals rows: the first `extra` of them one expert more), at the row of
// the pair among all GPUs' pairs (first_pair + t * used + r).
template <typename YT, unsigned int WIDTH>
__global__ void q8_expert_sum_kernel(const __grid_constant__ ProjParts from, const float *__restrict__ prob,
                                     const unsigned int *__restrict__ ids, unsigned int tokens_max,
                                     const unsigned int *tokens_dev, unsigned int hidden,
                                     unsigned int experts, unsigned int used, YT *__restrict__ out)
{
    constexpr unsigned int kTogether = 8u;
    unsigned int tokens = tokens_max;
    if (tokens_dev != nullptr) {
        unsigned int live = *tokens_dev;
        tokens = live < tokens_max ? live : tokens_max;
    }
    for (unsigned int t = blockIdx.x; t < tokens; t += gridDim.x) {
        for (unsigned int d = threadIdx.x * WIDTH; d < hidden; d += blockDim.x * WIDTH) {
            float sum[WIDTH];
#pragma unroll
            for (unsigned int i = 0; i < WIDTH; ++i) {
                sum[i] = 0.0f;
            }
            for (unsigned int r0 = 0; r0 < used; r0 += kTogether) {
                float value[kTogether][WIDTH];
                float p[kTogether];
#pragma unroll
                for (unsigned int q = 0; q < kTogether; ++q) {
                    const unsigned int r = r0 + q;
                    const unsigned int expert = r < used ? ids[(size_t)t * used + r] : 0xFFFFFFFFu;
                    // a selection outside the expert table has no probability and no projection
                    // (the product kernels leave it out): it adds nothing
                    p[q] = 0.0f;
#pragma unroll
                    for (unsigned int i = 0; i < WIDTH; ++i) {
                        value[q][i] = 0.0f;
                    }
                    if (expert < experts) {
                        p[q] = prob[(size_t)t * experts + expert];
                        const float *base = from.base[0];
                        if (from.parts > 1u) {
                            const unsigned int cut = from.extra * (from.share + 1u);
                            const unsigned int owner = expert < cut ? expert / (from.share + 1u)
                                                                    : from.extra + (expert - cut) / from.share;
                            base = from.base[owner];
                        }
                        const float *row = base + ((size_t)from.first_pair + (size_t)t * used + r) * hidden + d;
                        if (WIDTH == 4u) {
                            const float4 four = *reinterpret_cast<const float4 *>(row);
                            value[q][0] = four.x;
                            value[q][1 % WIDTH] = four.y;
                            value[q][2 % WIDTH] = four.z;
                            value[q][3 % WIDTH] = four.w;
                        } else {
#pragma unroll
                            for (unsigned int i = 0; i < WIDTH; ++i) {
                                value[q][i] = row[i];
                            }
                        }
                    }
                }
#pragma unroll
                for (unsigned int q = 0; q < kTogether; ++q) {
                    if (r0 + q < used) {
#pragma unroll
                        for (unsigned int i = 0; i < WIDTH; ++i) {
                            const float term = __fmul_rn(value[q][i], p[q]);
                            sum[i] = (r0 + q == 0u) ? term : __fadd_rn(sum[i], term);
                        }
                    }
                }
            }
#pragma unroll
            for (unsigned int i = 0; i < WIDTH; ++i) {
                store_out<YT>(out, (size_t)t * hidden + d + i, sum[i]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Launchers.
// ---------------------------------------------------------------------------------------
cudaError_t launch_dequant(cudaStream_t stream, const void *w, unsigned int k, unsigned int first_row,
                           unsigned int rows, void *out)
{
    unsigned long long blocks = (unsigned long long)rows * (k / Q8_BLOCK);
    if (blocks == 0ull) {
        return cudaSuccess;
    }
    const unsigned char *base = static_cast<const unsigned char *>(w) + row_bytes(k) * first_row;
    unsigned long long threads = blocks * 4ull;
    unsigned long long want = (threads + 255ull) / 256ull;
    unsigned int grid = (unsigned int)(want < 148ull * 16ull ? want : 148ull * 16ull);
    int wide = (reinterpret_cast<uintptr_t>(out) & 15u) == 0u;
    return launch_kernel(q8_dequant_kernel, grid, 256, 0, stream, base, blocks, static_cast<__half *>(out), wide);
}

template <typename XT, typename YT>
static cudaError_t launch_gemv_simt_typed(cudaStream_t stream, const void *w, unsigned int n,
                                          unsigned int k, const void *x, unsigned int m,
                                          const unsigned int *m_dev, void *y, unsigned int epilogue)
{
    unsigned int want = (n + Q8_SIMT_WARPS - 1u) / Q8_SIMT_WARPS;
    unsigned int grid = want < 148u * 8u ? want : 148u * 8u;
    if (epilogue == kEpilogueStore) {
        return launch_kernel(q8_gemv_simt_kernel<XT, YT>, grid, Q8_SIMT_WARPS * 32u, 0, stream,
                             static_cast<const unsigned char *>(w), n, k, static_cast<const XT *>(x), m, m_dev,
                             static_cast<YT *>(y));
    }
    return launch_kernel(q8_gemv_simt_fused_kernel<XT, YT>, grid, Q8_SIMT_WARPS * 32u, 0, stream,
                         static_cast<const unsigned char *>(w), n, k, static_cast<const XT *>(x), m, m_dev,
                         static_cast<YT *>(y), epilogue);
}

cudaError_t launch_gemv_simt(cudaStream_t stream, const void *w, unsigned int n, unsigned int k,
                             const void *x, int x_bf16, unsigned int m, const unsigned int *m_dev,
                             void *y, int y_dtype, unsigned int epilogue)
{
    if (n == 0u || m == 0u) {
        return cudaSuccess;
    }
    if ((epilogue == kEpilogueAdd && y_dtype != 0) || (epilogue == kEpilogueSwiglu && (n & 1u) != 0u)
        || epilogue > kEpilogueSwiglu) {
        return cudaErrorInvalidValue;
    }
#define Q8_CASE(XT, YD, YT)                                                                      \
    if (y_dtype == (YD)) {                                                                       \
        return launch_gemv_simt_typed<XT, YT>(stream, w, n, k, x, m, m_dev, y, epilogue);        \
    }
    if (x_bf16) {
        Q8_CASE(__nv_bfloat16, 0, float)
        Q8_CASE(__nv_bfloat16, 1, __half)
        Q8_CASE(__nv_bfloat16, 2, __nv_bfloat16)
    } else {
        Q8_CASE(__half, 0, float)
        Q8_CASE(__half, 1, __half)
        Q8_CASE(__half, 2, __nv_bfloat16)
    }
#undef Q8_CASE
    return cudaErrorInvalidValue;
}

cudaError_t launch_route(cudaStream_t stream, const void *x, const float *router, unsigned int tokens,
                         const unsigned int *tokens_dev, unsigned int hidden, unsigned int experts,
                         unsigned int used, float *prob, unsigned int *ids)
{
    if (tokens == 0u) {
        return cudaSuccess;
    }
    unsigned int groups = (tokens + Q8_ROUTE_TOKENS - 1u) / Q8_ROUTE_TOKENS;
    unsigned int grid = groups < 148u * 8u ? groups : 148u * 8u;
    size_t smem = (size_t)Q8_ROUTE_TOKENS * hidden * sizeof(float);
    if (smem > 160u * 1024u) {
        return cudaErrorInvalidValue;
    }
    static unsigned long long configured = 0ull;
    cudaError_t err = allow_shared_memory(q8_route_kernel, 160u * 1024u, &configured);
    if (err != cudaSuccess) {
        return err;
    }
    return launch_kernel(q8_route_kernel, grid, Q8_ROUTE_THREADS, smem, stream, static_cast<const __half *>(x), router,
                         tokens, tokens_dev, hidden, experts, used, prob, ids);
}

cudaError_t launch_expert_pairs_simt(cudaStream_t stream, const void *w_gate, const void *w_up,
                                     const void *w_down, unsigned int hidden, unsigned int ffn,
                                     const void *x, const unsigned int *ids, unsigned int experts,
                                     unsigned int tokens, const unsigned int *tokens_dev, unsigned int used,
                                     void *act, float *proj)
{
    unsigned int pairs = tokens * used;
    if (pairs == 0u) {
        return cudaSuccess;
    }
    unsigned int wave = pairs < 4096u ? pairs : 4096u;
    dim3 feed((ffn + Q8_SIMT_WARPS - 1u) / Q8_SIMT_WARPS, wave);
    dim3 down((hidden + Q8_SIMT_WARPS - 1u) / Q8_SIMT_WARPS, wave);
    cudaError_t err = launch_kernel(q8_expert_feed_kernel, feed, Q8_SIMT_WARPS * 32u, 0, stream,
                                    static_cast<const unsigned char *>(w_gate),
                                    static_cast<const unsigned char *>(w_up), hidden, ffn,
                                    static_cast<const __half *>(x), ids, experts, tokens, tokens_dev, used,
                                    static_cast<__half *>(act));
    if (err != cudaSuccess) {
        return err;
    }
    return launch_kernel(q8_expert_down_kernel, down, Q8_SIMT_WARPS * 32u, 0, stream,
                         static_cast<const unsigned char *>(w_down), hidden, ffn, static_cast<const __half *>(act),
                         ids, experts, tokens, tokens_dev, used, proj);
}

template <typename YT>
static cudaError_t expert_sum_launch(bool wide, unsigned int grid, cudaStream_t stream, const ProjParts &proj,
                                     const float *prob, const unsigned int *ids, unsigned int tokens,
                                     const unsigned int *tokens_dev, unsigned int hidden, unsigned int experts,
                                     unsigned int used, void *out)
{
    if (wide) {
        return launch_kernel(q8_expert_sum_kernel<YT, 4u>, grid, 256, 0, stream, proj, prob, ids, tokens, tokens_dev,
                             hidden, experts, used, static_cast<YT *>(out));
    }
    return launch_kernel(q8_expert_sum_kernel<YT, 1u>, grid, 256, 0, stream, proj, prob, ids, tokens, tokens_dev,
                         hidden, experts, used, static_cast<YT *>(out));
}

cudaError_t launch_expert_sum_parts(cudaStream_t stream, const ProjParts &proj, const float *prob,
                                    const unsigned int *ids, unsigned int tokens,
                                    const unsigned int *tokens_dev, unsigned int hidden, unsigned int experts,
                                    unsigned int used, void *out, int out_dtype)
{
    if (tokens == 0u) {
        return cudaSuccess;
    }
    unsigned int grid = tokens < 148u * 8u ? tokens : 148u * 8u;
    // 16-byte loads of proj need rows of a multiple of four floats on a 16-byte boundary
    bool wide = (hidden % 4u) == 0u;
    for (unsigned int i = 0; i < (proj.parts > 1u ? proj.parts : 1u); ++i) {
        wide = wide && (reinterpret_cast<uintptr_t>(proj.base[i]) & 15u) == 0u;
    }
    if (out_dtype == 0) {
        return expert_sum_launch<float>(wide, grid, stream, proj, prob, ids, tokens, tokens_dev, hidden, experts,
                                        used, out);
    }
    if (out_dtype == 1) {
        return expert_sum_launch<__half>(wide, grid, stream, proj, prob, ids, tokens, tokens_dev, hidden, experts,
                                         used, out);
    }
    if (out_dtype == 2) {
        return expert_sum_launch<__nv_bfloat16>(wide, grid, stream, proj, prob, ids, tokens, tokens_dev, hidden,
                                                experts, used, out);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_expert_sum(cudaStream_t stream, const float *proj, const float *prob,
                              const unsigned int *ids, unsigned int tokens,
                              const unsigned int *tokens_dev, unsigned int hidden, unsigned int experts,
                              unsigned int used, void *out, int out_dtype)
{
    ProjParts one = {};
    one.base[0] = proj;
    one.parts = 1u;
    return launch_expert_sum_parts(stream, one, prob, ids, tokens, tokens_dev, hidden, experts, used, out,
                                   out_dtype);
}

} // namespace q8
