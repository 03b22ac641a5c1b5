// Host side of the tensor-core products: which kernel serves a product, its tensor maps, its
// grid and its scratch.
//
//   rows of x     kernel                                                        file
//   1 .. 32       decode kernel, two blocks per SM, cluster split along k       q8_decode.cu
//   33 .. 128     decode-regime kernel, one block per SM (also the grouped      q8_stream.cu
//                 products of the routed experts, token tiles of 64)
//   129 ..        prefill kernel, token tiles of 256, weights in tensor memory  q8_wide.cu
//
// Shapes none of them takes (k not a multiple of 256, unaligned pointers) return
// cudaErrorNotSupported and the caller uses the general kernel (q8_simt.cu).  Reference: the
// regime switch of cuda/model/graph_host.cu:20-40 and cuda/model/product.cu:24-49, which this
// replaces with one launch per product.
#include <cuda.h>
#include <stdlib.h>

#include "q8_launch.h"
#include "q8_tile.cuh"

namespace q8 {

#ifdef Q8_TRACE
static unsigned long long *g_trace_base = nullptr;
static unsigned int g_trace_launches = 0;
#endif

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled()
{
#ifdef Q8_HOST_EMULATION
    return q8emu::encode_tiled; // the tests' stand-in: keeps the map's description for its copies
#endif
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) == cudaSuccess
            && result == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        }
    }
    return fn;
}

unsigned int umma_token_tile(unsigned int m)
{
    if (m <= 16u) {
        return 16u;
    }
    if (m <= 32u) {
        return 32u;
    }
    if (m <= 64u) {
        return 64u;
    }
    // Batches above 128 rows run on the 256-row kernel with the weights in tensor memory
    // (q8_wide.cu), one token tile of 256 rows at a time.
    if (m > 128u) {
        return 256u;
    }
    return 128u;
}

// x as binary16, 16 bytes a step (the conversion the kernels apply to an x tile in shared
// memory: exact between 2^-14 and 65504, saturating above).
__global__ void q8_x_to_f16_kernel(const uint4 *__restrict__ x, unsigned long long chunks, uint4 *__restrict__ out)
{
    for (unsigned long long at = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; at < chunks;
         at += (unsigned long long)gridDim.x * blockDim.x) {
        uint4 v = x[at];
        v.x = bf16x2_to_f16x2(v.x);
        v.y = bf16x2_to_f16x2(v.y);
        v.z = bf16x2_to_f16x2(v.z);
        v.w = bf16x2_to_f16x2(v.w);
        out[at] = v;
    }
}

bool umma_supports(const void *w, unsigned int n, unsigned int k, const void *x, unsigned int m)
{
    if (n == 0u || m == 0u || k == 0u || (k % kSegK) != 0u) {
        return false;
    }
    if ((reinterpret_cast<uintptr_t>(w) & 15u) != 0u || (reinterpret_cast<uintptr_t>(x) & 15u) != 0u) {
        return false;
    }
    return true;
}

cudaError_t launch_umma(cudaStream_t stream, const UmmaScratch &scratch, unsigned int sm_count,
                        const void *w, unsigned int n, unsigned int k, const void *x, int x_bf16,
                        unsigned int m, const unsigned int *m_dev, void *y, int y_dtype, unsigned int set,
                        bool overlap, const PeerOut *out, unsigned int epilogue)
{
    if (!umma_supports(w, n, k, x, m)) {
        return cudaErrorNotSupported;
    }
    EncodeTiledFn encode = encode_tiled();
    if (encode == nullptr) {
        return cudaErrorNotSupported;
    }
    const unsigned int ntok = umma_token_tile(m);
    const unsigned long long row_b = row_bytes(k);
    // bfloat16 activations at 33 to 128 rows: the one-block-per-SM kernel would turn every x
    // tile into binary16 in shared memory, in every block and for every weight row tile, as many
    // bytes again as the weights; one pass over x into the context's copy does it once
    if (x_bf16 && ntok >= 64u && ntok <= 128u && scratch.x16 != nullptr
        && (unsigned long long)m * k * 2ull <= scratch.x16_bytes) {
        const unsigned long long chunks = (unsigned long long)m * k / 8ull;
        const unsigned int blocks = (unsigned int)((chunks + 255ull) / 256ull < 4ull * sm_count
                                                       ? (chunks + 255ull) / 256ull : 4ull * sm_count);
        cudaError_t turned = launch_kernel(q8_x_to_f16_kernel, blocks, 256, 0, stream,
                                           static_cast<const uint4 *>(x), chunks, static_cast<uint4 *>(scratch.x16));
        if (turned != cudaSuccess) {
            return turned;
        }
        x = scratch.x16;
        x_bf16 = 0;
    }

    CUtensorMap tw, tx;
    {
        cuuint64_t dims[2] = {row_b / 4ull, n};
        cuuint64_t strides[1] = {row_b};
        cuuint32_t box[2] = {kSegWords, kRows};
        cuuint32_t elem[2] = {1, 1};
        CUresult r = encode(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(w), dims, strides, box,
                            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            return cudaErrorInvalidValue;
        }
    }
    {
        cuuint64_t dims[2] = {k, m};
        cuuint64_t strides[1] = {(cuuint64_t)k * 2ull};
        cuuint32_t box[2] = {kSubK, ntok};
        cuuint32_t elem[2] = {1, 1};
        CUresult r = encode(&tx, x_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                            const_cast<void *>(x), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            return cudaErrorInvalidValue;
        }
    }

    const unsigned long long row_tiles = (n + kRows - 1u) / kRows;
    const unsigned long long tok_tiles = (m + ntok - 1u) / ntok;
    const unsigned long long units = row_tiles * tok_tiles * (k / kSegK);
    unsigned int grid = sm_count < scratch.blocks ? sm_count : scratch.blocks;
    if (units < grid) {
        grid = (unsigned int)units;
    }
    if (scratch.tile_floats < (unsigned long long)kRows * ntok) {
        return cudaErrorInvalidValue;
    }

    UmmaArgs args = {};
    args.n = n;
    args.k = k;
    args.m_max = m;
    args.m_dev = m_dev;
    args.y = y;
    // Two sets of slots and flags alternate between launches, so that a launch whose blocks
    // start early never meets the slots of the launch before it.
    args.partial = scratch.partial + (unsigned long long)(set & 1u) * scratch.blocks * scratch.tile_floats;
    args.flags = scratch.flags + (unsigned long long)(set & 1u) * scratch.blocks * 4u;
    args.overlap = overlap ? 1u : 0u;
    args.group_tiles = nullptr;
    args.group_count = nullptr;
    args.row_map = nullptr;
    args.epilogue = epilogue;
    args.ldy = epilogue == kEpilogueSwiglu ? n / 2u : n;
    args.peers = 0u;
    args.col0 = 0u;
    if (out != nullptr) {
        args.ldy = out->ldy;
        args.col0 = out->col0;
        args.peers = out->peers;
        for (unsigned int i = 0; i < 8u; ++i) {
            args.y_peer[i] = i < out->peers ? out->y_peer[i] : nullptr;
        }
    }
    args.status = scratch.status;
    args.tile_floats = scratch.tile_floats;
    args.b_bf16 = x_bf16 ? 1u : 0u;
#ifdef Q8_TRACE
    if (getenv("Q8_TRACE") != nullptr) {
        // time stamps of the decode kernel: 8 words per block, 320 blocks, the last 256 launches
        if (g_trace_base == nullptr) {
            cudaMalloc((void **)&g_trace_base, 256ull * 320ull * 8ull * 8ull);
            cudaMemset(g_trace_base, 0, 256ull * 320ull * 8ull * 8ull);
        }
        args.trace = g_trace_base + (unsigned long long)(g_trace_launches % 256u) * 320ull * 8ull;
        g_trace_launches += 1;
    }
#endif
#ifdef Q8_TRACE
    const bool decode_kernel = getenv("Q8_DECODE") == nullptr || atoi(getenv("Q8_DECODE")) != 0;
#else
    const bool decode_kernel = true;
#endif
    if (ntok <= 32u && decode_kernel) {
        // one token tile: the decode kernel, two blocks per SM (q8_decode.cu); its unit
        // arithmetic is 32-bit
        if (units >= (1ull << 31)) {
            return cudaErrorNotSupported;
        }
        unsigned int cluster = 0u;
        const unsigned int decode_blocks = decode_grid((unsigned int)row_tiles, k / kSegK, sm_count,
                                                       scratch.blocks, &cluster);
        args.split = cluster;
        return launch_decode_kernel(stream, tw, tx, args, decode_blocks, cluster, ntok, y_dtype);
    }
    if (ntok <= 128u) {
        return launch_stream_kernel(stream, tw, tx, args, grid, ntok, y_dtype);
    }
    return launch_wide_kernel(stream, tw, tx, args, grid, y_dtype);
}

cudaError_t launch_umma_grouped(cudaStream_t stream, const UmmaScratch &scratch, unsigned int sm_count,
                                const void *w_stacked, unsigned int total_rows, unsigned int k,
                                const void *x_sorted, unsigned int x_rows, unsigned int ntok,
                                const GroupTile *tiles, const unsigned int *count_dev, unsigned int max_tiles,
                                const unsigned int *row_map, void *y, unsigned int ldy, int y_dtype,
                                unsigned int set, bool overlap, unsigned int epilogue)
{
    EncodeTiledFn encode = encode_tiled();
    if (encode == nullptr || (k % kSegK) != 0u || ntok > 128u) {
        return cudaErrorNotSupported;
    }
    if (max_tiles == 0u || x_rows == 0u) {
        return cudaSuccess;
    }
    const unsigned long long row_b = row_bytes(k);
    CUtensorMap tw, tx;
    {
        cuuint64_t dims[2] = {row_b / 4ull, total_rows};
        cuuint64_t strides[1] = {row_b};
        cuuint32_t box[2] = {kSegWords, kRows};
        cuuint32_t elem[2] = {1, 1};
        CUresult r = encode(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(w_stacked), dims, strides,
                            box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            return cudaErrorInvalidValue;
        }
    }
    {
        cuuint64_t dims[2] = {k, x_rows};
        cuuint64_t strides[1] = {(cuuint64_t)k * 2ull};
        cuuint32_t box[2] = {kSubK, ntok};
        cuuint32_t elem[2] = {1, 1};
        CUresult r = encode(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x_sorted), dims, strides,
                            box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            return cudaErrorInvalidValue;
        }
    }
    const unsigned long long units = (unsigned long long)max_tiles * (k / kSegK);
    unsigned int grid = sm_count < scratch.blocks ? sm_count : scratch.blocks;
    if (units < grid) {
        grid = (unsigned int)units;
    }
    UmmaArgs args = {};
    args.n = total_rows;
    args.k = k;
    args.m_max = x_rows;
    args.m_dev = nullptr;
    args.y = y;
    args.partial = scratch.partial + (unsigned long long)(set & 1u) * scratch.blocks * scratch.tile_floats;
    args.flags = scratch.flags + (unsigned long long)(set & 1u) * scratch.blocks * 4u;
    args.status = scratch.status;
    args.tile_floats = scratch.tile_floats;
    args.b_bf16 = 0u;
    args.overlap = overlap ? 1u : 0u;
    args.group_tiles = tiles;
    args.group_count = count_dev;
    args.row_map = row_map;
    args.ldy = ldy;
    args.peers = 0u;
    args.col0 = 0u;
    args.epilogue = epilogue;
    return launch_stream_kernel(stream, tw, tx, args, grid, ntok, y_dtype);
}

} // namespace q8

#ifdef Q8_TRACE
// The time stamps of the last 256 launches of the decode kernel ([launch][block][8] words) and the
// number of launches so far (development builds only, see aotx_b200/timeline.py).
extern "C" unsigned int q8_trace_read(unsigned long long *host)
{
    if (q8::g_trace_base != nullptr) {
        cudaMemcpy(host, q8::g_trace_base, 256ull * 320ull * 8ull * 8ull, cudaMemcpyDeviceToHost);
    }
    return q8::g_trace_launches;
}
#endif
