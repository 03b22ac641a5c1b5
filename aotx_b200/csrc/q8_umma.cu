// The prefill-regime kernel of the Q8_0 product for sm_100a (token tiles of 256 rows of x):
//     y[i][j] = sum_c x[i][c] * half(q[j][c] * d[j][c/32]),   float sums,
// over the reference's own 34-byte interleaved block layout, plus the host side that picks
// between this kernel and the decode-regime kernel of q8_stream.cu and builds their tensor maps.
//
// It was written to replace the reference's tensor-core kernel (cuda/model/gemm.cuh:55-189,
// launched by cuda/model/graph_host.cu:25-29) for batches above 128 rows, with the half-rounded
// weights of that kernel (cuda/model/gemm.cuh:108-113), bit for bit (bfloat16 when x is
// bfloat16).  It is NOT DISPATCHED at present: repeated launches on the same inputs differed in
// a fraction of a percent of the outputs, so batches above 128 rows run as token tiles of 128
// on the kernel of q8_stream.cu (umma_token_tile below).  Run whole on the host by the tests
// (every PTX instruction a stand-in, copies and MMAs completing later) the kernel gives correct
// and repeatable results, so its rings and schedule are sound; what is left is how the hardware
// orders the converters' shared-memory stores against the tensor core's reads.  The kernel stays
// in the library so that the fault can be found; only a build with -DQ8_EXPERIMENT and
// Q8_WIDE_TILE set in the environment reaches it.  (-DQ8_EXPERIMENT also compiles time stamps and switches that leave
// out one stage of the pipeline at a time; the product library is built without it.)
//
// Shape of the work.  The weight rows are the M side of the MMA: a tile is 128 rows of w by
// 256 rows of x, so the 34-byte blocks never need a transpose.  The depth is cut into segments
// of 256 weights (8 blocks = 272 bytes per row, the smallest run of blocks that is a multiple
// of 16 bytes).  Whole waves of tiles are dealt round-robin over one persistent block per SM;
// the tiles of the last partial wave are cut into (tile, segment) units and spread evenly, and
// a tile that is cut between blocks is summed through a scratch slot per block, in a fixed
// order, by the block that holds its first segment.
//
// Pipeline inside a block (15 warps):
//   warp 12   bulk tensor copies of raw weight segments  [128 rows x 272 B]  -> shared
//   warp 13   bulk tensor copies of x tiles [256 x 64], 128-byte swizzle     -> shared
//   warps 4-11 read a raw row (one thread per row and half segment), dequantise exactly
//             (see q8_common.cuh) and store 16-bit values in the K-major 128-byte-swizzled
//             operand layout
//   warp 14   one thread issues tcgen05.mma 128 x 256 x 16, float accumulators in TMEM,
//             two accumulator buffers
//   warps 0-3 read the accumulators from TMEM and store y (or the partial sums)
// All waits are bounded; a wait that runs out raises a status bit and the block runs to
// its end.
#include <cuda.h>
#include <stdlib.h>

#include "q8_launch.h"
#include "q8_tile.cuh"

namespace q8 {

#ifdef Q8_EXPERIMENT
static unsigned long long *g_trace_base = nullptr;
static unsigned int g_trace_launches = 0;
#endif

// Stage counts and the shared-memory map of the kernel for a token tile of NTOK rows.
template <int NTOK>
struct Shape {
    static constexpr uint32_t raw_stages = NTOK <= 64 ? 3 : 2;
    static constexpr uint32_t mma_stages = NTOK <= 128 ? 4 : 3;
    static constexpr uint32_t x_stages = NTOK <= 32 ? 8 : (NTOK == 64 ? 6 : (NTOK == 128 ? 4 : 3));
    static constexpr uint32_t x_stage_bytes = NTOK * kSubK * 2;
    static constexpr uint32_t tmem_columns = 2 * NTOK < 32 ? 32 : 2 * NTOK;
    static constexpr uint32_t a_offset = 0;
    static constexpr uint32_t x_offset = a_offset + mma_stages * kAStageBytes;
    static constexpr uint32_t raw_offset = x_offset + x_stages * x_stage_bytes;
    static constexpr uint32_t bar_offset = raw_offset + raw_stages * kRawStageBytes;
    static constexpr uint32_t bar_count = 2 * raw_stages + 2 * mma_stages + 2 * x_stages + 4 + 1;
    static constexpr uint32_t smem_bytes = bar_offset + bar_count * 8 + 16 + 1024;
    static_assert(smem_bytes <= 227u * 1024u, "one block's shared memory");
    static_assert(tmem_columns <= 512u, "two accumulators within the tensor memory");
};

template <int NTOK, typename YT>
__global__ void __launch_bounds__(kThreads, 1)
q8_umma_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const UmmaArgs args)
{
    using S = Shape<NTOK>;
    extern __shared__ unsigned char smem_raw_[];
    const uint32_t smem0 = (smem_u32(smem_raw_) + 1023u) & ~1023u;
    const uint32_t a_base = smem0 + S::a_offset;
    const uint32_t x_base = smem0 + S::x_offset;
    const uint32_t raw_base = smem0 + S::raw_offset;
    const uint32_t bar_base = smem0 + S::bar_offset;
    // barrier table
    const uint32_t raw_full = bar_base;
    const uint32_t raw_empty = raw_full + 8u * S::raw_stages;
    const uint32_t x_full = raw_empty + 8u * S::raw_stages;
    const uint32_t x_empty = x_full + 8u * S::x_stages;
    const uint32_t a_full = x_empty + 8u * S::x_stages;
    const uint32_t mma_empty = a_full + 8u * S::mma_stages;
    const uint32_t acc_full = mma_empty + 8u * S::mma_stages;
    const uint32_t acc_empty = acc_full + 16u;
    const uint32_t drain_bar = acc_empty + 16u;
    const uint32_t tmem_slot = drain_bar + 8u;
    unsigned char *generic0 = smem_raw_ + (smem0 - smem_u32(smem_raw_));
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(generic0 + (tmem_slot - smem0));
    volatile uint32_t *abort_flag = tmem_slot_ptr + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;

    // The live batch and the schedule; the same in every block.
    // The next kernel on the stream may start its blocks as this one's finish.  Work that only
    // reads the weights runs ahead of the kernels before this one; everything that reads x or
    // the live batch, or writes y or the scratch slots, first waits for them to finish.
    grid_launch_dependents();
    unsigned int m = args.m_max;
    if (args.m_dev != nullptr) {
        grid_dependency_wait();
        unsigned int live = *args.m_dev;
        m = live < m ? live : m;
    }
    if (m == 0u) {
        return;
    }
    const uint32_t segs = args.k / kSegK;
    const uint32_t row_tiles = (args.n + kRows - 1u) / kRows;
    const uint32_t tok_tiles = (m + (uint32_t)NTOK - 1u) / (uint32_t)NTOK;
    unsigned long long units = 0;
    // Whole waves of tiles are dealt round-robin (block b takes tiles b, b + G, ...: the token
    // tiles of one weight row tile then run at the same time on neighbouring SMs and share its
    // bytes in L2); the tiles of the last, partial wave are cut into units and spread evenly
    // over all blocks, first in every block's order of work.
    const unsigned long long tiles = (unsigned long long)row_tiles * tok_tiles;
    const uint32_t waves = (uint32_t)(tiles / gridDim.x);
    const uint32_t dp_tiles = waves * gridDim.x;
    units = (tiles - dp_tiles) * segs;                        // units of the partial wave
    const unsigned int blocks = units < gridDim.x ? (unsigned int)units : gridDim.x;
    WorkIter first_work;
    first_work.segs = segs;
    first_work.u = 0;
    first_work.u_end = 0;
    if (blockIdx.x < blocks) {
        unit_range(blockIdx.x, blocks, units, &first_work.u, &first_work.u_end);
    }
    first_work.sk_tile0 = dp_tiles;
    first_work.dp_next = 0;
    first_work.dp_count = waves;
    first_work.dp_first = blockIdx.x;
    first_work.dp_stride = gridDim.x;
    if (first_work.u >= first_work.u_end && waves == 0u) {
        return;
    }

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < S::raw_stages; ++i) {
            mbar_init(raw_full + 8u * i, 1u);
            mbar_init(raw_empty + 8u * i, kConvertThreads);
        }
        for (uint32_t i = 0; i < S::x_stages; ++i) {
            mbar_init(x_full + 8u * i, 1u);
            mbar_init(x_empty + 8u * i, 1u);
        }
        for (uint32_t i = 0; i < S::mma_stages; ++i) {
            mbar_init(a_full + 8u * i, kConvertThreads / 2u);
            mbar_init(mma_empty + 8u * i, 1u);
        }
        for (uint32_t i = 0; i < 2u; ++i) {
            mbar_init(acc_full + 8u * i, 1u);
            mbar_init(acc_empty + 8u * i, kEpilogueWarps);
        }
        mbar_init(drain_bar, 1u);
        *abort_flag = 0u;
        mbar_init_fence();
    }
    if (warp == kWeightWarp && lane == 0u) {
        tma_prefetch_desc(&tmap_w);
    }
    if (warp == kInputWarp && lane == 0u) {
        tma_prefetch_desc(&tmap_x);
    }
    if (warp == kMmaWarp) {
        tmem_alloc(tmem_slot, S::tmem_columns);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == kWeightWarp) {
        // ---------------------------------------------------------------- raw weight copies
        if (lane == 0u) {
            uint32_t g = 0;
            bool ok = true;
            WorkIter work = first_work;
            uint32_t tile = 0, s0 = 0, s1 = 0;
            for (; ok && work.next(tile, s0, s1);) {
                (void)tile;
                const uint32_t row_tile = tile / tok_tiles;
                for (uint32_t s = s0; s < s1; ++s, ++g) {
                    const uint32_t st = g % S::raw_stages;
                    const uint32_t ph = (g / S::raw_stages) & 1u;
                    if (!mbar_wait(raw_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                        ok = false;
                        break;
                    }
#ifdef Q8_SWITCHES
                    if (args.debug & 1u) {
                        mbar_arrive(raw_full + 8u * st);
                        continue;
                    }
#endif
                    mbar_expect_tx(raw_full + 8u * st, kRawStageBytes);
                    tma_load_2d(raw_base + st * kRawStageBytes, &tmap_w, raw_full + 8u * st,
                                (int)(s * kSegWords), (int)(row_tile * kRows));
                }
            }
            // Let every copy this thread started land before the block ends.
            uint32_t local_abort = 0;
            const uint32_t first = g > S::raw_stages ? g - S::raw_stages : 0u;
            for (uint32_t i = first; i < g; ++i) {
                mbar_wait(raw_full + 8u * (i % S::raw_stages), (i / S::raw_stages) & 1u, &local_abort,
                          nullptr);
            }
        }
    } else if (warp == kInputWarp) {
        // ---------------------------------------------------------------- x tile copies
        if (lane == 0u) {
            uint32_t q = 0;
            grid_dependency_wait();
            bool ok = true;
            WorkIter work = first_work;
            uint32_t tile = 0, s0 = 0, s1 = 0;
            for (; ok && work.next(tile, s0, s1);) {
                (void)tile;
                const uint32_t tok_tile = tile % tok_tiles;
                for (uint32_t s = s0; ok && s < s1; ++s) {
                    for (uint32_t j = 0; j < kSubs; ++j, ++q) {
                        const uint32_t st = q % S::x_stages;
                        const uint32_t ph = (q / S::x_stages) & 1u;
                        if (!mbar_wait(x_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                            ok = false;
                            break;
                        }
#ifdef Q8_SWITCHES
                        if (args.debug & 8u) {
                            mbar_arrive(x_full + 8u * st);
                            continue;
                        }
#endif
                        mbar_expect_tx(x_full + 8u * st, S::x_stage_bytes);
                        tma_load_2d(x_base + st * S::x_stage_bytes, &tmap_x, x_full + 8u * st,
                                    (int)(s * kSegK + j * kSubK), (int)(tok_tile * (uint32_t)NTOK));
                    }
                }
            }
            uint32_t local_abort = 0;
            const uint32_t first = q > S::x_stages ? q - S::x_stages : 0u;
            for (uint32_t i = first; i < q; ++i) {
                mbar_wait(x_full + 8u * (i % S::x_stages), (i / S::x_stages) & 1u, &local_abort,
                          nullptr);
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0u) {
            const uint32_t idesc = umma_idesc(kRows, (uint32_t)NTOK, args.b_bf16, args.b_bf16);
            uint32_t q = 0;
            uint32_t tc = 0;
            bool ok = true;
            WorkIter work = first_work;
            uint32_t tile = 0, s0 = 0, s1 = 0;
            for (; ok && work.next(tile, s0, s1); ++tc) {
                (void)tile;
                const uint32_t buf = tc & 1u;
                const uint32_t aph = (tc >> 1) & 1u;
                if (!mbar_wait(acc_empty + 8u * buf, aph ^ 1u, abort_flag, args.status)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * (uint32_t)NTOK;
                uint32_t accumulate = 0u;
                for (uint32_t s = s0; ok && s < s1; ++s) {
                    for (uint32_t j = 0; j < kSubs; ++j, ++q) {
                        const uint32_t st = q % S::mma_stages;
                        const uint32_t ph = (q / S::mma_stages) & 1u;
                        const uint32_t xst = q % S::x_stages;
                        const uint32_t xph = (q / S::x_stages) & 1u;
                        if (!mbar_wait(a_full + 8u * st, ph, abort_flag, args.status)
                            || !mbar_wait(x_full + 8u * xst, xph, abort_flag, args.status)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint64_t b_desc = umma_desc_sw128(x_base + xst * S::x_stage_bytes);
#ifdef Q8_SWITCHES
                        if (args.debug & 4u) {
                            umma_commit(mma_empty + 8u * st);
                            umma_commit(x_empty + 8u * xst);
                            continue;
                        }
#endif
                        const uint64_t a_desc = umma_desc_sw128(a_base + st * kAStageBytes);
#pragma unroll
                        for (uint32_t kk = 0; kk < kSubK / 16u; ++kk) {
                            // 16 halves = 32 bytes further along the swizzled row
                            umma_f16_ss(d_tmem, a_desc + 2u * kk, b_desc + 2u * kk, idesc, accumulate);
                            accumulate = 1u;
                        }
                        umma_commit(mma_empty + 8u * st);
                        umma_commit(x_empty + 8u * xst);
                    }
                }
                if (ok) {
                    umma_commit(acc_full + 8u * buf);
                }
            }
            if (!ok) {
                // Outstanding MMAs must finish before the tensor memory goes back.
                uint32_t local_abort = 0;
                umma_commit(drain_bar);
                mbar_wait(drain_bar, 0u, &local_abort, nullptr);
            }
        }
    } else if (warp >= kConvertWarp0) {
        // ---------------------------------------------------------------- dequantise
        const uint32_t cw = warp - kConvertWarp0;
        const uint32_t half_id = cw >> 2;
        const uint32_t row = (cw & 3u) * 32u + lane;
        uint32_t g = 0;
        bool ok = true;
        WorkIter work = first_work;
        uint32_t tile = 0, s0 = 0, s1 = 0;
        for (; ok && work.next(tile, s0, s1);) {
            (void)tile;
            for (uint32_t s = s0; ok && s < s1; ++s, ++g) {
                const uint32_t rst = g % S::raw_stages;
                const uint32_t rph = (g / S::raw_stages) & 1u;
                if (!mbar_wait(raw_full + 8u * rst, rph, abort_flag, args.status)) {
                    ok = false;
                    break;
                }
                uint32_t raw[36];
                const uint32_t raw_row = raw_base + rst * kRawStageBytes + row * kSegBytes;
#ifdef Q8_SWITCHES
                if (args.debug & 2u) {
#pragma unroll
                    for (int i = 0; i < 36; ++i) {
                        raw[i] = 0u;
                    }
                } else
#endif
                if (half_id == 0u) {
                    load_raw<0>(raw_row, raw);
                } else {
                    load_raw<1>(raw_row, raw);
                }
                // every thread releases the stage itself, after its own loads
                mbar_arrive(raw_empty + 8u * rst);
#pragma unroll
                for (uint32_t jj = 0; jj < 2u; ++jj) {
                    const uint32_t q = g * kSubs + half_id * 2u + jj;
                    const uint32_t st = q % S::mma_stages;
                    const uint32_t ph = (q / S::mma_stages) & 1u;
                    if (!mbar_wait(mma_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
#ifdef Q8_SWITCHES
                    if (args.debug & 2u) {
                        mbar_arrive(a_full + 8u * st);
                        continue;
                    }
#endif
                    {
                        const uint32_t a_stage = a_base + st * kAStageBytes;
                        if (args.b_bf16 != 0u) {
                            // bfloat16 activations: the weights go to bfloat16 as well
                            if (half_id == 0u) {
                                if (jj == 0u) {
                                    convert_stage<0, 0, true>(raw, a_stage, row);
                                } else {
                                    convert_stage<0, 1, true>(raw, a_stage, row);
                                }
                            } else {
                                if (jj == 0u) {
                                    convert_stage<1, 0, true>(raw, a_stage, row);
                                } else {
                                    convert_stage<1, 1, true>(raw, a_stage, row);
                                }
                            }
                        } else if (half_id == 0u) {
                            if (jj == 0u) {
                                convert_stage<0, 0, false>(raw, a_stage, row);
                            } else {
                                convert_stage<0, 1, false>(raw, a_stage, row);
                            }
                        } else {
                            if (jj == 0u) {
                                convert_stage<1, 0, false>(raw, a_stage, row);
                            } else {
                                convert_stage<1, 1, false>(raw, a_stage, row);
                            }
                        }
                        fence_proxy_async_smem();
                    }
                    // every thread publishes its own row: its stores, its proxy fence, its arrival
                    mbar_arrive(a_full + 8u * st);
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const uint32_t wq = warp; // 0..3: this warp reads TMEM lanes [32 wq, 32 wq + 32)
        uint32_t tc = 0;
        grid_dependency_wait();
        bool ok = true;
        WorkIter work = first_work;
        uint32_t tile = 0, s0 = 0, s1 = 0;
        for (; ok && work.next(tile, s0, s1); ++tc) {
            (void)tile;
            const uint32_t buf = tc & 1u;
            const uint32_t aph = (tc >> 1) & 1u;
            if (!mbar_wait(acc_full + 8u * buf, aph, abort_flag, args.status)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            epilogue_piece<NTOK, YT>(args, tmem_base + buf * (uint32_t)NTOK, wq, lane, tile,
                                     tile >= first_work.sk_tile0 ? tile - first_work.sk_tile0 : 0u, s0, s1, segs,
                                     tok_tiles, units, blocks, m, abort_flag, acc_empty + 8u * buf);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, S::tmem_columns);
    }
}

// ---------------------------------------------------------------------------------------
// Host side.
// ---------------------------------------------------------------------------------------
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

// How much of the next product's weights a launch asks L2 for: what the memory system moves
// while one launch drains and the next fills (a few microseconds), well below the 126 MB of L2.
static unsigned long long next_bytes_limit()
{
#ifdef Q8_EXPERIMENT
    const char *env = getenv("Q8_NEXT_MB");
    if (env != nullptr) {
        return (unsigned long long)atoi(env) << 20;
    }
#endif
    return 32ull << 20;
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

template <int NTOK, typename YT>
static cudaError_t launch_typed(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                                const UmmaArgs &args, unsigned int grid)
{
    using S = Shape<NTOK>;
    static unsigned long long configured = 0ull;
    cudaError_t err = allow_shared_memory(q8_umma_kernel<NTOK, YT>, S::smem_bytes, &configured);
    if (err != cudaSuccess) {
        return err;
    }
    return launch_tile_kernel(q8_umma_kernel<NTOK, YT>, grid, S::smem_bytes, stream, args.overlap != 0u,
                              tw, tx, args);
}

template <int NTOK>
static cudaError_t launch_tile(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                               const UmmaArgs &args, unsigned int grid, int y_dtype)
{
    switch (y_dtype) {
    case 0:
        return launch_typed<NTOK, float>(stream, tw, tx, args, grid);
    case 1:
        return launch_typed<NTOK, __half>(stream, tw, tx, args, grid);
    case 2:
        return launch_typed<NTOK, __nv_bfloat16>(stream, tw, tx, args, grid);
    default:
        return cudaErrorInvalidValue;
    }
}

cudaError_t launch_umma(cudaStream_t stream, const UmmaScratch &scratch, unsigned int sm_count,
                        const void *w, unsigned int n, unsigned int k, const void *x, int x_bf16,
                        unsigned int m, const unsigned int *m_dev, void *y, int y_dtype, unsigned int set,
                        bool overlap, const PeerOut *out, unsigned int epilogue, const NextWeights *next)
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
    args.next_w = nullptr;
    args.next_stride = 0ull;
    args.next_n = args.next_segs = args.next_tok_tiles = args.next_units = 0u;
    if (next != nullptr && next->w != nullptr && next->n != 0u && next->m != 0u && next->k != 0u
        && (next->k % kSegK) == 0u && (reinterpret_cast<uintptr_t>(next->w) & 15u) == 0u) {
        // the following product runs on this kernel too: same schedule arithmetic as below
        const unsigned int next_tile = umma_token_tile(next->m);
        args.next_w = static_cast<const unsigned char *>(next->w);
        args.next_stride = row_bytes(next->k);
        args.next_n = next->n;
        args.next_segs = next->k / kSegK;
        args.next_tok_tiles = (next->m + next_tile - 1u) / next_tile;
        // what the memory system moves while one launch drains and the next fills, per block
        const unsigned long long per_block = next_bytes_limit() / (sm_count == 0u ? 1u : sm_count);
        args.next_units = (unsigned int)(per_block / kRawStageBytes);
        if (args.next_units == 0u) {
            args.next_units = 1u;
        }
    }
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
#ifdef Q8_EXPERIMENT
    {
        const char *env = getenv("Q8_EXPERIMENT");
        args.debug = env != nullptr ? (unsigned int)atoi(env) : 0u;
        args.w = static_cast<const unsigned char *>(w);
        if (getenv("Q8_TRACE") != nullptr) {
            if (g_trace_base == nullptr) {
                cudaMalloc((void **)&g_trace_base, 256ull * 320ull * 8ull * 8ull);
                cudaMemset(g_trace_base, 0, 256ull * 320ull * 8ull * 8ull);
            }
            args.trace = g_trace_base + (unsigned long long)(g_trace_launches % 256u) * 320ull * 8ull;
            g_trace_launches += 1;
        } else {
            args.trace = nullptr;
        }
    }
#endif

#ifdef Q8_EXPERIMENT
    if (ntok <= 32u && getenv("Q8_DUO") != nullptr) {
        // the two-blocks-per-SM form of the decode-regime kernel (q8_duo.cu)
        unsigned int duo_grid = 2u * sm_count < scratch.blocks ? 2u * sm_count : scratch.blocks;
        if (units < duo_grid) {
            duo_grid = (unsigned int)units;
        }
        return launch_duo_kernel(stream, tw, tx, args, duo_grid, ntok, y_dtype);
    }
#endif
    if (ntok <= 32u) {
        // one token tile: the decode kernel, two blocks per SM (q8_decode.cu); its unit
        // arithmetic is 32-bit
        if (units >= (1ull << 31)) {
            return cudaErrorNotSupported;
        }
        unsigned int cluster = 0u;
        const unsigned int decode_blocks = decode_grid((unsigned int)row_tiles, k / kSegK, sm_count,
                                                       scratch.blocks, &cluster);
#ifdef Q8_EXPERIMENT
        if (getenv("Q8_NO_SPLIT") != nullptr && cluster != 0u) {
            cluster = 0u;
            const unsigned long long all = row_tiles * (k / kSegK);
            const unsigned int most = 2u * sm_count < scratch.blocks ? 2u * sm_count : scratch.blocks;
            args.split = 0u;
            return launch_decode_kernel(stream, tw, tx, args, all < most ? (unsigned int)all : most, 0u, ntok, y_dtype);
        }
#endif
        args.split = cluster;
        return launch_decode_kernel(stream, tw, tx, args, decode_blocks, cluster, ntok, y_dtype);
    }
    if (ntok <= 128u) {
        return launch_stream_kernel(stream, tw, tx, args, grid, ntok, y_dtype);
    }
#ifdef Q8_EXPERIMENT
    if (getenv("Q8_WIDE_TILE") != nullptr && atoi(getenv("Q8_WIDE_TILE")) == 1) {
        // the first 256-row form, both operands in shared memory (above): not dispatched
        return launch_tile<256>(stream, tw, tx, args, grid, y_dtype);
    }
#endif
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
    args.next_w = nullptr;
    args.next_stride = 0ull;
    args.next_n = args.next_segs = args.next_tok_tiles = args.next_units = 0u;
#ifdef Q8_EXPERIMENT
    args.debug = 0u;
    args.trace = nullptr;
    args.w = nullptr;
#endif
#ifdef Q8_EXPERIMENT
    if (ntok <= 32u && getenv("Q8_DUO") != nullptr) {
        unsigned int duo_grid = 2u * sm_count < scratch.blocks ? 2u * sm_count : scratch.blocks;
        if (units < duo_grid) {
            duo_grid = (unsigned int)units;
        }
        return launch_duo_kernel(stream, tw, tx, args, duo_grid, ntok, y_dtype);
    }
#endif
    return launch_stream_kernel(stream, tw, tx, args, grid, ntok, y_dtype);
}

} // namespace q8

#ifdef Q8_EXPERIMENT
extern "C" unsigned int q8_trace_read(unsigned long long *host)
{
    if (q8::g_trace_base != nullptr) {
        cudaMemcpy(host, q8::g_trace_base, 256ull * 320ull * 8ull * 8ull, cudaMemcpyDeviceToHost);
    }
    return q8::g_trace_launches;
}
#endif
