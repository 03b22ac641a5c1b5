// The decode-regime kernel of the Q8_0 product with one block per SM: token tiles of 64 and 128
// rows of x (batches of 33 to 128 rows) and the grouped products of the routed experts.  The
// weights stream through once at memory speed, whatever the batch.  Batches of up to 32 rows
// run on the two-blocks-per-SM form (q8_decode.cu), batches above 128 on q8_wide.cu.
//
// Tiles of 128 rows of w by NTOK rows of x, depth in segments of 256 weights, (tile, segment)
// units dealt evenly over one persistent block per SM.  Built around two facts of this regime:
//   * the dequantised weight tile never touches shared memory: each converter thread owns one
//     row, writes its 64-weight pieces straight into its lane of tensor memory with
//     tcgen05.st, and the MMA reads A from there.  Shared memory then holds only raw bytes in
//     flight (a ring of 34 KB segments) and the x tiles;
//   * a hand-off between warps costs far more than the MMAs of one 64-weight step at these
//     widths, so every ring is handed over once per 256-weight segment (16 MMAs), not once
//     per step.
//
// Warps: 0-3 epilogue, 4-11 converters (thread = row x half segment), 12 raw weight copies,
// 13 x copies, 14 MMA issue.  Reference kernels replaced: ptx/gemv_q8.ptx:18-223,
// cuda/model/gemv.cuh:33-145 and, below 129 rows, cuda/model/gemm.cuh:55-189.
#include <cuda.h>
#include <stdlib.h>

#include "q8_launch.h"
#include "q8_tile.cuh"

namespace q8 {

// Stage counts of the 64-row token tile (the routed-expert products and batches of 33 to 64
// rows).  Measured against 2 x / A stages with 4 raw segments in flight: 3 and 3 is faster.
// The static checks below hold the budget.
#ifndef Q8_DEPTH_64
#define Q8_DEPTH_64 3
#endif
#ifndef Q8_RAW_64
#define Q8_RAW_64 3
#endif

template <int NTOK>
struct StreamShape {
    // A (TMEM) and x (shared) segment stages
    static constexpr uint32_t depth = NTOK <= 32 ? 3 : (NTOK == 64 ? Q8_DEPTH_64 : 2);
    static constexpr uint32_t raw_stages = NTOK <= 32 ? 5 : (NTOK == 64 ? Q8_RAW_64 : 2);
    static constexpr uint32_t x_sub_bytes = NTOK * kSubK * 2;        // one [NTOK x 64] swizzled box
    static constexpr uint32_t x_seg_bytes = kSubs * x_sub_bytes;     // four boxes = 256 weights deep
    static constexpr uint32_t a_column0 = NTOK <= 64 ? 128 : 256;    // after the two accumulators
    static constexpr uint32_t a_seg_columns = kSegK / 2;             // 128 words per row per segment
    static constexpr uint32_t tmem_columns = 512;
    static constexpr uint32_t x_offset = 0;
    static constexpr uint32_t raw_offset = x_offset + depth * x_seg_bytes;
    static constexpr uint32_t bar_offset = raw_offset + raw_stages * kRawStageBytes;
    static constexpr uint32_t bar_count = 2 * raw_stages + 3 * depth + 4 + 1;
    // after the barriers: the storing warps' staging buffer (store_chunk_staged)
    // (token tiles of 64 and 128; the smaller ones, which only a development build reaches,
    // have no room for it beside their five raw stages)
    static constexpr uint32_t stage_offset = bar_offset + 256;
    static constexpr uint32_t stage_bytes = NTOK >= 64 ? kEpilogueWarps * kStoreStageBytes : 0;
    static constexpr uint32_t smem_bytes = stage_offset + stage_bytes + 1024;
    static_assert(bar_count * 8 + 16 <= 256, "barriers and the two words after them");
    static_assert(smem_bytes <= 227u * 1024u, "one block's shared memory");
    static_assert(a_column0 >= 2u * NTOK && a_column0 + depth * a_seg_columns <= tmem_columns,
                  "two accumulators, then the A segments, within the allocation");
};

template <int NTOK, typename YT>
__global__ void __launch_bounds__(kThreads, 1)
q8_stream_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 const UmmaArgs args)
{
    using S = StreamShape<NTOK>;
    extern __shared__ unsigned char smem_raw_[];
    const uint32_t smem0 = (smem_u32(smem_raw_) + 1023u) & ~1023u;
    const uint32_t x_base = smem0 + S::x_offset;
    const uint32_t raw_base = smem0 + S::raw_offset;
    const uint32_t bar_base = smem0 + S::bar_offset;
    const uint32_t raw_full = bar_base;
    const uint32_t raw_empty = raw_full + 8u * S::raw_stages;
    const uint32_t x_full = raw_empty + 8u * S::raw_stages;
    const uint32_t a_full = x_full + 8u * S::depth;
    const uint32_t seg_empty = a_full + 8u * S::depth;   // A piece and x piece of a stage are free
    const uint32_t acc_full = seg_empty + 8u * S::depth;
    const uint32_t acc_empty = acc_full + 16u;
    const uint32_t drain_bar = acc_empty + 16u;
    const uint32_t tmem_slot = drain_bar + 8u;
    unsigned char *generic0 = smem_raw_ + (smem0 - smem_u32(smem_raw_));
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(generic0 + (tmem_slot - smem0));
    volatile uint32_t *abort_flag = tmem_slot_ptr + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;

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
    unsigned long long units = (unsigned long long)row_tiles * tok_tiles * segs;
    if (args.group_tiles != nullptr) {
        // the table was built by the kernel before this one on the stream
        grid_dependency_wait();
        units = (unsigned long long)(*args.group_count) * segs;
    }
    // No more blocks than units take part, so that every block in the schedule has work.
    const unsigned int blocks = units < gridDim.x ? (unsigned int)units : gridDim.x;
    if (blockIdx.x >= blocks) {
        return;
    }
    unsigned long long u_begin, u_end;
    unit_range(blockIdx.x, blocks, units, &u_begin, &u_end);

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < S::raw_stages; ++i) {
            mbar_init(raw_full + 8u * i, 1u);
            mbar_init(raw_empty + 8u * i, 8u);
        }
        for (uint32_t i = 0; i < S::depth; ++i) {
            mbar_init(x_full + 8u * i, 1u);
            mbar_init(a_full + 8u * i, 8u);
            mbar_init(seg_empty + 8u * i, 1u);
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
            // the table entry of a tile is fetched one tile ahead: a trip to memory at every
            // change of tile would leave the ring of copies idle for that long
            TilePlace ahead = tile_place<NTOK>(args, (uint32_t)(u_begin / segs), tok_tiles, m);
            for (unsigned long long u = u_begin; ok && u < u_end;) {
                const uint32_t tile = (uint32_t)(u / segs);
                const uint32_t s0 = (uint32_t)(u % segs);
                const unsigned long long left = u_end - u;
                const uint32_t s1 = (segs - s0) < left ? segs : (uint32_t)(s0 + left);
                const uint32_t w_row = ahead.w_row;
                if (u + (s1 - s0) < u_end) {
                    ahead = tile_place<NTOK>(args, tile + 1u, tok_tiles, m);
                }
                for (uint32_t s = s0; s < s1; ++s, ++g) {
                    const uint32_t st = g % S::raw_stages;
                    const uint32_t ph = (g / S::raw_stages) & 1u;
                    if (!mbar_wait(raw_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(raw_full + 8u * st, kRawStageBytes);
                    tma_load_2d(raw_base + st * kRawStageBytes, &tmap_w, raw_full + 8u * st,
                                (int)(s * kSegWords), (int)w_row);
                }
                u += (s1 - s0);
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
        // ---------------------------------------------------------------- x copies
        if (lane == 0u) {
            uint32_t g = 0;
            grid_dependency_wait();
            bool ok = true;
            TilePlace ahead = tile_place<NTOK>(args, (uint32_t)(u_begin / segs), tok_tiles, m);
            for (unsigned long long u = u_begin; ok && u < u_end;) {
                const uint32_t tile = (uint32_t)(u / segs);
                const uint32_t s0 = (uint32_t)(u % segs);
                const unsigned long long left = u_end - u;
                const uint32_t s1 = (segs - s0) < left ? segs : (uint32_t)(s0 + left);
                const uint32_t tok0 = ahead.i0;   // fetched one tile ahead, as the weight copies do
                if (u + (s1 - s0) < u_end) {
                    ahead = tile_place<NTOK>(args, tile + 1u, tok_tiles, m);
                }
                for (uint32_t s = s0; s < s1; ++s, ++g) {
                    const uint32_t st = g % S::depth;
                    const uint32_t ph = (g / S::depth) & 1u;
                    if (!mbar_wait(seg_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(x_full + 8u * st, S::x_seg_bytes);
#pragma unroll
                    for (uint32_t j = 0; j < kSubs; ++j) {
                        tma_load_2d(x_base + st * S::x_seg_bytes + j * S::x_sub_bytes, &tmap_x,
                                    x_full + 8u * st, (int)(s * kSegK + j * kSubK),
                                    (int)tok0);
                    }
                }
                u += (s1 - s0);
            }
            uint32_t local_abort = 0;
            const uint32_t first = g > S::depth ? g - S::depth : 0u;
            for (uint32_t i = first; i < g; ++i) {
                mbar_wait(x_full + 8u * (i % S::depth), (i / S::depth) & 1u, &local_abort, nullptr);
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0u) {
            // bfloat16 activations were turned into binary16 in shared memory by the converters
            uint32_t idesc = umma_idesc(kRows, (uint32_t)NTOK, 0u, 0u);
            uint32_t g = 0;
            uint32_t tc = 0;
            bool ok = true;
            for (unsigned long long u = u_begin; ok && u < u_end; ++tc) {
                const uint32_t s0 = (uint32_t)(u % segs);
                const unsigned long long left = u_end - u;
                const uint32_t s1 = (segs - s0) < left ? segs : (uint32_t)(s0 + left);
                const uint32_t buf = tc & 1u;
                const uint32_t aph = (tc >> 1) & 1u;
                if (!mbar_wait(acc_empty + 8u * buf, aph ^ 1u, abort_flag, args.status)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * (uint32_t)NTOK;
                uint32_t accumulate = 0u;
                for (uint32_t s = s0; s < s1; ++s, ++g) {
                    const uint32_t st = g % S::depth;
                    const uint32_t ph = (g / S::depth) & 1u;
                    if (!mbar_wait(a_full + 8u * st, ph, abort_flag, args.status)
                        || !mbar_wait(x_full + 8u * st, ph, abort_flag, args.status)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_tmem = tmem_base + S::a_column0 + st * S::a_seg_columns;
#pragma unroll
                    for (uint32_t j = 0; j < kSubs; ++j) {
                        const uint64_t b_desc = umma_desc_sw128(x_base + st * S::x_seg_bytes + j * S::x_sub_bytes);
#pragma unroll
                        for (uint32_t kk = 0; kk < kSubK / 16u; ++kk) {
                            // 16 halves: 8 columns of A, 32 bytes along the swizzled row of x
                            umma_f16_ts(d_tmem, a_tmem + j * (kSubK / 2u) + 8u * kk, b_desc + 2u * kk, idesc,
                                        accumulate);
                            accumulate = 1u;
                        }
                    }
                    umma_commit(seg_empty + 8u * st);
                }
                if (ok) {
                    umma_commit(acc_full + 8u * buf);
                }
                u += (s1 - s0);
            }
            if (!ok) {
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
        // this warp owns TMEM lanes [32 (cw & 3), +32): its rows of the tile
        const uint32_t lane_base = tmem_base + (((cw & 3u) * 32u) << 16) + S::a_column0 + half_id * kSegK / 4u;
        uint32_t g = 0;
        bool ok = true;
        for (unsigned long long u = u_begin; ok && u < u_end;) {
            const uint32_t s0 = (uint32_t)(u % segs);
            const unsigned long long left = u_end - u;
            const uint32_t s1 = (segs - s0) < left ? segs : (uint32_t)(s0 + left);
            for (uint32_t s = s0; s < s1; ++s, ++g) {
                const uint32_t rst = g % S::raw_stages;
                const uint32_t rph = (g / S::raw_stages) & 1u;
                if (!mbar_wait(raw_full + 8u * rst, rph, abort_flag, args.status)) {
                    ok = false;
                    break;
                }
                uint32_t raw[36];
                const uint32_t raw_row = raw_base + rst * kRawStageBytes + row * kSegBytes;
                if (half_id == 0u) {
                    load_raw<0>(raw_row, raw);
                } else {
                    load_raw<1>(raw_row, raw);
                }
                raw_words_present(raw, args.status);
                __syncwarp();
                if (lane == 0u) {
                    mbar_arrive(raw_empty + 8u * rst);
                }
                const uint32_t st = g % S::depth;
                const uint32_t ph = (g / S::depth) & 1u;
                if (!mbar_wait(seg_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                    ok = false;
                    break;
                }
                {
                    const uint32_t taddr = lane_base + st * S::a_seg_columns;
                    tc_fence_after_sync();
                    if (half_id == 0u) {
                        convert_stage_tmem<0, 0>(raw, taddr);
                        convert_stage_tmem<0, 1>(raw, taddr + kSubK / 2u);
                    } else {
                        convert_stage_tmem<1, 0>(raw, taddr);
                        convert_stage_tmem<1, 1>(raw, taddr + kSubK / 2u);
                    }
                    tmem_st_wait();
                    tc_fence_before_sync();
                }
                if (args.b_bf16 != 0u) {
                    // One MMA takes both operands in one format: turn this segment's x tile into
                    // binary16 where it lies (the swizzle moves whole 16-byte chunks, so the
                    // conversion is chunk by chunk whatever the layout).
                    if (!mbar_wait(x_full + 8u * st, ph, abort_flag, args.status)) {
                        ok = false;
                        break;
                    }
                    const uint32_t x_seg = x_base + st * S::x_seg_bytes;
                    for (uint32_t c = cw * 32u + lane; c < S::x_seg_bytes / 16u; c += 256u) {
                        bf16_chunk_to_f16_inplace(x_seg + 16u * c);
                    }
                    fence_proxy_async_smem();
                }
                __syncwarp();
                if (lane == 0u) {
                    mbar_arrive(a_full + 8u * st);
                }
            }
            u += (s1 - s0);
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const uint32_t wq = warp;
        uint32_t tc = 0;
        grid_dependency_wait();
        bool ok = true;
        for (unsigned long long u = u_begin; ok && u < u_end; ++tc) {
            const uint32_t tile = (uint32_t)(u / segs);
            const uint32_t s0 = (uint32_t)(u % segs);
            const unsigned long long left = u_end - u;
            const uint32_t s1 = (segs - s0) < left ? segs : (uint32_t)(s0 + left);
            const uint32_t buf = tc & 1u;
            const uint32_t aph = (tc >> 1) & 1u;
            // where the tile goes (a table entry in grouped mode): asked for before the wait
            const TilePlace place = tile_place<NTOK>(args, tile, tok_tiles, m);
            if (!mbar_wait(acc_full + 8u * buf, aph, abort_flag, args.status)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            epilogue_piece<NTOK, YT>(args, tmem_base + buf * (uint32_t)NTOK, wq, lane, place, tile, s0, s1, segs,
                                     tok_tiles, units, blocks, m, abort_flag, acc_empty + 8u * buf,
                                     S::stage_bytes != 0u ? smem0 + S::stage_offset : 0u);
            u += (s1 - s0);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, S::tmem_columns);
    }
}

template <int NTOK, typename YT>
static cudaError_t launch_stream_typed(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                                       const UmmaArgs &args, unsigned int grid)
{
    using S = StreamShape<NTOK>;
    static unsigned long long configured = 0ull;
    cudaError_t err = allow_shared_memory(q8_stream_kernel<NTOK, YT>, S::smem_bytes, &configured);
    if (err != cudaSuccess) {
        return err;
    }
    return launch_tile_kernel(q8_stream_kernel<NTOK, YT>, grid, S::smem_bytes, stream, args.overlap != 0u, tw,
                              tx, args);
}

template <int NTOK>
static cudaError_t launch_stream_tile(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                                      const UmmaArgs &args, unsigned int grid, int y_dtype)
{
    switch (y_dtype) {
    case 0:
        return launch_stream_typed<NTOK, float>(stream, tw, tx, args, grid);
    case 1:
        return launch_stream_typed<NTOK, __half>(stream, tw, tx, args, grid);
    case 2:
        return launch_stream_typed<NTOK, __nv_bfloat16>(stream, tw, tx, args, grid);
    default:
        return cudaErrorInvalidValue;
    }
}

cudaError_t launch_stream_kernel(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                                 const UmmaArgs &args, unsigned int grid, unsigned int ntok, int y_dtype)
{
    switch (ntok) {
    case 16:
        return launch_stream_tile<16>(stream, tw, tx, args, grid, y_dtype);
    case 32:
        return launch_stream_tile<32>(stream, tw, tx, args, grid, y_dtype);
    case 64:
        return launch_stream_tile<64>(stream, tw, tx, args, grid, y_dtype);
    case 128:
        return launch_stream_tile<128>(stream, tw, tx, args, grid, y_dtype);
    default:
        return cudaErrorInvalidValue;
    }
}

} // namespace q8
