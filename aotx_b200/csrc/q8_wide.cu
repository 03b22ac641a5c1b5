// The prefill-regime kernel: batches above 128 rows of x, as token tiles of 256 rows, the
// dequantised weights in tensor memory.  It replaced an earlier form with both operands in
// shared memory, whose results differed in a few outputs from launch to launch on the GPU.
//
// What it takes from the two kernels it descends from:
//   * from the decode-regime kernel (q8_stream.cu): a converter thread owns one row of the weight
//     tile and writes its dequantised 64-weight pieces straight into its lane of tensor memory
//     (tcgen05.st); the MMA reads A from there.  No thread ever writes an MMA operand into shared
//     memory, so nothing depends on how stores by ordinary threads are ordered against reads by
//     the tensor core - the one thing the earlier form did that the decode-regime kernel does not;
//   * from the earlier form: the tile is 128 rows of w by 256 rows of x, so one pass of
//     dequantisation feeds twice the MMA work of a 128-row token tile; x comes in boxes of
//     [256 x 64] through a ring of its own (a whole 256-deep segment of x would be 128 KB);
//     whole waves of tiles are dealt round-robin and only the last partial wave is cut into
//     units.
// Tensor memory: the accumulator takes 256 columns and two segments of A take 128 each, which is
// all 512; there is one accumulator, so the MMAs of a tile start when the epilogue has read the
// tile before it (about 64 KB of stores against some 24 us of MMAs per tile at depth 4096).
// bfloat16 activations: the weights are rounded to bfloat16 (one rounding of the exact q * d)
// and both operands are bfloat16; x is never rewritten in shared memory.
//
// Warps as in the other two kernels: 0-3 epilogue, 4-11 converters, 12 raw weight copies, 13 x
// copies, 14 MMA issue.  Reference kernel replaced: cuda/model/gemm.cuh:55-189 (launched by
// cuda/model/graph_host.cu:25-29) for batches above 128 rows.
#include <cuda.h>
#include <stdlib.h>

#include "q8_launch.h"
#include "q8_tile.cuh"

namespace q8 {

struct WideShape {
    static constexpr uint32_t ntok = 256;
    static constexpr uint32_t a_stages = 2;                          // segments of A in tensor memory
    static constexpr uint32_t x_stages = 3;                          // [256 x 64] boxes of x
    static constexpr uint32_t raw_stages = 3;
    static constexpr uint32_t x_stage_bytes = ntok * kSubK * 2;
    static constexpr uint32_t a_column0 = ntok;                      // after the accumulator
    static constexpr uint32_t a_seg_columns = kSegK / 2;             // 128 words per row per segment
    static constexpr uint32_t tmem_columns = 512;
    static constexpr uint32_t x_offset = 0;
    static constexpr uint32_t raw_offset = x_offset + x_stages * x_stage_bytes;
    static constexpr uint32_t bar_offset = raw_offset + raw_stages * kRawStageBytes;
    static constexpr uint32_t bar_count = 2 * raw_stages + 2 * x_stages + 2 * a_stages + 2 + 1;
    // after the barriers: the storing warps' staging buffer (store_chunk_staged)
    static constexpr uint32_t stage_offset = bar_offset + 256;
    static constexpr uint32_t smem_bytes = stage_offset + kEpilogueWarps * kStoreStageBytes + 1024;
    static_assert(bar_count * 8 + 16 <= 256, "barriers and the two words after them");
    static_assert(smem_bytes <= 227u * 1024u, "one block's shared memory");
    static_assert(a_column0 >= ntok && a_column0 + a_stages * a_seg_columns <= tmem_columns,
                  "the accumulator, then the A segments, within the allocation");
};

template <typename YT>
__global__ void __launch_bounds__(kThreads, 1)
q8_wide_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const UmmaArgs args)
{
    using S = WideShape;
    constexpr int NTOK = (int)S::ntok;
    extern __shared__ unsigned char smem_raw_[];
    const uint32_t smem0 = (smem_u32(smem_raw_) + 1023u) & ~1023u;
    const uint32_t x_base = smem0 + S::x_offset;
    const uint32_t raw_base = smem0 + S::raw_offset;
    const uint32_t bar_base = smem0 + S::bar_offset;
    const uint32_t raw_full = bar_base;
    const uint32_t raw_empty = raw_full + 8u * S::raw_stages;
    const uint32_t x_full = raw_empty + 8u * S::raw_stages;
    const uint32_t x_empty = x_full + 8u * S::x_stages;
    const uint32_t a_full = x_empty + 8u * S::x_stages;
    const uint32_t a_empty = a_full + 8u * S::a_stages;
    const uint32_t acc_full = a_empty + 8u * S::a_stages;
    const uint32_t acc_empty = acc_full + 8u;
    const uint32_t drain_bar = acc_empty + 8u;
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
    // Whole waves of tiles are dealt round-robin (block b takes tiles b, b + G, ...: the token
    // tiles of one weight row tile then run at the same time on neighbouring SMs and share its
    // bytes in L2); the tiles of the last, partial wave are cut into units and spread evenly
    // over all blocks, first in every block's order of work.
    const unsigned long long tiles = (unsigned long long)row_tiles * tok_tiles;
    const uint32_t waves = (uint32_t)(tiles / gridDim.x);
    const uint32_t dp_tiles = waves * gridDim.x;
    const unsigned long long units = (tiles - dp_tiles) * segs;
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
            mbar_init(raw_empty + 8u * i, 8u);
        }
        for (uint32_t i = 0; i < S::x_stages; ++i) {
            mbar_init(x_full + 8u * i, 1u);
            mbar_init(x_empty + 8u * i, 1u);
        }
        for (uint32_t i = 0; i < S::a_stages; ++i) {
            mbar_init(a_full + 8u * i, 8u);
            mbar_init(a_empty + 8u * i, 1u);
        }
        mbar_init(acc_full, 1u);
        mbar_init(acc_empty, kEpilogueWarps);
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
                const uint32_t row_tile = tile / tok_tiles;
                for (uint32_t s = s0; s < s1; ++s, ++g) {
                    const uint32_t st = g % S::raw_stages;
                    const uint32_t ph = (g / S::raw_stages) & 1u;
                    if (!mbar_wait(raw_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                        ok = false;
                        break;
                    }
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
        // ---------------------------------------------------------------- x copies
        if (lane == 0u) {
            uint32_t q = 0;
            grid_dependency_wait();
            bool ok = true;
            WorkIter work = first_work;
            uint32_t tile = 0, s0 = 0, s1 = 0;
            for (; ok && work.next(tile, s0, s1);) {
                const uint32_t tok_tile = tile % tok_tiles;
                for (uint32_t s = s0; ok && s < s1; ++s) {
                    for (uint32_t j = 0; j < kSubs; ++j, ++q) {
                        const uint32_t st = q % S::x_stages;
                        const uint32_t ph = (q / S::x_stages) & 1u;
                        if (!mbar_wait(x_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                            ok = false;
                            break;
                        }
                        mbar_expect_tx(x_full + 8u * st, S::x_stage_bytes);
                        tma_load_2d(x_base + st * S::x_stage_bytes, &tmap_x, x_full + 8u * st,
                                    (int)(s * kSegK + j * kSubK), (int)(tok_tile * (uint32_t)NTOK));
                    }
                }
            }
            uint32_t local_abort = 0;
            const uint32_t first = q > S::x_stages ? q - S::x_stages : 0u;
            for (uint32_t i = first; i < q; ++i) {
                mbar_wait(x_full + 8u * (i % S::x_stages), (i / S::x_stages) & 1u, &local_abort, nullptr);
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0u) {
            const uint32_t idesc = umma_idesc(kRows, (uint32_t)NTOK, args.b_bf16, args.b_bf16);
            uint32_t g = 0;
            uint32_t q = 0;
            uint32_t tc = 0;
            bool ok = true;
            WorkIter work = first_work;
            uint32_t tile = 0, s0 = 0, s1 = 0;
            for (; ok && work.next(tile, s0, s1); ++tc) {
                (void)tile;
                // one accumulator: the epilogue has read the piece before this one
                if (!mbar_wait(acc_empty, (tc & 1u) ^ 1u, abort_flag, args.status)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base;
                uint32_t accumulate = 0u;
                for (uint32_t s = s0; ok && s < s1; ++s, ++g) {
                    const uint32_t st = g % S::a_stages;
                    const uint32_t ph = (g / S::a_stages) & 1u;
                    if (!mbar_wait(a_full + 8u * st, ph, abort_flag, args.status)) {
                        ok = false;
                        break;
                    }
                    const uint32_t a_tmem = tmem_base + S::a_column0 + st * S::a_seg_columns;
                    for (uint32_t j = 0; j < kSubs; ++j, ++q) {
                        const uint32_t xst = q % S::x_stages;
                        const uint32_t xph = (q / S::x_stages) & 1u;
                        if (!mbar_wait(x_full + 8u * xst, xph, abort_flag, args.status)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint64_t b_desc = umma_desc_sw128(x_base + xst * S::x_stage_bytes);
#pragma unroll
                        for (uint32_t kk = 0; kk < kSubK / 16u; ++kk) {
                            // 16 halves: 8 columns of A, 32 bytes along the swizzled row of x
                            umma_f16_ts(d_tmem, a_tmem + j * (kSubK / 2u) + 8u * kk, b_desc + 2u * kk, idesc,
                                        accumulate);
                            accumulate = 1u;
                        }
                        umma_commit(x_empty + 8u * xst);
                    }
                    if (ok) {
                        umma_commit(a_empty + 8u * st);
                    }
                }
                if (ok) {
                    umma_commit(acc_full);
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
        // this warp owns TMEM lanes [32 (cw & 3), +32): its rows of the tile
        const uint32_t lane_base = tmem_base + (((cw & 3u) * 32u) << 16) + S::a_column0 + half_id * kSegK / 4u;
        uint32_t g = 0;
        bool ok = true;
        WorkIter work = first_work;
        uint32_t tile = 0, s0 = 0, s1 = 0;
        for (; ok && work.next(tile, s0, s1);) {
            (void)tile;
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
                const uint32_t st = g % S::a_stages;
                const uint32_t ph = (g / S::a_stages) & 1u;
                if (!mbar_wait(a_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                    ok = false;
                    break;
                }
                const uint32_t taddr = lane_base + st * S::a_seg_columns;
                tc_fence_after_sync();
                if (args.b_bf16 != 0u) {
                    if (half_id == 0u) {
                        convert_stage_tmem<0, 0, true>(raw, taddr);
                        convert_stage_tmem<0, 1, true>(raw, taddr + kSubK / 2u);
                    } else {
                        convert_stage_tmem<1, 0, true>(raw, taddr);
                        convert_stage_tmem<1, 1, true>(raw, taddr + kSubK / 2u);
                    }
                } else if (half_id == 0u) {
                    convert_stage_tmem<0, 0, false>(raw, taddr);
                    convert_stage_tmem<0, 1, false>(raw, taddr + kSubK / 2u);
                } else {
                    convert_stage_tmem<1, 0, false>(raw, taddr);
                    convert_stage_tmem<1, 1, false>(raw, taddr + kSubK / 2u);
                }
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0u) {
                    mbar_arrive(a_full + 8u * st);
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const uint32_t wq = warp;
        uint32_t tc = 0;
        grid_dependency_wait();
        bool ok = true;
        WorkIter work = first_work;
        uint32_t tile = 0, s0 = 0, s1 = 0;
        for (; ok && work.next(tile, s0, s1); ++tc) {
            if (!mbar_wait(acc_full, tc & 1u, abort_flag, args.status)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            epilogue_piece<NTOK, YT>(args, tmem_base, wq, lane, tile_place<NTOK>(args, tile, tok_tiles, m),
                                     tile >= first_work.sk_tile0 ? tile - first_work.sk_tile0 : 0u, s0, s1, segs,
                                     tok_tiles, units, blocks, m, abort_flag, acc_empty, smem0 + S::stage_offset);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, S::tmem_columns);
    }
}

template <typename YT>
static cudaError_t launch_wide_typed(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                                     const UmmaArgs &args, unsigned int grid)
{
    static unsigned long long configured = 0ull;
    cudaError_t err = allow_shared_memory(q8_wide_kernel<YT>, WideShape::smem_bytes, &configured);
    if (err != cudaSuccess) {
        return err;
    }
    return launch_tile_kernel(q8_wide_kernel<YT>, grid, WideShape::smem_bytes, stream, args.overlap != 0u, tw, tx,
                              args);
}

cudaError_t launch_wide_kernel(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                               const UmmaArgs &args, unsigned int grid, int y_dtype)
{
    switch (y_dtype) {
    case 0:
        return launch_wide_typed<float>(stream, tw, tx, args, grid);
    case 1:
        return launch_wide_typed<__half>(stream, tw, tx, args, grid);
    case 2:
        return launch_wide_typed<__nv_bfloat16>(stream, tw, tx, args, grid);
    default:
        return cudaErrorInvalidValue;
    }
}

} // namespace q8
