// The decode-regime kernel in a form of which two blocks fit on one SM (token tiles of 16 and
// 32 rows of x).  NOT DISPATCHED by the product build: written to test one idea on the GPU,
// checked so far only on the tests' host emulation; a build with -DQ8_EXPERIMENT reaches it with
// Q8_DUO=1 in the environment.
//
// The idea.  A decode step is a chain of products of 18 to 125 MB, each of which depends on the
// one before it.  With one block per SM (q8_stream.cu: 480 threads of 128 registers, 200 KB of
// shared memory, all of tensor memory) a block of the next launch cannot start on an SM before
// the block of this launch has left it, so every launch pays its own set-up, the memory latency
// of its first copies and its own tail - about 8 us per launch, more than the transfer time of
// the small projections.  Two lighter blocks per SM overlap these: while one block stores its
// last tile, or waits for the launch before it to finish, the other block's copies are in
// flight; and with programmatic dependent launch a block of the next product starts on an SM,
// sets itself up and streams and dequantises its first weights as soon as ONE of the two blocks
// there has left.
//
// What a block is here: 352 threads (warps 0-3 epilogue, 4-7 converters, 8 raw weight copies,
// 9 x copies, 10 MMA issue), 80 registers and no spills, about 101 KB of shared memory (two raw
// segments of 34 KB in flight, two x segments), 256 columns of tensor memory (two accumulators
// of NTOK columns, three A pieces of 64 columns).  A converter thread still owns one row of the
// weight tile, but takes the two halves of a 256-weight segment one after the other, and the
// hand-over to the MMA thread is per half segment (8 MMAs).  Tiling, unit schedule, fix-up of
// cut tiles and stores are those of q8_stream.cu (q8_tile.cuh).  bfloat16 activations: the
// weights are rounded to bfloat16 (one rounding of the exact q * d) and both MMA operands are
// bfloat16; x is not rewritten in shared memory.
//
// Reference kernels replaced: ptx/gemv_q8.ptx:18-223, cuda/model/gemv.cuh:33-145.
#include <cuda.h>
#include <stdlib.h>

#include "q8_launch.h"
#include "q8_tile.cuh"

namespace q8 {

constexpr uint32_t kDuoThreads = 352;
constexpr uint32_t kDuoConvertWarp0 = 4;
constexpr uint32_t kDuoConvertWarps = 4;
constexpr uint32_t kDuoWeightWarp = 8;
constexpr uint32_t kDuoInputWarp = 9;
constexpr uint32_t kDuoMmaWarp = 10;

template <int NTOK>
struct DuoShape {
    static_assert(NTOK == 16 || NTOK == 32, "two accumulators and three A pieces in 256 columns");
    static constexpr uint32_t raw_stages = 2;
    static constexpr uint32_t x_depth = 2;                           // x segments in shared memory
    static constexpr uint32_t a_stages = 3;                          // half segments of A in tensor memory
    static constexpr uint32_t x_sub_bytes = NTOK * kSubK * 2;        // one [NTOK x 64] swizzled box
    static constexpr uint32_t x_seg_bytes = kSubs * x_sub_bytes;     // four boxes = 256 weights deep
    static constexpr uint32_t a_column0 = 64;                        // after the two accumulators
    static constexpr uint32_t a_stage_columns = kSegK / 4;           // 64 words per row per half segment
    static constexpr uint32_t tmem_columns = 256;
    static constexpr uint32_t x_offset = 0;
    static constexpr uint32_t raw_offset = x_offset + x_depth * x_seg_bytes;
    static constexpr uint32_t bar_offset = raw_offset + raw_stages * kRawStageBytes;
    static constexpr uint32_t bar_count = 2 * raw_stages + 2 * x_depth + 2 * a_stages + 4 + 1;
    static constexpr uint32_t smem_bytes = bar_offset + bar_count * 8 + 16 + 1024;
    // two blocks and the 1 KB the system keeps per block within the 228 KB of an SM
    static_assert(2u * (smem_bytes + 1024u) <= 228u * 1024u, "two blocks' shared memory on one SM");
    static_assert(a_column0 >= 2u * NTOK && a_column0 + a_stages * a_stage_columns <= tmem_columns
                      && 2u * tmem_columns <= 512u,
                  "two accumulators, then the A pieces, in half of the tensor memory");
};

template <int NTOK, typename YT>
__global__ void __launch_bounds__(kDuoThreads, 2)
q8_duo_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
              const UmmaArgs args)
{
    using S = DuoShape<NTOK>;
    extern __shared__ unsigned char smem_raw_[];
    const uint32_t smem0 = (smem_u32(smem_raw_) + 1023u) & ~1023u;
    const uint32_t x_base = smem0 + S::x_offset;
    const uint32_t raw_base = smem0 + S::raw_offset;
    const uint32_t bar_base = smem0 + S::bar_offset;
    const uint32_t raw_full = bar_base;
    const uint32_t raw_empty = raw_full + 8u * S::raw_stages;
    const uint32_t x_full = raw_empty + 8u * S::raw_stages;
    const uint32_t x_empty = x_full + 8u * S::x_depth;
    const uint32_t a_full = x_empty + 8u * S::x_depth;
    const uint32_t a_empty = a_full + 8u * S::a_stages;
    const uint32_t acc_full = a_empty + 8u * S::a_stages;
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
            mbar_init(raw_empty + 8u * i, kDuoConvertWarps);
        }
        for (uint32_t i = 0; i < S::x_depth; ++i) {
            mbar_init(x_full + 8u * i, 1u);
            mbar_init(x_empty + 8u * i, 1u);
        }
        for (uint32_t i = 0; i < S::a_stages; ++i) {
            mbar_init(a_full + 8u * i, kDuoConvertWarps);
            mbar_init(a_empty + 8u * i, 1u);
        }
        for (uint32_t i = 0; i < 2u; ++i) {
            mbar_init(acc_full + 8u * i, 1u);
            mbar_init(acc_empty + 8u * i, kEpilogueWarps);
        }
        mbar_init(drain_bar, 1u);
        *abort_flag = 0u;
        mbar_init_fence();
    }
    if (warp == kDuoWeightWarp && lane == 0u) {
        tma_prefetch_desc(&tmap_w);
    }
    if (warp == kDuoInputWarp && lane == 0u) {
        tma_prefetch_desc(&tmap_x);
    }
    if (warp == kDuoMmaWarp) {
        tmem_alloc(tmem_slot, S::tmem_columns);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == kDuoWeightWarp) {
        // ---------------------------------------------------------------- raw weight copies
        if (lane == 0u) {
            uint32_t g = 0;
            bool ok = true;
            for (unsigned long long u = u_begin; ok && u < u_end;) {
                const uint32_t tile = (uint32_t)(u / segs);
                const uint32_t s0 = (uint32_t)(u % segs);
                const unsigned long long left = u_end - u;
                const uint32_t s1 = (segs - s0) < left ? segs : (uint32_t)(s0 + left);
                const uint32_t w_row = tile_place<NTOK>(args, tile, tok_tiles, m).w_row;
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
            if (ok && args.next_w != nullptr) {
                prefetch_next_units(args);
            }
            // Let every copy this thread started land before the block ends.
            uint32_t local_abort = 0;
            const uint32_t first = g > S::raw_stages ? g - S::raw_stages : 0u;
            for (uint32_t i = first; i < g; ++i) {
                mbar_wait(raw_full + 8u * (i % S::raw_stages), (i / S::raw_stages) & 1u, &local_abort,
                          nullptr);
            }
        }
    } else if (warp == kDuoInputWarp) {
        // ---------------------------------------------------------------- x copies
        if (lane == 0u) {
            uint32_t g = 0;
            grid_dependency_wait();
            bool ok = true;
            for (unsigned long long u = u_begin; ok && u < u_end;) {
                const uint32_t tile = (uint32_t)(u / segs);
                const uint32_t s0 = (uint32_t)(u % segs);
                const unsigned long long left = u_end - u;
                const uint32_t s1 = (segs - s0) < left ? segs : (uint32_t)(s0 + left);
                const uint32_t tok0 = tile_place<NTOK>(args, tile, tok_tiles, m).i0;
                for (uint32_t s = s0; s < s1; ++s, ++g) {
                    const uint32_t st = g % S::x_depth;
                    const uint32_t ph = (g / S::x_depth) & 1u;
                    if (!mbar_wait(x_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(x_full + 8u * st, S::x_seg_bytes);
#pragma unroll
                    for (uint32_t j = 0; j < kSubs; ++j) {
                        tma_load_2d(x_base + st * S::x_seg_bytes + j * S::x_sub_bytes, &tmap_x,
                                    x_full + 8u * st, (int)(s * kSegK + j * kSubK), (int)tok0);
                    }
                }
                u += (s1 - s0);
            }
            uint32_t local_abort = 0;
            const uint32_t first = g > S::x_depth ? g - S::x_depth : 0u;
            for (uint32_t i = first; i < g; ++i) {
                mbar_wait(x_full + 8u * (i % S::x_depth), (i / S::x_depth) & 1u, &local_abort, nullptr);
            }
        }
    } else if (warp == kDuoMmaWarp) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0u) {
            const uint32_t idesc = umma_idesc(kRows, (uint32_t)NTOK, args.b_bf16, args.b_bf16);
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
                for (uint32_t s = s0; ok && s < s1; ++s, ++g) {
                    const uint32_t xst = g % S::x_depth;
                    const uint32_t xph = (g / S::x_depth) & 1u;
                    if (!mbar_wait(x_full + 8u * xst, xph, abort_flag, args.status)) {
                        ok = false;
                        break;
                    }
                    for (uint32_t half = 0; half < 2u; ++half) {
                        const uint32_t hh = 2u * g + half;
                        const uint32_t st = hh % S::a_stages;
                        const uint32_t ph = (hh / S::a_stages) & 1u;
                        if (!mbar_wait(a_full + 8u * st, ph, abort_flag, args.status)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t a_tmem = tmem_base + S::a_column0 + st * S::a_stage_columns;
#pragma unroll
                        for (uint32_t jl = 0; jl < 2u; ++jl) {
                            const uint32_t j = 2u * half + jl;
                            const uint64_t b_desc =
                                umma_desc_sw128(x_base + xst * S::x_seg_bytes + j * S::x_sub_bytes);
#pragma unroll
                            for (uint32_t kk = 0; kk < kSubK / 16u; ++kk) {
                                // 16 values: 8 columns of A, 32 bytes along the swizzled row of x
                                umma_f16_ts(d_tmem, a_tmem + jl * (kSubK / 2u) + 8u * kk, b_desc + 2u * kk, idesc,
                                            accumulate);
                                accumulate = 1u;
                            }
                        }
                        umma_commit(a_empty + 8u * st);
                    }
                    if (ok) {
                        umma_commit(x_empty + 8u * xst);
                    }
                }
                if (ok) {
                    umma_commit(acc_full + 8u * buf);
                }
                u += (s1 - s0);
            }
            if (!ok) {
                // Outstanding MMAs must finish before the tensor memory goes back.
                uint32_t local_abort = 0;
                umma_commit(drain_bar);
                mbar_wait(drain_bar, 0u, &local_abort, nullptr);
            }
        }
    } else if (warp >= kDuoConvertWarp0) {
        // ---------------------------------------------------------------- dequantise
        const uint32_t cw = warp - kDuoConvertWarp0;
        const uint32_t row = cw * 32u + lane;
        // this warp owns TMEM lanes [32 cw, +32): its rows of the tile
        const uint32_t lane_base = tmem_base + ((cw * 32u) << 16) + S::a_column0;
        uint32_t g = 0;
        bool ok = true;
        for (unsigned long long u = u_begin; ok && u < u_end;) {
            const uint32_t s0 = (uint32_t)(u % segs);
            const unsigned long long left = u_end - u;
            const uint32_t s1 = (segs - s0) < left ? segs : (uint32_t)(s0 + left);
            for (uint32_t s = s0; ok && s < s1; ++s, ++g) {
                const uint32_t rst = g % S::raw_stages;
                const uint32_t rph = (g / S::raw_stages) & 1u;
                if (!mbar_wait(raw_full + 8u * rst, rph, abort_flag, args.status)) {
                    ok = false;
                    break;
                }
                const uint32_t raw_row = raw_base + rst * kRawStageBytes + row * kSegBytes;
#pragma unroll
                for (uint32_t half = 0; half < 2u; ++half) {
                    uint32_t raw[36];
                    if (half == 0u) {
                        load_raw<0>(raw_row, raw);
                    } else {
                        load_raw<1>(raw_row, raw);
                        // the second half is in registers: the raw segment may be overwritten
                        __syncwarp();
                        if (lane == 0u) {
                            mbar_arrive(raw_empty + 8u * rst);
                        }
                    }
                    const uint32_t hh = 2u * g + half;
                    const uint32_t st = hh % S::a_stages;
                    const uint32_t ph = (hh / S::a_stages) & 1u;
                    if (!mbar_wait(a_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                        ok = false;
                        break;
                    }
                    const uint32_t taddr = lane_base + st * S::a_stage_columns;
                    tc_fence_after_sync();
                    if (args.b_bf16 != 0u) {
                        if (half == 0u) {
                            convert_stage_tmem<0, 0, true>(raw, taddr);
                            convert_stage_tmem<0, 1, true>(raw, taddr + kSubK / 2u);
                        } else {
                            convert_stage_tmem<1, 0, true>(raw, taddr);
                            convert_stage_tmem<1, 1, true>(raw, taddr + kSubK / 2u);
                        }
                    } else if (half == 0u) {
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
            if (!mbar_wait(acc_full + 8u * buf, aph, abort_flag, args.status)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            // one block's partial sums in flight at a time: 80 registers hold that without spills
            epilogue_piece<NTOK, YT, false>(args, tmem_base + buf * (uint32_t)NTOK, wq, lane, tile, tile, s0, s1,
                                            segs, tok_tiles, units, blocks, m, abort_flag, acc_empty + 8u * buf);
            u += (s1 - s0);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == kDuoMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, S::tmem_columns);
    }
}

template <int NTOK, typename YT>
static cudaError_t launch_duo_typed(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                                    const UmmaArgs &args, unsigned int grid)
{
    using S = DuoShape<NTOK>;
    static unsigned long long configured = 0ull;
    cudaError_t err = allow_shared_memory(q8_duo_kernel<NTOK, YT>, S::smem_bytes, &configured, true);
    if (err != cudaSuccess) {
        return err;
    }
    return launch_tile_kernel(q8_duo_kernel<NTOK, YT>, grid, S::smem_bytes, stream, args.overlap != 0u, tw, tx,
                              args, kDuoThreads);
}

template <int NTOK>
static cudaError_t launch_duo_tile(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                                   const UmmaArgs &args, unsigned int grid, int y_dtype)
{
    switch (y_dtype) {
    case 0:
        return launch_duo_typed<NTOK, float>(stream, tw, tx, args, grid);
    case 1:
        return launch_duo_typed<NTOK, __half>(stream, tw, tx, args, grid);
    case 2:
        return launch_duo_typed<NTOK, __nv_bfloat16>(stream, tw, tx, args, grid);
    default:
        return cudaErrorInvalidValue;
    }
}

cudaError_t launch_duo_kernel(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                              const UmmaArgs &args, unsigned int grid, unsigned int ntok, int y_dtype)
{
    switch (ntok) {
    case 16:
        return launch_duo_tile<16>(stream, tw, tx, args, grid, y_dtype);
    case 32:
        return launch_duo_tile<32>(stream, tw, tx, args, grid, y_dtype);
    default:
        return cudaErrorInvalidValue;
    }
}

} // namespace q8
