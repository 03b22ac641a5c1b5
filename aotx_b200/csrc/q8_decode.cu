// The decode-regime kernel of the Q8_0 product for batches of up to 32 rows of x (one token
// tile of 16 or 32): y[i][j] = sum_c x[i][c] * half(q[j][c] * d[j][c / 32]), float sums.
//
// HBM-bound: a launch moves n * (k / 32) * 34 bytes of weights once, whatever the batch.  What
// decides the time of the 18 to 125 MB products of a decode step is not only the steady stream
// but the ends of a launch, so the kernel is built around these things:
//   * two blocks fit on one SM (352 threads, 80 registers, about 103 KB of shared memory, half
//     of the tensor memory each): while one block stores, or waits for the launch before it, the
//     other block's copies are in flight, and with programmatic dependent launch the blocks of
//     the next product start as soon as a place is free and stream and dequantise their first
//     weights while this product finishes; only x, the live batch and the stores wait for it;
//   * when the weight tensor has few row tiles (n up to about 9000), a tile is cut along k over
//     a CLUSTER of 2, 4 or 8 blocks, one piece each, and the pieces are summed through
//     distributed shared memory: every block writes each token column of its piece into the
//     shared memory of the block that owns the column, the owner adds the pieces in block order
//     and stores.  No global scratch, no flags to poll, and every block stores a share of the
//     tile;
//   * larger tensors run as (tile, segment) units dealt evenly over 2 blocks per SM.  A tile cut
//     between blocks belongs to the block that holds its first segment, which is that block's
//     last piece; the other holders publish their partial sums at the start of their ranges;
//   * successive MMAs of a piece go to 64 / NTOK accumulators in turn, which the store adds up:
//     an MMA of this shape does little work but takes about 0.1 us from issue to completion, and
//     MMAs into one accumulator run one after the other;
//   * the code is kept small (a short launch fetches its code cold, at its start and again at
//     its end): the accumulator is read and stored in chunks of 8 columns inside ordinary loops,
//     the store with every option (add, gated unit, several output buffers, row map) is one
//     out-of-line function beside a short inline path for the plain store, and a wait is out of
//     line too, except in the converters' loop.
//
// Inside a block (11 warps): warp 8 issues bulk tensor copies of raw weight segments
// [128 rows x 272 B] into a two-deep ring; warps 4-7 are converters, thread = row: nine 16-byte
// shared loads per half segment, exact dequantisation in registers, tcgen05.st of 64 packed
// words into the thread's lane of tensor memory (three half-segment stages), and - for bfloat16
// activations - a few 16-byte chunks of the segment's x tile turned into binary16 where it
// lies (one MMA takes both operands in one format; exact for magnitudes in [2^-14, 65504],
// saturating above); warp 10 issues tcgen05.mma 128 x NTOK x 16 with A from tensor memory and
// B = the x tile in shared memory (128-byte swizzle); warp 9 copies x tiles; warps 0-3 read the
// sums and store.  The schedule never depends on the live batch (one token tile), so the batch
// word is read only by the storing warps, after the launches before this one finished.  Every
// wait on a barrier or flag is bounded and raises a status bit when it runs out; after a wait
// the lanes of a warp vote, so that a wait that ends differently for two lanes (the bound runs
// out for one just as the phase completes for another) cannot leave a lane behind at a
// warp-wide step.
//
// Reference kernels replaced: ptx/gemv_q8.ptx:18-223, cuda/model/gemv.cuh:33-145 (and the
// three-node switch of cuda/model/graph_host.cu:31-39 for these batches).
#include <cuda.h>
#include <stdlib.h>

#include "q8_launch.h"
#include "q8_tile.cuh"

namespace q8 {

constexpr uint32_t kDecThreads = 352;
constexpr uint32_t kDecConvertWarp0 = 4;
constexpr uint32_t kDecConvertWarps = 4;
constexpr uint32_t kDecWeightWarp = 8;
constexpr uint32_t kDecInputWarp = 9;
constexpr uint32_t kDecMmaWarp = 10;
constexpr uint32_t kDecMaxCluster = 8;

template <int NTOK>
struct DecodeShape {
    static_assert(NTOK == 16 || NTOK == 32, "two accumulators and three A pieces in 256 columns");
    static constexpr uint32_t raw_stages = 2;
    static constexpr uint32_t x_depth = 2;                           // x segments in shared memory
    static constexpr uint32_t a_stages = 3;                          // half segments of A in tensor memory
    static constexpr uint32_t x_sub_bytes = NTOK * kSubK * 2;        // one [NTOK x 64] swizzled box
    static constexpr uint32_t x_seg_bytes = kSubs * x_sub_bytes;     // four boxes = 256 weights deep
    // The 64 accumulator columns hold 64 / NTOK sums of one piece: successive MMAs go to them in
    // turn and the store adds them up.  An MMA of this shape does little work but takes about
    // 0.1 us from issue to completion, and MMAs into one accumulator run one after the other, so
    // a single sum holds the whole block to sixteen such latencies per segment.
    static constexpr uint32_t chains = 64 / NTOK;
    static constexpr uint32_t a_column0 = 64;                        // after the accumulators
    static constexpr uint32_t a_stage_columns = kSegK / 4;           // 64 words per row per half segment
    static constexpr uint32_t tmem_columns = 256;
    static constexpr uint32_t x_offset = 0;
    static constexpr uint32_t raw_offset = x_offset + x_depth * x_seg_bytes;
    static constexpr uint32_t bar_offset = raw_offset + raw_stages * kRawStageBytes;
    static constexpr uint32_t bar_count = 2 * raw_stages + 3 * x_depth + 2 * a_stages + 4 + 1;
    static constexpr uint32_t smem_bytes = bar_offset + bar_count * 8 + 16 + 1024;
    // what a block receives from the other blocks of its cluster lies over the x ring, which is
    // idle by then: per sending block its share of the token columns, 128 floats each
    static constexpr uint32_t recv_bytes = (NTOK + kDecMaxCluster - 1u) * kRows * 4u;
    static_assert(recv_bytes <= x_depth * x_seg_bytes, "the exchange buffer fits in the x ring");
    // two blocks and the 1 KB the system keeps per block within the 228 KB of an SM
    static_assert(2u * (smem_bytes + 1024u) <= 228u * 1024u, "two blocks' shared memory on one SM");
    static_assert(a_column0 >= 2u * NTOK && a_column0 + a_stages * a_stage_columns <= tmem_columns
                      && 2u * tmem_columns <= 512u,
                  "two accumulators, then the A pieces, in half of the tensor memory");
};

#ifdef Q8_TRACE
#define Q8_STAMP(slot, cond)                                                         \
    if (args.trace != nullptr && (cond)) {                                           \
        unsigned long long t_;                                                       \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                       \
        args.trace[blockIdx.x * 8u + (slot)] = t_;                                   \
    }
#else
#define Q8_STAMP(slot, cond)
#endif

// The store with every option, once per kernel instance (see store_chunk in q8_tile.cuh).
template <typename YT>
static __device__ __noinline__ void store_eight_any(const UmmaArgs &args, const TilePlace &place, uint32_t lane_row,
                                                    uint32_t j, uint32_t first_row, uint32_t (&v)[8])
{
    store_chunk<8u, YT>(args, place, lane_row, j, first_row, v);
}

// The column-split store: the same eight sums into every GPU's copy of y.  Everything the
// stores need is in registers before the first of them (behind a call the compiler must assume
// that a store may have changed the argument block, and would fetch it again after each one),
// and a sum is rounded once, not once per copy.
template <typename YT>
static __device__ __noinline__ void store_eight_peers(const UmmaArgs &args, uint32_t i_limit, uint32_t j,
                                                      uint32_t first_row, uint32_t (&v)[8])
{
    const uint32_t peers = args.peers;
    const size_t ldy = args.ldy;
    const size_t col = args.col0 + j;
    YT *out[8];
#pragma unroll
    for (uint32_t p = 0; p < 8u; ++p) {
        out[p] = static_cast<YT *>(args.y_peer[p]);
    }
    float value[8];
#pragma unroll
    for (uint32_t i = 0; i < 8u; ++i) {
        value[i] = __uint_as_float(v[i]);
    }
#pragma unroll
    for (uint32_t p = 0; p < 8u; ++p) {
        if (p < peers) {
#pragma unroll
            for (uint32_t i = 0; i < 8u; ++i) {
                if (first_row + i < i_limit) {
                    store_out<YT>(out[p], (size_t)(first_row + i) * ldy + col, value[i]);
                }
            }
        }
    }
}

// Eight finished sums of column j of y, rows first_row .. first_row + 7 of x.
template <typename YT>
__device__ __forceinline__ void store_eight(const UmmaArgs &args, const TilePlace &place, uint32_t lane_row,
                                            uint32_t j, uint32_t first_row, uint32_t (&v)[8])
{
    if (args.epilogue == kEpilogueStore && args.row_map == nullptr) {
        if (j < place.j_limit && first_row < place.i_limit) {
            if (args.peers != 0u) {
                store_eight_peers<YT>(args, place.i_limit, j, first_row, v);
                return;
            }
            YT *y = static_cast<YT *>(args.y);
#pragma unroll
            for (uint32_t i = 0; i < 8u; ++i) {
                if (first_row + i < place.i_limit) {
                    store_out<YT>(y, (size_t)(first_row + i) * args.ldy + j, __uint_as_float(v[i]));
                }
            }
        }
        return;
    }
    store_eight_any<YT>(args, place, lane_row, j, first_row, v);
}

// Four finished sums of column j of y that lie `step` rows of x apart (the columns of a tile
// that one block of a cluster stores).
template <typename YT>
static __device__ __noinline__ void store_four_any(const UmmaArgs &args, const TilePlace &place, uint32_t lane_row,
                                                   uint32_t j, uint32_t first_row, uint32_t step, uint32_t (&v)[4])
{
    store_chunk<4u, YT>(args, place, lane_row, j, first_row, v, step);
}

template <typename YT>
__device__ __forceinline__ void store_four(const UmmaArgs &args, const TilePlace &place, uint32_t lane_row,
                                           uint32_t j, uint32_t first_row, uint32_t step, uint32_t (&v)[4])
{
    if (args.epilogue == kEpilogueStore && args.peers == 0u && args.row_map == nullptr) {
        if (j < place.j_limit) {
            YT *y = static_cast<YT *>(args.y);
#pragma unroll
            for (uint32_t i = 0; i < 4u; ++i) {
                if (first_row + i * step < place.i_limit) {
                    store_out<YT>(y, (size_t)(first_row + i * step) * args.ldy + j, __uint_as_float(v[i]));
                }
            }
        }
        return;
    }
    store_four_any<YT>(args, place, lane_row, j, first_row, step, v);
}

// Barriers and buffers of a block, as shared-space addresses.
struct DecodeRings {
    uint32_t x_base, raw_base;
    uint32_t raw_full, raw_empty, x_land, x_full, x_empty, a_full, a_empty, acc_full, acc_empty;
};

// Eight columns of a finished piece: the 64 / NTOK sums the MMAs went to in turn, added up.
template <int NTOK>
__device__ __forceinline__ void load_sums(uint32_t taddr, uint32_t (&v)[8])
{
    tmem_ld_32x8(taddr, v);
    tmem_ld_wait();
#pragma unroll
    for (uint32_t c = 1; c < 64u / (uint32_t)NTOK; ++c) {
        uint32_t more[8];
        tmem_ld_32x8(taddr + c * (uint32_t)NTOK, more);
        tmem_ld_wait();
#pragma unroll
        for (uint32_t i = 0; i < 8u; ++i) {
            v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(more[i]));
        }
    }
}

// One unit (a 256-weight segment of the block's 128 rows), half H of it: this thread's row from
// the raw ring into registers, exact dequantisation, 64 packed words into the thread's lane of
// the A stage.  The four warps of a half hand the stage over together.  (Handing a stage over
// one call later, so that the stores into tensor memory overlap the next fetch, was measured
// and is slower: with three stages the MMA thread then waits for its operand.)
template <int NTOK, int H>
__device__ __forceinline__ bool convert_unit(const DecodeRings &r, uint32_t g, uint32_t row, uint32_t lane,
                                             uint32_t lane_base, bool b_bf16, volatile uint32_t *abort_flag,
                                             unsigned int *status)
{
    using S = DecodeShape<NTOK>;
    const uint32_t rst = g % S::raw_stages;
    const uint32_t rph = (g / S::raw_stages) & 1u;
    // a wait can end differently for the lanes of a warp when the bound runs out for some just as
    // the phase completes for others: the warp decides together, so that no lane is left behind
    // at a warp-wide step
    if (!__all_sync(0xFFFFFFFFu, mbar_wait_hot(r.raw_full + 8u * rst, rph, abort_flag, status))) {
        return false;
    }
    uint32_t raw[36];
    load_raw<H>(r.raw_base + rst * kRawStageBytes + row * kSegBytes, raw);
    if (H == 1) {
        raw_words_present(raw, status);
        // both halves are in registers by now: as far as this warp goes, the raw segment may be
        // overwritten
        __syncwarp();
        if (lane == 0u) {
            mbar_arrive(r.raw_empty + 8u * rst);
        }
    }
    const uint32_t hh = 2u * g + (uint32_t)H;
    const uint32_t st = hh % S::a_stages;
    const uint32_t ph = (hh / S::a_stages) & 1u;
    if (!__all_sync(0xFFFFFFFFu, mbar_wait_hot(r.a_empty + 8u * st, ph ^ 1u, abort_flag, status))) {
        return false;
    }
    const uint32_t taddr = lane_base + st * S::a_stage_columns;
    tc_fence_after_sync();
    convert_stage_tmem<H, 0, false>(raw, taddr);
    convert_stage_tmem<H, 1, false>(raw, taddr + kSubK / 2u);
    tmem_st_wait();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0u) {
        mbar_arrive(r.a_full + 8u * st);
    }
    if (b_bf16) {
        // One MMA takes both operands in one format: the 256 converter threads turn the unit's
        // x segment into binary16 where it lies, a few 16-byte chunks each (the swizzle moves
        // whole chunks, so the conversion is chunk by chunk whatever the layout).  After the
        // weights, so that the conversion of weights never waits for x.
        const uint32_t xst = g % S::x_depth;
        const uint32_t xph = (g / S::x_depth) & 1u;
        if (!__all_sync(0xFFFFFFFFu, mbar_wait_hot(r.x_land + 8u * xst, xph, abort_flag, status))) {
            return false;
        }
        const uint32_t x_seg = r.x_base + xst * S::x_seg_bytes;
        const uint32_t me = (uint32_t)H * 128u + row;
#pragma unroll
        for (uint32_t c = 0; c < S::x_seg_bytes / 16u / 256u; ++c) {
            bf16_chunk_to_f16_inplace(x_seg + 16u * (me + 256u * c));
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0u) {
            mbar_arrive(r.x_full + 8u * xst);
        }
    }
    return true;
}

template <int NTOK, typename YT>
__global__ void __launch_bounds__(kDecThreads, 2)
q8_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 const UmmaArgs args)
{
    using S = DecodeShape<NTOK>;
    extern __shared__ unsigned char smem_raw_[];
    const uint32_t smem0 = (smem_u32(smem_raw_) + 1023u) & ~1023u;
    DecodeRings r;
    r.x_base = smem0 + S::x_offset;
    r.raw_base = smem0 + S::raw_offset;
    const uint32_t bar_base = smem0 + S::bar_offset;
    r.raw_full = bar_base;
    r.raw_empty = r.raw_full + 8u * S::raw_stages;
    r.x_land = r.raw_empty + 8u * S::raw_stages;  // the copy of an x segment is complete
    r.x_full = r.x_land + 8u * S::x_depth;        // ... and, for bfloat16 activations, turned into binary16
    r.x_empty = r.x_full + 8u * S::x_depth;
    r.a_full = r.x_empty + 8u * S::x_depth;
    r.a_empty = r.a_full + 8u * S::a_stages;
    r.acc_full = r.a_empty + 8u * S::a_stages;
    r.acc_empty = r.acc_full + 16u;
    const uint32_t drain_bar = r.acc_empty + 16u;
    const uint32_t tmem_slot = drain_bar + 8u;
    unsigned char *generic0 = smem_raw_ + (smem0 - smem_u32(smem_raw_));
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(generic0 + (tmem_slot - smem0));
    volatile uint32_t *abort_flag = tmem_slot_ptr + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    Q8_STAMP(0u, threadIdx.x == 0u)

    // The next kernel on the stream may start its blocks beside this one's.  Work that only
    // reads the weights runs ahead of the kernels before this one; everything that reads x or
    // the live batch, or writes y or the scratch slots, first waits for them to finish.
    grid_launch_dependents();

    const uint32_t segs = args.k / kSegK;
    const uint32_t row_tiles = (args.n + kRows - 1u) / kRows;
    const uint32_t units = row_tiles * segs; // the host refuses products with 2^31 units or more
    const bool split = args.split != 0u;
    uint32_t crank = 0u;
    uint32_t csize = 1u;
    uint32_t blocks = gridDim.x;
    uint32_t u_begin, u_end;
    if (split) {
        // one tile per cluster, one run of its segments per block
        csize = cluster_nctarank();
        crank = cluster_ctarank();
        const uint32_t tile = blockIdx.x / csize;
        u_begin = tile * segs + crank * segs / csize;
        u_end = tile * segs + (crank + 1u) * segs / csize;
    } else {
        // No more blocks than units take part, so that every block in the schedule has work.
        blocks = units < gridDim.x ? units : gridDim.x;
        if (blockIdx.x >= blocks) {
            return;
        }
        decode_range(blockIdx.x, blocks, units, &u_begin, &u_end);
    }
    const uint32_t tile_begin = u_begin / segs;      // the tile and segment of the first unit
    const uint32_t seg_begin = u_begin - tile_begin * segs;

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < S::raw_stages; ++i) {
            mbar_init(r.raw_full + 8u * i, 1u);
            mbar_init(r.raw_empty + 8u * i, kDecConvertWarps);
        }
        for (uint32_t i = 0; i < S::x_depth; ++i) {
            mbar_init(r.x_land + 8u * i, 1u);
            mbar_init(r.x_full + 8u * i, 2u * kDecConvertWarps);
            mbar_init(r.x_empty + 8u * i, 1u);
        }
        for (uint32_t i = 0; i < S::a_stages; ++i) {
            mbar_init(r.a_full + 8u * i, kDecConvertWarps);
            mbar_init(r.a_empty + 8u * i, 1u);
        }
        for (uint32_t i = 0; i < 2u; ++i) {
            mbar_init(r.acc_full + 8u * i, 1u);
            mbar_init(r.acc_empty + 8u * i, kEpilogueWarps);
        }
        mbar_init(drain_bar, 1u);
        *abort_flag = 0u;
        mbar_init_fence();
    }
    if (warp == kDecWeightWarp && lane == 0u) {
        tma_prefetch_desc(&tmap_w);
    }
    if (warp == kDecInputWarp && lane == 0u) {
        tma_prefetch_desc(&tmap_x);
    }
    if (warp == kDecMmaWarp) {
        tmem_alloc(tmem_slot, S::tmem_columns);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;

    unsigned int m_live = 0u;

    if (warp == kDecWeightWarp) {
        // ---------------------------------------------------------------- raw weight copies
        if (lane == 0u) {
            uint32_t g = 0;
            uint32_t tile = tile_begin;
            uint32_t s = seg_begin;
            for (uint32_t u = u_begin; u < u_end; ++u, ++g) {
                const uint32_t st = g % S::raw_stages;
                const uint32_t ph = (g / S::raw_stages) & 1u;
                if (!mbar_wait(r.raw_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                    break;
                }
                mbar_expect_tx(r.raw_full + 8u * st, kRawStageBytes);
                tma_load_2d(r.raw_base + st * kRawStageBytes, &tmap_w, r.raw_full + 8u * st,
                            (int)(s * kSegWords), (int)(tile * kRows));
                if (++s == segs) {
                    s = 0u;
                    ++tile;
                }
            }
            // Let every copy this thread started land before the block ends.
            uint32_t local_abort = 0;
            const uint32_t first = g > S::raw_stages ? g - S::raw_stages : 0u;
            for (uint32_t i = first; i < g; ++i) {
                mbar_wait(r.raw_full + 8u * (i % S::raw_stages), (i / S::raw_stages) & 1u, &local_abort,
                          nullptr);
            }
        }
    } else if (warp == kDecInputWarp) {
        // ---------------------------------------------------------------- x copies
        const uint32_t total = u_end - u_begin;
        uint32_t next_seg = seg_begin;
        uint32_t issued = 0;
        if (lane == 0u) {
            grid_dependency_wait();
            Q8_STAMP(2u, true)                     // the launches before this one have finished
            for (; issued < total; ++issued) {
                const uint32_t st = issued % S::x_depth;
                const uint32_t ph = (issued / S::x_depth) & 1u;
                if (!mbar_wait(r.x_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                    break;
                }
                mbar_expect_tx(r.x_land + 8u * st, S::x_seg_bytes);
#pragma unroll
                for (uint32_t j = 0; j < kSubs; ++j) {
                    tma_load_2d(r.x_base + st * S::x_seg_bytes + j * S::x_sub_bytes, &tmap_x, r.x_land + 8u * st,
                                (int)(next_seg * kSegK + j * kSubK), 0);
                }
                if (++next_seg == segs) {
                    next_seg = 0u;
                }
            }
        }
        if (lane == 0u) {
            // Let every copy this thread started land before the block ends.
            uint32_t local_abort = 0;
            const uint32_t first = issued > S::x_depth ? issued - S::x_depth : 0u;
            for (uint32_t i = first; i < issued; ++i) {
                mbar_wait(r.x_land + 8u * (i % S::x_depth), (i / S::x_depth) & 1u, &local_abort, nullptr);
            }
        }
    } else if (warp == kDecMmaWarp) {
        // ---------------------------------------------------------------- MMA issue
        // Lane 0 issues the MMAs.
        const uint32_t idesc = umma_idesc(kRows, (uint32_t)NTOK, 0u, 0u);
        uint32_t g = 0;
        uint32_t tc = 0;
        uint32_t s0 = seg_begin;
        bool ok = true;
        for (uint32_t u = u_begin; ok && u < u_end; ++tc) {
            const uint32_t left = u_end - u;
            const uint32_t s1 = (segs - s0) < left ? segs : s0 + left;
            const uint32_t aph = tc & 1u;
            uint32_t chain = 0u;
            uint32_t started = 0u;   // bit c: sum c holds MMAs of this piece already
            for (uint32_t s = s0; ok && s < s1; ++s, ++g) {
                const uint32_t xst = g % S::x_depth;
                const uint32_t xph = (g / S::x_depth) & 1u;
                if (lane == 0u) {
                    // the x segment has landed and, where it was bfloat16, the converters have
                    // turned it into binary16
                    if (!mbar_wait((args.b_bf16 != 0u ? r.x_full : r.x_land) + 8u * xst, xph, abort_flag,
                                   args.status)) {
                        ok = false;
                    }
                    Q8_STAMP(1u, g == 0u)                   // the first x segment is ready
                    if (ok && s == s0 && !mbar_wait(r.acc_empty, aph ^ 1u, abort_flag, args.status)) {
                        ok = false;
                    }
#pragma unroll 1
                    for (uint32_t half = 0; ok && half < 2u; ++half) {
                        const uint32_t hh = 2u * g + half;
                        const uint32_t st = hh % S::a_stages;
                        const uint32_t ph = (hh / S::a_stages) & 1u;
                        if (!mbar_wait(r.a_full + 8u * st, ph, abort_flag, args.status)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t a_tmem = tmem_base + S::a_column0 + st * S::a_stage_columns;
#pragma unroll
                        for (uint32_t jl = 0; jl < 2u; ++jl) {
                            const uint32_t j = 2u * half + jl;
                            const uint64_t b_desc =
                                umma_desc_sw128(r.x_base + xst * S::x_seg_bytes + j * S::x_sub_bytes);
#pragma unroll
                            for (uint32_t kk = 0; kk < kSubK / 16u; ++kk) {
                                // 16 values: 8 columns of A, 32 bytes along the swizzled row of x
                                umma_f16_ts(tmem_base + chain * (uint32_t)NTOK, a_tmem + jl * (kSubK / 2u) + 8u * kk,
                                            b_desc + 2u * kk, idesc, (started >> chain) & 1u);
                                started |= 1u << chain;
                                chain = chain + 1u == S::chains ? 0u : chain + 1u;
                            }
                        }
                        umma_commit(r.a_empty + 8u * st);
                    }
                    if (ok) {
                        umma_commit(r.x_empty + 8u * xst);
                    }
                }
                // lane 0's waits may have run out: every lane leaves together
                ok = __all_sync(0xFFFFFFFFu, ok) != 0;
            }
            if (ok && lane == 0u) {
                umma_commit(r.acc_full);
            }
            u += (s1 - s0);
            s0 = 0u;
        }
        if (!ok && lane == 0u) {
            // Outstanding MMAs must finish before the tensor memory goes back.
            uint32_t local_abort = 0;
            umma_commit(drain_bar);
            mbar_wait(drain_bar, 0u, &local_abort, nullptr);
        }
    } else if (warp >= kDecConvertWarp0) {
        // ---------------------------------------------------------------- dequantise
        const uint32_t cw = warp - kDecConvertWarp0;
        const uint32_t row = cw * 32u + lane;
        // this warp owns TMEM lanes [32 cw, +32): its rows of the tile
        const uint32_t lane_base = tmem_base + ((cw * 32u) << 16) + S::a_column0;
        uint32_t g = 0;
        for (uint32_t u = u_begin; u < u_end; ++u, ++g) {
            if (!convert_unit<NTOK, 0>(r, g, row, lane, lane_base, args.b_bf16 != 0u, abort_flag, args.status)
                || !convert_unit<NTOK, 1>(r, g, row, lane, lane_base, args.b_bf16 != 0u, abort_flag, args.status)) {
                break;
            }
        }
        Q8_STAMP(3u, cw == 0u && lane == 0u)       // conversion of the block's units done
    } else {
        // ---------------------------------------------------------------- read sums, store
        const uint32_t wq = warp;
        const uint32_t lane_row = wq * 32u + lane;
        const uint32_t lane_taddr = tmem_base + ((wq * 32u) << 16);
        grid_dependency_wait();
        m_live = args.m_max;
        if (args.m_dev != nullptr) {
            const unsigned int live = *args.m_dev;
            m_live = live < m_live ? live : m_live;
        }
        if (!split) {
            uint32_t tile = tile_begin;
            uint32_t s0 = seg_begin;
            uint32_t tc = 0;
            for (uint32_t done = u_begin; done < u_end; ++tc) {
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(r.acc_full, tc & 1u, abort_flag, args.status))) {
                    break;
                }
                const uint32_t left = u_end - done;
                const uint32_t s1 = (segs - s0) < left ? segs : s0 + left;
                const bool owner = s0 == 0u;
                const bool whole = owner && s1 == segs;
                TilePlace place;
                place.w_row = place.j0 = tile * kRows;
                place.j_limit = args.n;
                place.i0 = 0u;
                place.i_limit = m_live;
                const uint32_t j = place.j0 + lane_row;
                unsigned int last_cc = blockIdx.x;
                if (owner && !whole) {
                    // The other holders of this tile are the blocks right after this one; they
                    // met it at the start of their ranges and have published their partial sums.
                    last_cc = decode_holder((tile + 1u) * segs - 1u, blocks, units);
                    for (unsigned int base = blockIdx.x + 1u; base <= last_cc; base += 32u) {
                        const unsigned int cc = base + lane;
                        if (cc <= last_cc) {
                            const unsigned int *flag = args.flags + 4u * cc + wq;
                            const long long begin = clock64();
                            while (ld_acquire_gpu(flag) == 0u) {
                                if (clock64() - begin > Q8_WAIT_CYCLES || *abort_flag != 0u) {
                                    atomicOr(args.status, Q8_DEV_FLAG_TIMEOUT);
                                    break;
                                }
                            }
                        }
                    }
                    __syncwarp();
                }
                tc_fence_after_sync();
                float *own_slot = args.partial + (unsigned long long)blockIdx.x * args.tile_floats + lane_row;
                // the other blocks' partial sums, added up in block order; all the loads of one
                // block's partial tile go out together (a trip to L2 each would cost more than
                // the whole store otherwise)
                float others[NTOK];
                if (last_cc != blockIdx.x) {
                    const float *slot = args.partial + (unsigned long long)(blockIdx.x + 1u) * args.tile_floats
                                      + lane_row;
    #pragma unroll
                    for (uint32_t i = 0; i < (uint32_t)NTOK; ++i) {
                        others[i] = __ldcg(slot + (unsigned long long)i * kRows);
                    }
                }
    #pragma unroll 1
                for (unsigned int cc = blockIdx.x + 2u; cc <= last_cc; ++cc) {
                    const float *slot = args.partial + (unsigned long long)cc * args.tile_floats + lane_row;
    #pragma unroll
                    for (uint32_t c0 = 0; c0 < (uint32_t)NTOK; c0 += 16u) {
                        float a[16];
    #pragma unroll
                        for (uint32_t i = 0; i < 16u; ++i) {
                            a[i] = __ldcg(slot + (unsigned long long)(c0 + i) * kRows);
                        }
    #pragma unroll
                        for (uint32_t i = 0; i < 16u; ++i) {
                            others[c0 + i] += a[i];
                        }
                    }
                }
    #pragma unroll
                for (uint32_t c0 = 0; c0 < (uint32_t)NTOK; c0 += 8u) {
                    uint32_t v[8];
                    load_sums<NTOK>(lane_taddr + c0, v);
                    if (!owner) {
    #pragma unroll
                        for (uint32_t i = 0; i < 8u; ++i) {
                            __stcg(own_slot + (unsigned long long)(c0 + i) * kRows, __uint_as_float(v[i]));
                        }
                    } else {
                        if (last_cc != blockIdx.x) {
    #pragma unroll
                            for (uint32_t i = 0; i < 8u; ++i) {
                                v[i] = __float_as_uint(__uint_as_float(v[i]) + others[c0 + i]);
                            }
                        }
                        store_eight<YT>(args, place, lane_row, j, c0, v);
                    }
                }
                // The accumulator buffer is free again.
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0u) {
                    mbar_arrive(r.acc_empty);
                }
                if (!owner) {
                    // Publish this warp's quarter of the partial tile; every lane makes its own
                    // stores visible first.
                    __threadfence();
                    __syncwarp();
                    if (lane == 0u) {
                        st_release_gpu(args.flags + 4u * blockIdx.x + wq, 1u);
                    }
                } else if (!whole) {
                    // Hand the consumed slots back for the next launch that uses this set
                    // (ordered by the end of the kernel).
                    for (unsigned int base = blockIdx.x + 1u; base <= last_cc; base += 32u) {
                        const unsigned int cc = base + lane;
                        if (cc <= last_cc) {
                            *reinterpret_cast<volatile unsigned int *>(args.flags + 4u * cc + wq) = 0u;
                        }
                    }
                }
                done += (s1 - s0);
                s0 = 0u;
                ++tile;
            }
        } else {
            // the block's one piece: wait for its MMAs, the exchange below reads the accumulator
            mbar_wait(r.acc_full, 0u, abort_flag, args.status);
            tc_fence_after_sync();
            Q8_STAMP(5u, wq == 0u && lane == 0u)
        }
    }

    if (!split) {
        tc_fence_before_sync();
        __syncthreads();
        if (warp == kDecMmaWarp) {
            tc_fence_after_sync();
            tmem_dealloc(tmem_base, S::tmem_columns);
        }
        Q8_STAMP(7u, threadIdx.x == 0u)
        return;
    }

    // ------------------------------------------------------------ sum of a cluster's pieces
    // The token columns of the tile are dealt to the blocks of the cluster in runs: block o owns
    // columns [o * share, (o + 1) * share).  Every block writes the columns of its piece into
    // their owners' shared memory (its own into its own), over the x ring, which is idle once
    // every block's MMAs have finished: per sending block and row of w the owner's `share` sums
    // lie next to each other, so a thread sends them 16 bytes at a time (a store into another
    // block's shared memory costs the same for one float as for four).  The owner adds the
    // pieces in block order and stores.
    const uint32_t share = (uint32_t)NTOK / csize;   // 2 to 32: the cluster size is a power of two up to 8
    __syncwarp();
    cluster_arrive_release();
    cluster_wait_acquire();
    Q8_STAMP(4u, threadIdx.x == 0u)
    const uint32_t lane_row = warp * 32u + lane;
    if (warp < kEpilogueWarps) {
        const uint32_t lane_taddr = tmem_base + ((warp * 32u) << 16);
        const uint32_t mine = r.x_base + (crank * kRows + lane_row) * share * 4u;   // in the owner's memory
#pragma unroll 1
        for (uint32_t c0 = 0; c0 < (uint32_t)NTOK; c0 += 8u) {
            uint32_t v[8];
            load_sums<NTOK>(lane_taddr + c0, v);
            if (share >= 4u) {
#pragma unroll
                for (uint32_t h = 0; h < 8u; h += 4u) {
                    const uint32_t col = c0 + h;
                    st_shared_cluster_v4_f32(mapa_shared(mine + (col % share) * 4u, col / share),
                                             __uint_as_float(v[h]), __uint_as_float(v[h + 1u]),
                                             __uint_as_float(v[h + 2u]), __uint_as_float(v[h + 3u]));
                }
            } else {
#pragma unroll
                for (uint32_t h = 0; h < 8u; h += 2u) {
                    const uint32_t col = c0 + h;
                    st_shared_cluster_v2_f32(mapa_shared(mine + (col % share) * 4u, col / share),
                                             __uint_as_float(v[h]), __uint_as_float(v[h + 1u]));
                }
            }
        }
        tc_fence_before_sync();
    }
    __syncwarp();
    cluster_arrive_release();
    cluster_wait_acquire();
    Q8_STAMP(6u, threadIdx.x == 0u)
    if (warp == kDecMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, S::tmem_columns);
    }
    if (warp < kEpilogueWarps) {
        const uint32_t tile = blockIdx.x / csize;
        TilePlace place;
        place.w_row = place.j0 = tile * kRows;
        place.j_limit = args.n;
        place.i0 = 0u;
        place.i_limit = m_live;
        const uint32_t j = place.j0 + lane_row;
        const uint32_t width = share < 4u ? share : 4u;
#pragma unroll 1
        for (uint32_t local = 0; local < share; local += 4u) {
            // up to four of this block's columns at a time: the pieces of every sending block,
            // fetched together, added in block order
            float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (uint32_t src = 0; src < kDecMaxCluster; ++src) {
                if (src < csize) {
                    const uint32_t at = r.x_base + ((src * kRows + lane_row) * share + local) * 4u;
                    float piece[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (share >= 4u) {
                        uint32_t w0, w1, w2, w3;
                        ld_shared_v4(at, w0, w1, w2, w3);
                        piece[0] = __uint_as_float(w0);
                        piece[1] = __uint_as_float(w1);
                        piece[2] = __uint_as_float(w2);
                        piece[3] = __uint_as_float(w3);
                    } else {
                        piece[0] = ld_shared_f32(at);
                        piece[1] = ld_shared_f32(at + 4u);
                    }
#pragma unroll
                    for (uint32_t q = 0; q < 4u; ++q) {
                        sum[q] = src == 0u ? piece[q] : sum[q] + piece[q];
                    }
                }
            }
            uint32_t sums[4];
#pragma unroll
            for (uint32_t q = 0; q < 4u; ++q) {
                sums[q] = __float_as_uint(sum[q]);
            }
            // only this block's columns: a run of two leaves the other two of the four out
            TilePlace run = place;
            const uint32_t first = crank * share + local;
            run.i_limit = place.i_limit < first + width ? place.i_limit : first + width;
            store_four<YT>(args, run, lane_row, j, first, 1u, sums);
        }
    }
    Q8_STAMP(7u, threadIdx.x == 0u)
}

template <int NTOK, typename YT>
static cudaError_t launch_decode_typed(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                                       const UmmaArgs &args, unsigned int grid, unsigned int cluster)
{
    using S = DecodeShape<NTOK>;
    static unsigned long long configured = 0ull;
    cudaError_t err = allow_shared_memory(q8_decode_kernel<NTOK, YT>, S::smem_bytes, &configured, true);
    if (err != cudaSuccess) {
        return err;
    }
    return launch_tile_kernel(q8_decode_kernel<NTOK, YT>, grid, S::smem_bytes, stream, args.overlap != 0u, tw, tx,
                              args, kDecThreads, cluster);
}

template <int NTOK>
static cudaError_t launch_decode_tile(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                                      const UmmaArgs &args, unsigned int grid, unsigned int cluster, int y_dtype)
{
    switch (y_dtype) {
    case 0:
        return launch_decode_typed<NTOK, float>(stream, tw, tx, args, grid, cluster);
    case 1:
        return launch_decode_typed<NTOK, __half>(stream, tw, tx, args, grid, cluster);
    case 2:
        return launch_decode_typed<NTOK, __nv_bfloat16>(stream, tw, tx, args, grid, cluster);
    default:
        return cudaErrorInvalidValue;
    }
}

// How a product of `row_tiles` weight row tiles and `segs` segments per row runs on `sm_count`
// SMs: *cluster = 0 and the number of blocks for the unit schedule, or *cluster = the number of
// blocks that share one tile (1 to 8) and row_tiles * *cluster blocks.
unsigned int decode_grid(unsigned int row_tiles, unsigned int segs, unsigned int sm_count,
                         unsigned int scratch_blocks, unsigned int *cluster)
{
    *cluster = 0u;
#ifndef Q8_HOST_EMULATION
    if (2u * row_tiles <= sm_count) {
        // As many pieces per tile as fill two blocks per SM.  (One block per SM and launch, so
        // that the next product's blocks always find a free place, was measured and is slower:
        // half as many blocks convert.)
        unsigned int pieces = 2u * sm_count / row_tiles;
        unsigned int most = kDecMaxCluster;
#ifdef Q8_TRACE
        if (getenv("Q8_ONE_PER_SM") != nullptr) {
            pieces = sm_count / row_tiles;   // development builds: the other placement, for comparison
        }
#endif
        pieces = pieces > most ? most : pieces;
        pieces = pieces > segs ? segs : pieces;
        // a power of two: clusters of 6 took three times as long to be placed as clusters of 4 or 8
        while ((pieces & (pieces - 1u)) != 0u) {
            pieces &= pieces - 1u;
        }
        *cluster = pieces;
        return row_tiles * pieces;
    }
#endif
    const unsigned long long units = (unsigned long long)row_tiles * segs;
    unsigned int grid = 2u * sm_count < scratch_blocks ? 2u * sm_count : scratch_blocks;
    return units < grid ? (unsigned int)units : grid;
}

cudaError_t launch_decode_kernel(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                                 const UmmaArgs &args, unsigned int grid, unsigned int cluster, unsigned int ntok,
                                 int y_dtype)
{
    switch (ntok) {
    case 16:
        return launch_decode_tile<16>(stream, tw, tx, args, grid, cluster, y_dtype);
    case 32:
        return launch_decode_tile<32>(stream, tw, tx, args, grid, cluster, y_dtype);
    default:
        return cudaErrorInvalidValue;
    }
}

} // namespace q8
