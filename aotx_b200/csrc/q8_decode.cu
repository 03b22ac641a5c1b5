// The decode-regime kernel of the Q8_0 product for batches of up to 32 rows of x (one token
// tile of 16 or 32): y[i][j] = sum_c x[i][c] * half(q[j][c] * d[j][c / 32]), float sums.
//
// HBM-bound: a launch moves n * (k / 32) * 34 bytes of weights once, whatever the batch.  What
// decides the time of the 18 to 125 MB products of a decode step is not the steady stream but
// the ends of a launch, so the kernel is built around three things:
//   * two blocks fit on one SM (352 threads, 88 registers, about 102 KB of shared memory, half
//     of the tensor memory each).  With programmatic dependent launch the blocks of the next
//     product start beside the blocks of this one and stream and dequantise their first weights
//     while this product finishes; only x, the live batch and the stores wait for it;
//   * when the weight tensor has few row tiles (n up to about 9000), a tile is cut along k over
//     a CLUSTER of up to 8 blocks, one piece each, and the pieces are summed through
//     distributed shared memory: every block sends each other block its slice of the token
//     columns, adds what it receives in block order and stores its own columns.  No global
//     scratch, no flags to poll, and every block stores a share of the tile;
//   * larger tensors run as (tile, segment) units dealt evenly over 2 blocks per SM.  A tile cut
//     between blocks belongs to the block that holds its first segment, which is that block's
//     last piece; the other holders publish their partial sums at the start of their ranges, and
//     the owner fetches and adds them while its own last MMAs still run.
//
// Inside a block (11 warps): warp 8 issues bulk tensor copies of raw weight segments
// [128 rows x 272 B] into a two-deep ring; warps 4-7 are converters, thread = row: nine 16-byte
// shared loads per half segment, exact dequantisation in registers, tcgen05.st of 64 packed
// words into the thread's lane of tensor memory; warp 10 issues tcgen05.mma 128 x NTOK x 16 with
// A from tensor memory and B = the x tile in shared memory (128-byte swizzle); warp 9 copies x
// tiles and turns a bfloat16 x tile into binary16 where it lies (one MMA takes both operands
// in one format; exact for magnitudes in [2^-14, 65504], saturating above); warps 0-3 read the
// accumulator and store.  The schedule never depends on the live batch (one token tile), so the
// batch word is read only by the storing warps, after the launches before this one finished.
// Every wait on a barrier or flag is bounded and raises a status bit when it runs out.
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
    static constexpr uint32_t a_column0 = 64;                        // after the two accumulators
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

// The accumulator of one piece into registers: NTOK columns of this thread's lane.
template <int NTOK>
__device__ __forceinline__ void load_accumulator(uint32_t taddr, uint32_t (&v)[NTOK])
{
    if (NTOK == 32) {
        tmem_ld_32x32(taddr, v);
    } else {
        tmem_ld_32x16(taddr, v);
    }
    tmem_ld_wait();
}

template <int NTOK, typename YT>
__global__ void __launch_bounds__(kDecThreads, 2)
q8_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 const UmmaArgs args)
{
    using S = DecodeShape<NTOK>;
    extern __shared__ unsigned char smem_raw_[];
    const uint32_t smem0 = (smem_u32(smem_raw_) + 1023u) & ~1023u;
    const uint32_t x_base = smem0 + S::x_offset;
    const uint32_t raw_base = smem0 + S::raw_offset;
    const uint32_t bar_base = smem0 + S::bar_offset;
    const uint32_t raw_full = bar_base;
    const uint32_t raw_empty = raw_full + 8u * S::raw_stages;
    const uint32_t x_land = raw_empty + 8u * S::raw_stages;  // the copy of an x segment is complete
    const uint32_t x_full = x_land + 8u * S::x_depth;        // ... and it is binary16
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

    // The next kernel on the stream may start its blocks beside this one's.  Work that only
    // reads the weights runs ahead of the kernels before this one; everything that reads x or
    // the live batch, or writes y or the scratch slots, first waits for them to finish.
    grid_launch_dependents();

    const uint32_t segs = args.k / kSegK;
    const uint32_t row_tiles = (args.n + kRows - 1u) / kRows;
    const unsigned long long units = (unsigned long long)row_tiles * segs;
    const bool split = args.split != 0u;
    uint32_t crank = 0u;
    uint32_t csize = 1u;
    unsigned int blocks = gridDim.x;
    unsigned long long u_begin, u_end;
    if (split) {
        // one tile per cluster, one run of its segments per block
        csize = cluster_nctarank();
        crank = cluster_ctarank();
        const unsigned long long tile = blockIdx.x / csize;
        u_begin = tile * segs + (unsigned long long)crank * segs / csize;
        u_end = tile * segs + (unsigned long long)(crank + 1u) * segs / csize;
    } else {
        // No more blocks than units take part, so that every block in the schedule has work.
        blocks = units < gridDim.x ? (unsigned int)units : gridDim.x;
        if (blockIdx.x >= blocks) {
            return;
        }
        unit_range(blockIdx.x, blocks, units, &u_begin, &u_end);
    }

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < S::raw_stages; ++i) {
            mbar_init(raw_full + 8u * i, 1u);
            mbar_init(raw_empty + 8u * i, kDecConvertWarps);
        }
        for (uint32_t i = 0; i < S::x_depth; ++i) {
            mbar_init(x_land + 8u * i, 1u);
            mbar_init(x_full + 8u * i, 1u);
            mbar_init(x_empty + 8u * i, 1u);
        }
        for (uint32_t i = 0; i < S::a_stages; ++i) {
            mbar_init(a_full + 8u * i, kDecConvertWarps);
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
    // an x segment is ready for the MMA when its copy landed (binary16) or was turned (bfloat16)
    const uint32_t x_ready = args.b_bf16 != 0u ? x_full : x_land;

    // In a cluster launch the block's single piece stays in these registers of the storing warps
    // until the exchange at the end of the kernel.
    uint32_t vals[NTOK];
    unsigned int m_live = 0u;

    if (warp == kDecWeightWarp) {
        // ---------------------------------------------------------------- raw weight copies
        if (lane == 0u) {
            uint32_t g = 0;
            bool ok = true;
            for (unsigned long long u = u_begin; ok && u < u_end;) {
                const uint32_t tile = (uint32_t)(u / segs);
                const uint32_t s0 = (uint32_t)(u % segs);
                const unsigned long long left = u_end - u;
                const uint32_t s1 = (segs - s0) < left ? segs : (uint32_t)(s0 + left);
                const uint32_t w_row = tile * kRows;
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
    } else if (warp == kDecInputWarp) {
        // ---------------------------------------------------------------- x copies
        // Lane 0 keeps the copies of two segments in flight; for bfloat16 activations the whole
        // warp then turns each landed segment into binary16 where it lies (the swizzle moves
        // whole 16-byte chunks, so the conversion is chunk by chunk whatever the layout).
        const uint32_t total = (uint32_t)(u_end - u_begin);
        const uint32_t first_seg = (uint32_t)(u_begin % segs);
        uint32_t issued = 0;
        bool ok = true;
        grid_dependency_wait();
        for (uint32_t g = 0; ok && g < total; ++g) {
            if (lane == 0u) {
                while (ok && issued < total && issued < g + S::x_depth) {
                    const uint32_t st = issued % S::x_depth;
                    const uint32_t ph = (issued / S::x_depth) & 1u;
                    if (!mbar_wait(x_empty + 8u * st, ph ^ 1u, abort_flag, args.status)) {
                        ok = false;
                        break;
                    }
                    const uint32_t s = (first_seg + issued) % segs;
                    mbar_expect_tx(x_land + 8u * st, S::x_seg_bytes);
#pragma unroll
                    for (uint32_t j = 0; j < kSubs; ++j) {
                        tma_load_2d(x_base + st * S::x_seg_bytes + j * S::x_sub_bytes, &tmap_x, x_land + 8u * st,
                                    (int)(s * kSegK + j * kSubK), 0);
                    }
                    ++issued;
                }
            }
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            if (!ok) {
                break;
            }
            if (args.b_bf16 != 0u) {
                const uint32_t st = g % S::x_depth;
                const uint32_t ph = (g / S::x_depth) & 1u;
                if (!mbar_wait(x_land + 8u * st, ph, abort_flag, args.status)) {
                    ok = false;
                    break;
                }
                const uint32_t x_seg = x_base + st * S::x_seg_bytes;
#pragma unroll 4
                for (uint32_t c = lane; c < S::x_seg_bytes / 16u; c += 32u) {
                    bf16_chunk_to_f16_inplace(x_seg + 16u * c);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0u) {
                    mbar_arrive(x_full + 8u * st);
                }
            }
        }
        if (lane == 0u) {
            // Let every copy this thread started land before the block ends.
            uint32_t local_abort = 0;
            const uint32_t first = issued > S::x_depth ? issued - S::x_depth : 0u;
            for (uint32_t i = first; i < issued; ++i) {
                mbar_wait(x_land + 8u * (i % S::x_depth), (i / S::x_depth) & 1u, &local_abort, nullptr);
            }
        }
    } else if (warp == kDecMmaWarp) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0u) {
            const uint32_t idesc = umma_idesc(kRows, (uint32_t)NTOK, 0u, 0u);
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
                    if (!mbar_wait(x_ready + 8u * xst, xph, abort_flag, args.status)) {
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
    } else if (warp >= kDecConvertWarp0) {
        // ---------------------------------------------------------------- dequantise
        const uint32_t cw = warp - kDecConvertWarp0;
        const uint32_t row = cw * 32u + lane;
        // this warp owns TMEM lanes [32 cw, +32): its rows of the tile
        const uint32_t lane_base = tmem_base + ((cw * 32u) << 16) + S::a_column0;
        uint32_t g = 0;
        bool ok = true;
        for (unsigned long long u = u_begin; ok && u < u_end; ++u, ++g) {
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
                if (half == 0u) {
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
        if (split) {
            if (mbar_wait(acc_full, 0u, abort_flag, args.status)) {
                tc_fence_after_sync();
                load_accumulator<NTOK>(lane_taddr, vals);
            } else {
#pragma unroll
                for (uint32_t i = 0; i < (uint32_t)NTOK; ++i) {
                    vals[i] = 0u;
                }
            }
            tc_fence_before_sync();
        } else {
            uint32_t tc = 0;
            bool ok = true;
            for (unsigned long long u = u_begin; ok && u < u_end; ++tc) {
                const uint32_t tile = (uint32_t)(u / segs);
                const uint32_t s0 = (uint32_t)(u % segs);
                const unsigned long long left = u_end - u;
                const uint32_t s1 = (segs - s0) < left ? segs : (uint32_t)(s0 + left);
                const uint32_t buf = tc & 1u;
                const uint32_t aph = (tc >> 1) & 1u;
                const bool owner = s0 == 0u;
                const bool whole = owner && s1 == segs;
                TilePlace place;
                place.w_row = place.j0 = tile * kRows;
                place.j_limit = args.n;
                place.i0 = 0u;
                place.i_limit = m_live;
                const uint32_t j = place.j0 + lane_row;
                unsigned int last_cc = blockIdx.x;
                float others[NTOK];
                if (owner && !whole) {
                    // The other holders of this tile are the blocks right after this one; they
                    // met it at the start of their ranges.  Fetch and add their partial sums, in
                    // block order, while this block's own MMAs of the tile still run.
                    last_cc = last_holder(blockIdx.x, blocks, units, ((unsigned long long)tile + 1ull) * segs);
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
                    for (unsigned int cc = blockIdx.x + 1u; cc <= last_cc; ++cc) {
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
                                others[c0 + i] = cc == blockIdx.x + 1u ? a[i] : others[c0 + i] + a[i];
                            }
                        }
                    }
                }
                if (!mbar_wait(acc_full + 8u * buf, aph, abort_flag, args.status)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                float *own_slot = args.partial + (unsigned long long)blockIdx.x * args.tile_floats + lane_row;
#pragma unroll
                for (uint32_t c0 = 0; c0 < (uint32_t)NTOK; c0 += 16u) {
                    uint32_t v[16];
                    tmem_ld_32x16(lane_taddr + buf * (uint32_t)NTOK + c0, v);
                    tmem_ld_wait();
                    if (!owner) {
#pragma unroll
                        for (uint32_t i = 0; i < 16u; ++i) {
                            __stcg(own_slot + (unsigned long long)(c0 + i) * kRows, __uint_as_float(v[i]));
                        }
                    } else {
                        if (!whole) {
#pragma unroll
                            for (uint32_t i = 0; i < 16u; ++i) {
                                v[i] = __float_as_uint(__uint_as_float(v[i]) + others[c0 + i]);
                            }
                        }
                        store_chunk<16u, YT>(args, place, lane_row, j, c0, v);
                    }
                }
                // The accumulator buffer is free again.
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0u) {
                    mbar_arrive(acc_empty + 8u * buf);
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
                    // Hand the consumed slots back for the next launch that uses this set (ordered
                    // by the end of the kernel).
                    for (unsigned int base = blockIdx.x + 1u; base <= last_cc; base += 32u) {
                        const unsigned int cc = base + lane;
                        if (cc <= last_cc) {
                            *reinterpret_cast<volatile unsigned int *>(args.flags + 4u * cc + wq) = 0u;
                        }
                    }
                }
                u += (s1 - s0);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == kDecMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, S::tmem_columns);
    }
    if (!split) {
        return;
    }

    // ------------------------------------------------------------ sum of a cluster's pieces
    // Token column i of the tile belongs to block (i mod cluster size) of the cluster.  A block
    // sends every other block that block's columns of its piece, receives its own columns of
    // theirs, adds them in block order and stores.
    const uint32_t tile = blockIdx.x / csize;
    TilePlace place;
    place.w_row = place.j0 = tile * kRows;
    place.j_limit = args.n;
    place.i0 = 0u;
    place.i_limit = m_live;
    const uint32_t lane_row = warp * 32u + lane;
    const uint32_t j = place.j0 + lane_row;
    if (csize == 1u) {
        if (warp < kEpilogueWarps) {
            store_chunk<(uint32_t)NTOK, YT>(args, place, lane_row, j, 0u, vals);
        }
        return;
    }
    const uint32_t share = ((uint32_t)NTOK + csize - 1u) / csize; // columns per block, at most
    // every block of the cluster has finished its MMAs: the x rings are free
    __syncwarp();
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp < kEpilogueWarps) {
        uint32_t owner = 0u;
        uint32_t local = 0u;
#pragma unroll
        for (uint32_t i = 0; i < (uint32_t)NTOK; ++i) {
            if (owner != crank) {
                const uint32_t at = x_base + ((crank * share + local) * kRows + lane_row) * 4u;
                st_shared_cluster_f32(mapa_shared(at, owner), __uint_as_float(vals[i]));
            }
            if (++owner == csize) {
                owner = 0u;
                ++local;
            }
        }
    }
    __syncwarp();
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp < kEpilogueWarps) {
        uint32_t owner = 0u;
        uint32_t local = 0u;
#pragma unroll
        for (uint32_t i = 0; i < (uint32_t)NTOK; ++i) {
            if (owner == crank) {
                float sum = 0.0f;
                for (uint32_t src = 0; src < csize; ++src) {
                    const float piece = src == crank
                        ? __uint_as_float(vals[i])
                        : ld_shared_f32(x_base + ((src * share + local) * kRows + lane_row) * 4u);
                    sum = src == 0u ? piece : sum + piece;
                }
                uint32_t one[1] = {__float_as_uint(sum)};
                store_chunk<1u, YT>(args, place, lane_row, j, i, one);
            }
            if (++owner == csize) {
                owner = 0u;
                ++local;
            }
        }
    }
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
        unsigned int pieces = sm_count / row_tiles;
        pieces = pieces > kDecMaxCluster ? kDecMaxCluster : pieces;
        pieces = pieces > segs ? segs : pieces;
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
