// Pieces shared by the two tensor-core kernels of the Q8_0 product: tile constants, the
// kernel arguments, the unit schedule, the raw-row loader, the exact converters (to shared
// memory in the swizzled operand layout, or to tensor memory) and the epilogue that stores a
// finished tile or hands a partial one to the tile's owner.
#pragma once

#include <cuda.h>

#include "q8_common.cuh"
#include "q8_launch.h"

namespace q8 {

constexpr uint32_t kRows = 128;                          // rows of w per tile (MMA M)
constexpr uint32_t kSegK = 256;                          // weights per row per segment
constexpr uint32_t kSegBytes = 272;                      // bytes per row per segment
constexpr uint32_t kSegWords = kSegBytes / 4;            // 68
constexpr uint32_t kRawStageBytes = kRows * kSegBytes;   // 34816
constexpr uint32_t kSubK = 64;                           // weights per row per MMA stage
constexpr uint32_t kSubs = kSegK / kSubK;                // 4 MMA stages per segment
constexpr uint32_t kAStageBytes = kRows * kSubK * 2;     // 16384
constexpr uint32_t kThreads = 15 * 32;
constexpr uint32_t kEpilogueWarps = 4;
constexpr uint32_t kConvertWarp0 = 4;
constexpr uint32_t kConvertThreads = 8 * 32;                // warps 4..11
constexpr uint32_t kWeightWarp = 12;
constexpr uint32_t kInputWarp = 13;
constexpr uint32_t kMmaWarp = 14;

struct GroupTile {
    unsigned int w_row;     // first row of the tile in the stacked weight tensor
    unsigned int j0;        // first column of y the tile produces
    unsigned int j_limit;   // columns of y of this expert's tensor (store j < j_limit)
    unsigned int tok0;      // first row of the sorted activations
    unsigned int tok_limit; // one past the last row that belongs to the tile
};

// Where a tile reads and writes.
struct TilePlace {
    unsigned int w_row;
    unsigned int j0;
    unsigned int j_limit;
    unsigned int i0;
    unsigned int i_limit;
};

struct UmmaArgs {
    unsigned int n;
    unsigned int k;
    unsigned int m_max;
    const unsigned int *m_dev;
    void *y;
    float *partial;
    unsigned int *flags;
    unsigned int *status;
    unsigned long long tile_floats;
    unsigned int b_bf16;
    unsigned int overlap; // launched with the programmatic-dependent-launch attribute
    // Grouped mode (routed experts): the tiles come from a table built on the device, one
    // entry per (expert, token tile, row tile); w is then all experts' rows stacked, x the
    // activation rows sorted by expert, and a result row i goes to y row row_map[i].
    const GroupTile *group_tiles;      // null outside grouped mode
    const unsigned int *group_count;   // device word: number of table entries
    const unsigned int *row_map;       // may be null
    unsigned int ldy;                  // row stride of y in elements
    // Column-split mode: this launch computes columns [col0, col0 + n) of a wider y and stores
    // its tiles into `peers` copies of it (this GPU's own and the peers' buffers, reached by
    // ordinary stores through peer-mapped addresses).  peers == 0: store into `y` only.
    void *y_peer[8];
    unsigned int peers;
    unsigned int col0;
    // What the store does with a finished sum (kEpilogue*): write it; add it to the float that
    // y holds (residual stream); or, with rows 2p and 2p+1 of w being the gate and up rows of
    // output column p, write silu(gate) * up to column p of a y that is n / 2 wide.
    unsigned int epilogue;
    // Decode kernel (q8_decode.cu): nonzero when the launch is one cluster of blocks per weight
    // row tile, each block taking one run of the tile's segments; zero for the unit schedule.
    unsigned int split;
#ifdef Q8_TRACE
    // development builds (-DQ8_TRACE): time stamps of the decode kernel, 8 words per block, or null
    unsigned long long *trace;
#endif
};

// The units [begin, end) of block `b` out of `blocks`, of `units` in all.
__host__ __device__ __forceinline__ void unit_range(unsigned int b, unsigned int blocks,
                                                    unsigned long long units, unsigned long long *begin,
                                                    unsigned long long *end)
{
    *begin = (unsigned long long)b * units / blocks;
    *end = (unsigned long long)(b + 1u) * units / blocks;
}

// The decode kernel's form of the same (q8_decode.cu): the units of block b of `blocks`, `units` in all (32-bit arithmetic: the first `units mod
// blocks` blocks take one unit more), and the block that holds unit `u`.
__host__ __device__ __forceinline__ void decode_range(uint32_t b, uint32_t blocks, uint32_t units,
                                                      uint32_t *begin, uint32_t *end)
{
    const uint32_t q = units / blocks;
    const uint32_t rem = units - q * blocks;
    *begin = b * q + (b < rem ? b : rem);
    *end = *begin + q + (b < rem ? 1u : 0u);
}

__host__ __device__ __forceinline__ uint32_t decode_holder(uint32_t u, uint32_t blocks, uint32_t units)
{
    const uint32_t q = units / blocks;
    const uint32_t rem = units - q * blocks;
    const uint32_t cut = rem * (q + 1u);
    return u < cut ? u / (q + 1u) : rem + (u - cut) / q;
}

// A tile that is cut between blocks is finished by block `b`, which holds its first segment.
// Returns the last of the blocks after `b` that hold later segments of the tile, whose units
// end at `tile_end` (b itself if there is none).
__host__ __device__ __forceinline__ unsigned int last_holder(unsigned int b, unsigned int blocks,
                                                             unsigned long long units,
                                                             unsigned long long tile_end)
{
    unsigned int last_cc = b;
    for (unsigned int cc = b + 1u; cc < blocks; ++cc) {
        unsigned long long ob, oe;
        unit_range(cc, blocks, units, &ob, &oe);
        if (ob >= tile_end) {
            break;
        }
        last_cc = cc;
        if (oe >= tile_end) {
            break;
        }
    }
    return last_cc;
}

// The two blocks of one MMA stage that this thread owns: `raw` holds 36 words, bytes
// [H * 128, H * 128 + 144) of the thread's 272-byte row segment; the thread's four blocks start
// at byte 34 * (4H + lb), lb = 0..3, that is at local byte (H ? 8 : 0) + 34 * lb.
// They become 32 packed words (64 16-bit values in order of k: binary16, or
// bfloat16 with BF), written to this thread's lane of tensor memory: column c of the stage holds
// weights 2c and 2c+1 of the stage.
template <int H, int JJ, bool BF = false>
__device__ __forceinline__ void convert_stage_tmem(const uint32_t (&raw)[36], uint32_t taddr)
{
    uint32_t out[32];
#pragma unroll
    for (int jb = 0; jb < 2; ++jb) {
        const int lb = 2 * JJ + jb;
        const int byte_off = (H ? 8 : 0) + 34 * lb;
        const int wi = byte_off / 4;
        const bool odd = (byte_off % 4) == 2;
        uint32_t d_bits = prmt(raw[wi], raw[wi], odd ? 0x3232u : 0x1010u);
        __half2 d2 = *reinterpret_cast<__half2 *>(&d_bits);
#pragma unroll
        for (int p = 0; p < 16; ++p) {
            // odd: the payload starts at the next word boundary; else in the high half of the
            // scale's word
            const int word = odd ? wi + 1 + p / 2 : wi + (p + 1) / 2;
            const bool high = odd ? (p % 2) != 0 : ((p + 1) % 2) != 0;
            const uint32_t flipped = raw[word] ^ 0x80808080u;
            if constexpr (BF) {
                const float d = __low2float(d2);
                out[16 * jb + p] = high ? dequant_pair_bf16<1>(flipped, d) : dequant_pair_bf16<0>(flipped, d);
            } else {
                out[16 * jb + p] = high ? dequant_pair<1>(flipped, d2) : dequant_pair<0>(flipped, d2);
            }
        }
    }
    tmem_st_32x32(taddr, out);
}

template <int H>
__device__ __forceinline__ void load_raw(uint32_t raw_row, uint32_t (&raw)[36])
{
#pragma unroll
    for (int i = 0; i < 9; ++i) {
        ld_shared_v4(raw_row + (uint32_t)(H * 128 + 16 * i), raw[4 * i], raw[4 * i + 1], raw[4 * i + 2],
                     raw[4 * i + 3]);
    }
}

// Before a warp hands a raw stage back to the copying thread, every lane must HAVE the words of
// its row, not merely have asked for them: the hand-over lets the next bulk copy overwrite the
// stage from its first rows on, and a load still on its way then reads the next segment's bytes
// (seen on the GPU as one weight row of a tile wrong in one launch in forty, lanes 0 to 3 only,
// and only in the one kernel variant whose instruction order left the loads unconsumed).  The
// vote needs a value computed from all 36 words of every lane, so it cannot issue before the
// loads have returned; it is true about once in 2^64 loads, and then does nothing.
__device__ __forceinline__ void raw_words_present(const uint32_t (&raw)[36], unsigned int *status)
{
    uint32_t all = raw[0];
    uint32_t odd = raw[1];
#pragma unroll
    for (int i = 2; i < 36; i += 2) {
        all ^= raw[i];
        odd += raw[i + 1];
    }
    if (__any_sync(0xFFFFFFFFu, all == 0x5F3759DFu && odd == 0x9E3779B9u)) {
        atomicOr(status, 0u);
    }
}

// The order of work of one block: first its share [u, u_end) of the units of the tiles that
// are cut between blocks (tile ids from sk_tile0), then whole tiles dp_first + i * dp_stride.
struct WorkIter {
    unsigned long long u;
    unsigned long long u_end;
    uint32_t segs;
    uint32_t sk_tile0;
    uint32_t dp_next;
    uint32_t dp_count;
    uint32_t dp_first;
    uint32_t dp_stride;

    __host__ __device__ __forceinline__ bool next(uint32_t &tile, uint32_t &s0, uint32_t &s1)
    {
        if (u < u_end) {
            tile = sk_tile0 + (uint32_t)(u / segs);
            s0 = (uint32_t)(u % segs);
            const unsigned long long left = u_end - u;
            s1 = (segs - s0) < left ? segs : (uint32_t)(s0 + left);
            u += (s1 - s0);
            return true;
        }
        if (dp_next < dp_count) {
            tile = dp_first + dp_next * dp_stride;
            s0 = 0;
            s1 = segs;
            dp_next += 1;
            return true;
        }
        return false;
    }
};

// One piece of a tile is in the accumulator at `taddr_acc` (column base of the buffer).  The
// warp `wq` of the four epilogue warps owns TMEM lanes [32 wq, 32 wq + 32).  `chunk` columns are
// read per TMEM load.
template <int NTOK>
__device__ __forceinline__ TilePlace tile_place(const UmmaArgs &args, uint32_t tile, uint32_t tok_tiles,
                                                unsigned int m)
{
    TilePlace place;
    if (args.group_tiles != nullptr) {
        const GroupTile entry = args.group_tiles[tile];
        place.w_row = entry.w_row;
        place.j0 = entry.j0;
        place.j_limit = entry.j_limit;
        place.i0 = entry.tok0;
        place.i_limit = entry.tok_limit;
    } else {
        const uint32_t row_tile = tile / tok_tiles;
        const uint32_t tok_tile = tile % tok_tiles;
        place.w_row = row_tile * kRows;
        place.j0 = row_tile * kRows;
        place.j_limit = args.n;
        place.i0 = tok_tile * (uint32_t)NTOK;
        place.i_limit = m;
    }
    return place;
}

// What the owner of a tile does with `COUNT` finished sums of one row of w (one column j of y),
// for the rows first_row .. first_row + COUNT - 1 of x: store them, add them to the float y
// holds, or - with rows 2p and 2p+1 of w the gate and up rows of output column p - store
// silu(gate) * up in column p.  Every lane of the warp calls this together (the gated unit
// exchanges values between neighbouring lanes).  `lane_row` is the row within the tile.
// `row_step`: the sums belong to rows first_row, first_row + row_step, ... of x.
template <uint32_t COUNT, typename YT>
__device__ __forceinline__ void store_chunk(const UmmaArgs &args, const TilePlace &place, uint32_t lane_row,
                                            uint32_t j, uint32_t first_row, uint32_t (&v)[COUNT],
                                            uint32_t row_step = 1u)
{
    // Everything the stores need is read before the first of them: where this runs behind a
    // call, the compiler must assume that a store may have changed the argument block and
    // would fetch a field again after every store (measured: 7 us per copy of y and launch).
    const uint32_t epilogue = args.epilogue;
    const uint32_t peers = args.peers;
    const size_t ldy = args.ldy;
    const uint32_t col0 = args.col0;
    const unsigned int *row_map = args.row_map;
    const uint32_t i_limit = place.i_limit;
    const uint32_t j_limit = place.j_limit;
    const bool swiglu = epilogue == kEpilogueSwiglu;
    float value[COUNT];
#pragma unroll
    for (uint32_t i = 0; i < COUNT; ++i) {
        value[i] = __uint_as_float(v[i]);
    }
    if (swiglu) {
        // Gate and up sums of one output column sit in neighbouring lanes.  The arithmetic is
        // that of the separate kernel (cuda/model/norm.cu:92-105).
#pragma unroll
        for (uint32_t i = 0; i < COUNT; ++i) {
            const float mine = value[i];
            const float other = __shfl_xor_sync(0xFFFFFFFFu, mine, 1u);
            const float unit = mine / (1.0f + expf(-mine));
            value[i] = unit * other;
        }
    }
    const bool writes = j < j_limit && (!swiglu || (lane_row & 1u) == 0u);
    if (!writes) {
        return;
    }
    const size_t col = swiglu ? ((col0 + j) >> 1) : (col0 + j);
    // the rows of y, all loads of the map together
    uint32_t row_of[COUNT];
#pragma unroll
    for (uint32_t i = 0; i < COUNT; ++i) {
        const uint32_t row_x = first_row + i * row_step;
        row_of[i] = (row_map != nullptr && row_x < i_limit) ? __ldg(row_map + row_x) : row_x;
    }
    const uint32_t copies = peers == 0u ? 1u : peers;
    for (uint32_t peer = 0; peer < copies; ++peer) {
        YT *out = static_cast<YT *>(peers == 0u ? args.y : args.y_peer[peer]);
        if (epilogue == kEpilogueAdd) {
            // y is the float residual stream: one rounded add, as the separate kernel does it
            // (cuda/model/norm.cu:78-89).  The old values are fetched together, then added and
            // stored: one at a time each fetch would wait behind the store before it.
            float *sums = reinterpret_cast<float *>(out);
            float before[COUNT];
#pragma unroll
            for (uint32_t i = 0; i < COUNT; ++i) {
                before[i] = first_row + i * row_step < i_limit ? sums[(size_t)row_of[i] * ldy + col] : 0.0f;
            }
#pragma unroll
            for (uint32_t i = 0; i < COUNT; ++i) {
                if (first_row + i * row_step < i_limit) {
                    sums[(size_t)row_of[i] * ldy + col] = before[i] + value[i];
                }
            }
        } else {
#pragma unroll
            for (uint32_t i = 0; i < COUNT; ++i) {
                if (first_row + i * row_step < i_limit) {
                    store_out<YT>(out, (size_t)row_of[i] * ldy + col, value[i]);
                }
            }
        }
    }
}

// The bits of one result in the output type (the low 16 bits for the 16-bit types).
template <typename YT>
__device__ __forceinline__ uint32_t out_bits(float v);
template <>
__device__ __forceinline__ uint32_t out_bits<float>(float v)
{
    return __float_as_uint(v);
}
template <>
__device__ __forceinline__ uint32_t out_bits<__half>(float v)
{
    return (uint32_t)__half_as_ushort(__float2half_rn(v));
}
template <>
__device__ __forceinline__ uint32_t out_bits<__nv_bfloat16>(float v)
{
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
}

constexpr uint32_t kStoreStageBytes = 4096;   // per storing warp: 32 rows of x by 32 columns of y, floats

// Whether a tile's plain store can go through the staging buffer: whole 16-byte pieces of rows
// of y, all of the tile's 128 columns inside the tensor.
template <typename YT>
__device__ __forceinline__ bool staged_store_fits(const UmmaArgs &args, const TilePlace &place, uint32_t stage)
{
    return stage != 0u
        && (args.epilogue == kEpilogueStore || args.epilogue == kEpilogueSwiglu
            || (args.epilogue == kEpilogueAdd && sizeof(YT) == 4))
        && args.peers == 0u && args.col0 == 0u
        && place.j0 + kRows <= place.j_limit && (place.j0 % 16u) == 0u
        && (((size_t)args.ldy * sizeof(YT)) % 16u) == 0u && (reinterpret_cast<uintptr_t>(args.y) % 16u) == 0u;
}

// 32 rows of x by this warp's 32 columns of y: every lane holds one column.  A store of a
// column is 32 instructions that each write one 2- or 4-byte value per lane into a different
// row of y, and the one-block-per-SM kernels spent a quarter to two fifths of their time in
// them (prefill gate+up 839 us with the stores, 498 us without).  Here the warp turns its
// 32 x 32 piece round in shared memory (its own 4 KB, no other warp involved) and writes rows:
// 16 bytes per lane, 4 (16-bit) or 8 (float) instructions instead of 32.
// GATED: the warp's 32 sums of a row are 16 gate / up pairs in neighbouring lanes and become 16
// values silu(gate) * up (the arithmetic of cuda/model/norm.cu:92-105), held by the even lanes;
// first_col then counts columns of the narrower y.
template <typename YT, bool GATED>
__device__ __forceinline__ void store_chunk_staged(const UmmaArgs &args, const TilePlace &place, uint32_t stage_warp,
                                                   uint32_t lane, uint32_t first_col, uint32_t first_row,
                                                   const uint32_t (&v)[32])
{
    constexpr uint32_t kColumns = GATED ? 16u : 32u;
    constexpr uint32_t kRowBytes = kColumns * sizeof(YT);      // this warp's part of a row of y
    constexpr uint32_t kLanesPerRow = kRowBytes / 16u;         // 2, 4 or 8
    constexpr uint32_t kRowsPerStep = 32u / kLanesPerRow;      // 16, 8 or 4
    const unsigned int *row_map = args.row_map;
    const size_t ldy = args.ldy;
    const uint32_t i_limit = place.i_limit;
    unsigned char *y = static_cast<unsigned char *>(args.y);
    const uint32_t column = GATED ? lane / 2u : lane;
#pragma unroll
    for (uint32_t i = 0; i < 32u; ++i) {
        float value = __uint_as_float(v[i]);
        if (GATED) {
            const float other = __shfl_xor_sync(0xFFFFFFFFu, value, 1u);
            value = value / (1.0f + expf(-value)) * other;
        }
        const uint32_t bits = out_bits<YT>(value);
        if (!GATED || (lane & 1u) == 0u) {
            if (sizeof(YT) == 4) {
                st_shared_b32(stage_warp + i * kRowBytes + column * 4u, bits);
            } else {
                st_shared_b16(stage_warp + i * kRowBytes + column * 2u, bits);
            }
        }
    }
    __syncwarp();
    const uint32_t part = lane % kLanesPerRow;
    constexpr uint32_t kSteps = 32u / kRowsPerStep;
    const bool adds = !GATED && sizeof(YT) == 4 && args.epilogue == kEpilogueAdd;
    uint4 *at[kSteps];
#pragma unroll
    for (uint32_t step = 0; step < kSteps; ++step) {
        const uint32_t row_x = first_row + step * kRowsPerStep + lane / kLanesPerRow;
        at[step] = nullptr;
        if (row_x < i_limit) {
            const uint32_t row_y = row_map != nullptr ? __ldg(row_map + row_x) : row_x;
            at[step] = reinterpret_cast<uint4 *>(y + ((size_t)row_y * ldy + first_col) * sizeof(YT) + part * 16u);
        }
    }
    // y as the float residual stream: one rounded add per value, as the separate kernel does it
    // (cuda/model/norm.cu:78-89); the old values are fetched together, before the first store
    uint4 before[kSteps];
    if (adds) {
#pragma unroll
        for (uint32_t step = 0; step < kSteps; ++step) {
            before[step] = at[step] != nullptr ? *at[step] : make_uint4(0u, 0u, 0u, 0u);
        }
    }
#pragma unroll
    for (uint32_t step = 0; step < kSteps; ++step) {
        const uint32_t r = step * kRowsPerStep + lane / kLanesPerRow;
        uint4 piece;
        ld_shared_v4(stage_warp + r * kRowBytes + part * 16u, piece.x, piece.y, piece.z, piece.w);
        if (adds) {
            piece.x = __float_as_uint(__uint_as_float(before[step].x) + __uint_as_float(piece.x));
            piece.y = __float_as_uint(__uint_as_float(before[step].y) + __uint_as_float(piece.y));
            piece.z = __float_as_uint(__uint_as_float(before[step].z) + __uint_as_float(piece.z));
            piece.w = __float_as_uint(__uint_as_float(before[step].w) + __uint_as_float(piece.w));
        }
        if (at[step] != nullptr) {
            *at[step] = piece;
        }
    }
    __syncwarp();
}

// PAIRS: the owner of a cut tile keeps the partial sums of two blocks in flight at a time (the
// kernels with 128 registers a thread); without it one block's at a time, the same additions
// in the same order.
template <int NTOK, typename YT, bool PAIRS = true>
__device__ __forceinline__ void epilogue_piece(const UmmaArgs &args, uint32_t taddr_acc, uint32_t wq,
                                               uint32_t lane, const TilePlace &place, uint32_t cut_tile, uint32_t s0,
                                               uint32_t s1,
                                               uint32_t segs, uint32_t tok_tiles,
                                               unsigned long long units, unsigned int blocks,
                                               unsigned int m, volatile uint32_t *abort_flag,
                                               uint32_t acc_empty_bar, uint32_t stage = 0u)
{
    constexpr uint32_t kChunk = NTOK < 32 ? 16 : 32;
    // `stage`: 4 x kStoreStageBytes of shared memory for the storing warps (0: none)
    const bool staged = kChunk == 32u && staged_store_fits<YT>(args, place, stage);
    const uint32_t lane_row = wq * 32u + lane;
    const uint32_t j = place.j0 + lane_row;              // row of w = column of y
    const uint32_t i0 = place.i0;                        // first row of x of the tile
    const uint32_t taddr = taddr_acc + ((wq * 32u) << 16);
    // A tile that is cut between blocks belongs to the block that holds its first
    // segment.  That is the owner's last piece of work, while the other holders meet
    // the tile at the very start of their ranges, so their partial sums are published
    // long before the owner asks for them.
    const bool whole = (s0 == 0u && s1 == segs);
    const bool owner = (s0 == 0u);
    // `cut_tile` counts the tile among those that are cut into units (`units` of them in all)
    const unsigned long long tile_end = ((unsigned long long)cut_tile + 1ull) * segs;
    float *own_slot = args.partial + (unsigned long long)blockIdx.x * args.tile_floats;

    // The other holders of this tile are the blocks right after this one, up to `last_cc`.
    unsigned int last_cc = blockIdx.x;
    if (owner && !whole) {
        last_cc = last_holder(blockIdx.x, blocks, units, tile_end);
        // Wait for their partial sums; each lane watches one of them.
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

    // columns at and beyond the tile's live rows hold nothing that is ever stored
    const uint32_t live_cols = place.i_limit > place.i0 ? place.i_limit - place.i0 : 0u;
#pragma unroll 1
    for (uint32_t c0 = 0; c0 < (uint32_t)NTOK && c0 < live_cols; c0 += kChunk) {
        uint32_t v[kChunk];
        if (kChunk == 32u) {
            tmem_ld_32x32(taddr + c0, v);
        } else {
            tmem_ld_32x16(taddr + c0, v);
        }
        tmem_ld_wait();
        if (!owner) {
#pragma unroll
            for (uint32_t i = 0; i < kChunk; ++i) {
                __stcg(own_slot + (unsigned long long)(c0 + i) * kRows + lane_row, __uint_as_float(v[i]));
            }
        } else {
            // Add the partial sums in block order, two blocks' loads in flight at a time.
            for (unsigned int cc = blockIdx.x + 1u; cc <= last_cc; cc += PAIRS ? 2u : 1u) {
                const float *slot0 = args.partial + (unsigned long long)cc * args.tile_floats
                                   + (unsigned long long)c0 * kRows + lane_row;
                const bool two = PAIRS && cc + 1u <= last_cc;
                const float *slot1 = two ? slot0 + args.tile_floats : slot0;
                float a0[kChunk];
                float a1[kChunk];
#pragma unroll
                for (uint32_t i = 0; i < kChunk; ++i) {
                    a0[i] = __ldcg(slot0 + (unsigned long long)i * kRows);
                }
#pragma unroll
                for (uint32_t i = 0; i < kChunk; ++i) {
                    a1[i] = two ? __ldcg(slot1 + (unsigned long long)i * kRows) : 0.0f;
                }
#pragma unroll
                for (uint32_t i = 0; i < kChunk; ++i) {
                    float sum = __uint_as_float(v[i]) + a0[i];
                    if (two) {
                        sum += a1[i];
                    }
                    v[i] = __float_as_uint(sum);
                }
            }
            if constexpr (kChunk == 32u) {
                if (staged) {
                    if (args.epilogue == kEpilogueSwiglu) {
                        store_chunk_staged<YT, true>(args, place, stage + wq * kStoreStageBytes, lane,
                                                     (place.j0 + wq * 32u) / 2u, i0 + c0, v);
                    } else {
                        store_chunk_staged<YT, false>(args, place, stage + wq * kStoreStageBytes, lane,
                                                      place.j0 + wq * 32u, i0 + c0, v);
                    }
                    continue;
                }
            }
            store_chunk<kChunk, YT>(args, place, lane_row, j, i0 + c0, v);
        }
    }
    // The accumulator buffer is free again.
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0u) {
        mbar_arrive(acc_empty_bar);
    }
    if (!owner) {
        // Publish this warp's quarter of the partial tile.  Every lane makes its own stores
        // visible first; this happens at the start of a block's range, off the critical path.
        __threadfence();
        __syncwarp();
        if (lane == 0u) {
            st_release_gpu(args.flags + 4u * blockIdx.x + wq, 1u);
        }
    } else if (!whole) {
        // Hand the consumed slots back for the next launch (ordered by the end of the kernel).
        for (unsigned int base = blockIdx.x + 1u; base <= last_cc; base += 32u) {
            const unsigned int cc = base + lane;
            if (cc <= last_cc) {
                *reinterpret_cast<volatile unsigned int *>(args.flags + 4u * cc + wq) = 0u;
            }
        }
    }
}

// Launch with or without the programmatic-dependent-launch attribute.  In the tests' host
// emulation the blocks run as host threads instead (emulate_grid, q8_launch.h).
template <typename Kernel>
inline cudaError_t launch_tile_kernel(Kernel kernel, unsigned int grid, unsigned int smem_bytes,
                                      cudaStream_t stream, bool overlap, const CUtensorMap &tw,
                                      const CUtensorMap &tx, const UmmaArgs &args, unsigned int threads = kThreads,
                                      unsigned int cluster = 0u)
{
#ifdef Q8_HOST_EMULATION
    (void)smem_bytes;
    (void)stream;
    (void)overlap;
    (void)cluster;
    emulate_grid(dim3(grid, 1, 1), threads, [&] { kernel(tw, tx, args); });
    return cudaSuccess;
#else
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid, 1, 1);
    config.blockDim = dim3(threads, 1, 1);
    config.dynamicSmemBytes = smem_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    unsigned int count = 0;
    if (overlap) {
        attribute[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    if (cluster > 1u) {
        // `cluster` consecutive blocks run together and reach each other's shared memory
        attribute[count].id = cudaLaunchAttributeClusterDimension;
        attribute[count].val.clusterDim.x = cluster;
        attribute[count].val.clusterDim.y = 1;
        attribute[count].val.clusterDim.z = 1;
        ++count;
    }
    config.attrs = attribute;
    config.numAttrs = count;
    return cudaLaunchKernelEx(&config, kernel, tw, tx, args);
#endif
}

// Host launcher of the decode-regime kernel (q8_stream.cu), token tiles 16..128.
cudaError_t launch_stream_kernel(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                                 const UmmaArgs &args, unsigned int grid, unsigned int ntok, int y_dtype);

// Host launcher of the decode kernel for batches of up to 32 rows (q8_decode.cu) and the choice
// of its grid: a cluster of `*cluster` blocks per weight row tile, or (0) the unit schedule.
unsigned int decode_grid(unsigned int row_tiles, unsigned int segs, unsigned int sm_count,
                         unsigned int scratch_blocks, unsigned int *cluster);
cudaError_t launch_decode_kernel(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                                 const UmmaArgs &args, unsigned int grid, unsigned int cluster, unsigned int ntok,
                                 int y_dtype);

// Host launcher of the second prefill-regime kernel (q8_wide.cu), token tiles of 256.
cudaError_t launch_wide_kernel(cudaStream_t stream, const CUtensorMap &tw, const CUtensorMap &tx,
                               const UmmaArgs &args, unsigned int grid, int y_dtype);

} // namespace q8
