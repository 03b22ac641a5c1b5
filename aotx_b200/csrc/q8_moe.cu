// Routed experts as grouped products: the (token, rank) pairs are sorted by expert on the
// device, each expert's rows then form token tiles of 64, and the decode-regime tensor-core
// kernel runs over a table of (expert, token tile, weight row tile) entries, reading every
// expert's weights once for all of its tokens.
//
// The reference runs one single-row product per token and rank on the token's expert slice
// (cuda/model/expert_matrix.cu:8-27, loop cuda/model/experts_host.cu:99-111), which re-reads an
// expert's weights for every token routed to it.  The results are the same products; the
// rank-ordered weighted sum (cuda/model/experts.cu:77-98) is kept as it is.
#include <stdlib.h>

#include "q8_launch.h"
#include "q8_tile.cuh"

namespace q8 {

#define Q8_GROUP_THREADS 1024u
#define Q8_GROUP_MAX_EXPERTS 256u
#define Q8_GROUP_TOKENS_MAX 64u /* largest token tile of the grouped products */

#ifndef Q8_GROUP_TOKENS
#define Q8_GROUP_TOKENS 64u /* token tile of the grouped products */
#endif

static unsigned int group_tokens()
{
    return Q8_GROUP_TOKENS;
}

// One block.  Counts the pairs of every expert, places each pair in its expert's run of
// `sorted_pair` in ascending order of the pair index (a stable sort: the place of a pair, and
// with it the token tile it lands in and the points where that tile's sums are cut between
// blocks, is a function of the selections alone, so the results repeat bit for bit from run to
// run), and writes the two tile tables.
//
// Every warp takes one contiguous run of the pairs.  Pass 1 counts, per warp and expert, the
// warp's pairs (lanes that name the same expert find each other with a match); a scan over the
// warps turns the counts into each warp's first place within the expert; pass 2 walks the
// same run again and places the pairs, lanes in order within a step, steps in order within
// the warp, warps in order within the expert.
__global__ void __launch_bounds__(Q8_GROUP_THREADS)
q8_group_build_kernel(const unsigned int *__restrict__ ids, unsigned int tokens_max,
                      const unsigned int *tokens_dev, unsigned int used, unsigned int experts,
                      unsigned int ffn, unsigned int hidden, unsigned int *__restrict__ sorted_pair,
                      GroupTile *__restrict__ tiles_feed, GroupTile *__restrict__ tiles_down,
                      unsigned int *__restrict__ counts, unsigned int tile_tokens)
{
    __shared__ unsigned int count[Q8_GROUP_MAX_EXPERTS];
    __shared__ unsigned int offset[Q8_GROUP_MAX_EXPERTS];
    __shared__ unsigned int feed_base[Q8_GROUP_MAX_EXPERTS];
    __shared__ unsigned int down_base[Q8_GROUP_MAX_EXPERTS];
    __shared__ unsigned int placed;
    __shared__ unsigned int scan_pairs[Q8_GROUP_MAX_EXPERTS];
    __shared__ unsigned int scan_tiles[Q8_GROUP_MAX_EXPERTS];
    // per warp and expert: first the number of the warp's pairs, then the next free place of
    // the warp within the expert's run
    __shared__ unsigned int warp_place[Q8_GROUP_THREADS / 32u][Q8_GROUP_MAX_EXPERTS];
    unsigned int tokens = tokens_max;
    if (tokens_dev != nullptr) {
        unsigned int live = *tokens_dev;
        tokens = live < tokens_max ? live : tokens_max;
    }
    const unsigned int pairs = tokens * used;
    const unsigned int feed_rows = (ffn + kRows - 1u) / kRows;
    const unsigned int down_rows = (hidden + kRows - 1u) / kRows;
    const unsigned int warp = threadIdx.x >> 5;
    const unsigned int lane = threadIdx.x & 31u;
    const unsigned int warps = blockDim.x >> 5;
    // the warp's run of pairs, a whole number of steps of 32
    const unsigned int per_warp = ((pairs + warps - 1u) / warps + 31u) / 32u * 32u;
    const unsigned int run_begin = warp * per_warp < pairs ? warp * per_warp : pairs;
    const unsigned int run_end = run_begin + per_warp < pairs ? run_begin + per_warp : pairs;
    const unsigned int none = 0xFFFFFFFFu;

    for (unsigned int e = lane; e < experts; e += 32u) {
        warp_place[warp][e] = 0u;
    }
    __syncwarp();
    // A selection outside the expert table is left out of both passes (its result row is then
    // never written), rather than indexing past the tables.
    for (unsigned int first = run_begin; first < run_end; first += 32u) {
        const unsigned int p = first + lane;
        unsigned int e = p < run_end ? ids[p] : none;
        if (e >= experts) {
            e = none;
        }
        const unsigned int same = __match_any_sync(0xFFFFFFFFu, e);
        if (e != none && (same & ((1u << lane) - 1u)) == 0u) {
            warp_place[warp][e] += (unsigned int)__popc(same); // the lowest lane speaks for the expert
        }
        __syncwarp();
    }
    __syncthreads();
    for (unsigned int e = threadIdx.x; e < experts; e += blockDim.x) {
        unsigned int running = 0u;
        for (unsigned int w = 0u; w < warps; ++w) {
            const unsigned int here = warp_place[w][e];
            warp_place[w][e] = running;
            running += here;
        }
        count[e] = running;
    }
    __syncthreads();
    // running totals over the experts of the pairs and of the token tiles (a scan in shared
    // memory, one thread per expert): an expert's first place and first table entries
    {
        const unsigned int e = threadIdx.x;
        const unsigned int mine = e < experts ? count[e] : 0u;
        const unsigned int mine_tiles = (mine + tile_tokens - 1u) / tile_tokens;
        if (e < Q8_GROUP_MAX_EXPERTS) {
            scan_pairs[e] = mine;
            scan_tiles[e] = mine_tiles;
        }
        __syncthreads();
        for (unsigned int step = 1u; step < Q8_GROUP_MAX_EXPERTS; step <<= 1) {
            unsigned int add_pairs = 0u;
            unsigned int add_tiles = 0u;
            if (e < Q8_GROUP_MAX_EXPERTS && e >= step) {
                add_pairs = scan_pairs[e - step];
                add_tiles = scan_tiles[e - step];
            }
            __syncthreads();
            if (e < Q8_GROUP_MAX_EXPERTS) {
                scan_pairs[e] += add_pairs;
                scan_tiles[e] += add_tiles;
            }
            __syncthreads();
        }
        if (e < experts) {
            offset[e] = scan_pairs[e] - mine;
            feed_base[e] = (scan_tiles[e] - mine_tiles) * feed_rows;
            down_base[e] = (scan_tiles[e] - mine_tiles) * down_rows;
            if (e == experts - 1u) {
                counts[0] = scan_tiles[e] * feed_rows;
                counts[1] = scan_tiles[e] * down_rows;
                placed = scan_pairs[e];
            }
        }
    }
    __syncthreads();
    for (unsigned int first = run_begin; first < run_end; first += 32u) {
        const unsigned int p = first + lane;
        unsigned int e = p < run_end ? ids[p] : none;
        if (e >= experts) {
            e = none;
        }
        const unsigned int same = __match_any_sync(0xFFFFFFFFu, e);
        const unsigned int below = (unsigned int)__popc(same & ((1u << lane) - 1u));
        const unsigned int base = e != none ? warp_place[warp][e] : 0u;
        __syncwarp();
        if (e != none) {
            sorted_pair[offset[e] + base + below] = p;
            if (below == 0u) {
                warp_place[warp][e] = base + (unsigned int)__popc(same);
            }
        }
        __syncwarp();
    }
    // the places that pairs left out would have taken name no pair (the gather skips them)
    for (unsigned int at = placed + threadIdx.x; at < pairs; at += blockDim.x) {
        sorted_pair[at] = 0xFFFFFFFFu;
    }
    // the tile tables: a warp per expert, a lane per weight row tile
    for (unsigned int e = warp; e < experts; e += warps) {
        const unsigned int tok_tiles = (count[e] + tile_tokens - 1u) / tile_tokens;
        for (unsigned int tt = 0u; tt < tok_tiles; ++tt) {
            const unsigned int tok0 = offset[e] + tt * tile_tokens;
            unsigned int tok_limit = offset[e] + count[e];
            if (tok_limit > tok0 + tile_tokens) {
                tok_limit = tok0 + tile_tokens;
            }
            for (unsigned int r = lane; r < feed_rows; r += 32u) {
                GroupTile t;
                t.w_row = e * ffn + r * kRows;
                t.j0 = r * kRows;
                t.j_limit = ffn;
                t.tok0 = tok0;
                t.tok_limit = tok_limit;
                tiles_feed[feed_base[e] + tt * feed_rows + r] = t;
            }
            for (unsigned int r = lane; r < down_rows; r += 32u) {
                GroupTile t;
                t.w_row = e * hidden + r * kRows;
                t.j0 = r * kRows;
                t.j_limit = hidden;
                t.tok0 = tok0;
                t.tok_limit = tok_limit;
                tiles_down[down_base[e] + tt * down_rows + r] = t;
            }
        }
    }
}

// x_sorted[i] = x[sorted_pair[i] / used], rows of `hidden` halves, 16 bytes per thread step.
// Expert parallel: token t is row t % rows_per_part of array t / rows_per_part (the tokens of
// all GPUs, each GPU's in its own array, read through peer-mapped addresses).
__global__ void q8_gather_rows_kernel(const __grid_constant__ RowParts x, const unsigned int *__restrict__ sorted_pair,
                                      unsigned int tokens_max, const unsigned int *tokens_dev,
                                      unsigned int used, unsigned int row_chunks, uint4 *__restrict__ out)
{
    unsigned int tokens = tokens_max;
    if (tokens_dev != nullptr) {
        unsigned int live = *tokens_dev;
        tokens = live < tokens_max ? live : tokens_max;
    }
    const unsigned int pairs = tokens * used;
    for (unsigned int i = blockIdx.x; i < pairs; i += gridDim.x) {
        const unsigned int p = sorted_pair[i];
        if (p >= pairs) {
            continue; // no pair here: a selection outside the expert table was left out
        }
        unsigned int t = p / used;
        const uint4 *from = static_cast<const uint4 *>(x.base[0]);
        if (x.parts > 1u) {
            from = static_cast<const uint4 *>(x.base[t / x.rows_per_part]);
            t = t % x.rows_per_part;
        }
        for (unsigned int c = threadIdx.x; c < row_chunks; c += blockDim.x) {
            out[(size_t)i * row_chunks + c] = from[(size_t)t * row_chunks + c];
        }
    }
}

// ids_all[q * count + i] = ids_of_rank[q][i] - first: the selections of every GPU's tokens,
// numbered from this GPU's first expert (unsigned: an expert below it wraps to a number that
// names no local expert, like one above the last).
struct IdParts {
    const unsigned int *base[8];
};

__global__ void q8_collect_ids_kernel(const __grid_constant__ IdParts ids, unsigned int parts, unsigned int count,
                                      unsigned int first, unsigned int *__restrict__ ids_all)
{
    const unsigned int total = parts * count;
    for (unsigned int at = blockIdx.x * blockDim.x + threadIdx.x; at < total; at += gridDim.x * blockDim.x) {
        const unsigned int q = at / count;
        ids_all[at] = ids.base[q][at - q * count] - first;
    }
}

cudaError_t launch_collect_ids(cudaStream_t stream, const unsigned int *const *ids_of_rank, unsigned int parts,
                               unsigned int count, unsigned int first_expert, unsigned int *ids_all)
{
    IdParts ids = {};
    for (unsigned int q = 0; q < parts && q < 8u; ++q) {
        ids.base[q] = ids_of_rank[q];
    }
    const unsigned int total = parts * count;
    const unsigned int grid = (total + 255u) / 256u < 148u * 4u ? (total + 255u) / 256u : 148u * 4u;
    return launch_kernel(q8_collect_ids_kernel, grid, 256, 0, stream, ids, parts, count, first_expert, ids_all);
}

// act = half(silu(gate) * up), silu(g) = g / (1 + exp(-g))  (cuda/model/norm.cu:92-105)
__global__ void q8_swiglu_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                 unsigned int tokens_max, const unsigned int *tokens_dev, unsigned int used,
                                 unsigned int ffn, __half *__restrict__ act)
{
    unsigned int tokens = tokens_max;
    if (tokens_dev != nullptr) {
        unsigned int live = *tokens_dev;
        tokens = live < tokens_max ? live : tokens_max;
    }
    const size_t total = (size_t)tokens * used * ffn;
    for (size_t at = (size_t)blockIdx.x * blockDim.x + threadIdx.x; at < total;
         at += (size_t)gridDim.x * blockDim.x) {
        float g = gate[at];
        float unit = g / (1.0f + expf(-g));
        act[at] = __float2half_rn(unit * up[at]);
    }
}

bool moe_grouped_supports(const void *w_gate, const void *w_up, const void *w_down, const void *x,
                          unsigned int hidden, unsigned int ffn, unsigned int experts)
{
    auto aligned16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0u; };
    return (hidden % kSegK) == 0u && (ffn % kSegK) == 0u && experts <= Q8_GROUP_MAX_EXPERTS && aligned16(w_gate)
        && aligned16(w_up) && aligned16(w_down) && aligned16(x);
}

static size_t up256(size_t v)
{
    return (v + 255u) / 256u * 256u;
}

MoeWorkspace moe_workspace_layout(unsigned int tokens, unsigned int used, unsigned int hidden,
                                  unsigned int ffn, unsigned int experts)
{
    MoeWorkspace ws;
    const size_t pairs = (size_t)tokens * used;
    const size_t tok_tiles = pairs / 16u + experts; /* room for the smallest token tile */
    /* room for the interleaved gate+up form as well, which has twice the rows */
    ws.max_feed = (unsigned int)(tok_tiles * ((2u * ffn + kRows - 1u) / kRows));
    ws.max_down = (unsigned int)(tok_tiles * ((hidden + kRows - 1u) / kRows));
    size_t at = 0;
    ws.act = at;
    at += up256(pairs * ffn * sizeof(unsigned short));
    ws.proj = at;
    at += up256(pairs * hidden * sizeof(float));
    ws.sorted_pair = at;
    at += up256(pairs * sizeof(unsigned int));
    ws.counts = at;
    at += 256;
    ws.tiles_feed = at;
    at += up256((size_t)ws.max_feed * sizeof(GroupTile));
    ws.tiles_down = at;
    at += up256((size_t)ws.max_down * sizeof(GroupTile));
    ws.x_sorted = at;
    at += up256(pairs * hidden * sizeof(unsigned short));
    ws.gate = at;
    at += up256(pairs * ffn * sizeof(float));
    ws.up = at;
    at += up256(pairs * ffn * sizeof(float));
    ws.bytes = at;
    return ws;
}

cudaError_t launch_moe_grouped(cudaStream_t stream, const UmmaScratch &scratch, unsigned int sm_count,
                               unsigned int *launches, bool overlap, const void *w_gate, const void *w_up,
                               const void *w_down, unsigned int experts, unsigned int hidden,
                               unsigned int ffn, const void *x, const unsigned int *ids, unsigned int tokens,
                               const unsigned int *tokens_dev, unsigned int used, unsigned char *workspace,
                               const MoeWorkspace &ws, const RowParts *x_parts, float *proj_out)
{
    const unsigned int pairs = tokens * used;
    const unsigned int tile_tokens = group_tokens();
    unsigned int *sorted_pair = reinterpret_cast<unsigned int *>(workspace + ws.sorted_pair);
    unsigned int *counts = reinterpret_cast<unsigned int *>(workspace + ws.counts);
    GroupTile *tiles_feed = reinterpret_cast<GroupTile *>(workspace + ws.tiles_feed);
    GroupTile *tiles_down = reinterpret_cast<GroupTile *>(workspace + ws.tiles_down);
    __half *x_sorted = reinterpret_cast<__half *>(workspace + ws.x_sorted);
    float *gate = reinterpret_cast<float *>(workspace + ws.gate);
    float *up = reinterpret_cast<float *>(workspace + ws.up);
    __half *act = reinterpret_cast<__half *>(workspace + ws.act);
    float *proj = proj_out != nullptr ? proj_out : reinterpret_cast<float *>(workspace + ws.proj);
    RowParts rows = {};
    rows.base[0] = x;
    rows.parts = 1u;
    if (x_parts != nullptr) {
        rows = *x_parts;
    }

    cudaError_t err = launch_kernel(q8_group_build_kernel, 1, Q8_GROUP_THREADS, 0, stream, ids, tokens, tokens_dev,
                                    used, experts, ffn, hidden, sorted_pair, tiles_feed, tiles_down, counts,
                                    tile_tokens);
    if (err != cudaSuccess) {
        return err;
    }
    const unsigned int wave = pairs < 148u * 16u ? pairs : 148u * 16u;
    err = launch_kernel(q8_gather_rows_kernel, wave, 128, 0, stream, rows, sorted_pair, tokens,
                        tokens_dev, used, hidden / 8u, reinterpret_cast<uint4 *>(x_sorted));
    if (err != cudaSuccess) {
        return err;
    }
    err = launch_umma_grouped(stream, scratch, sm_count, w_gate, experts * ffn, hidden, x_sorted, pairs,
                              tile_tokens, tiles_feed, counts + 0, ws.max_feed, nullptr, gate, ffn, 0,
                              (*launches)++, overlap);
    if (err != cudaSuccess) {
        return err;
    }
    err = launch_umma_grouped(stream, scratch, sm_count, w_up, experts * ffn, hidden, x_sorted, pairs,
                              tile_tokens, tiles_feed, counts + 0, ws.max_feed, nullptr, up, ffn, 0,
                              (*launches)++, overlap);
    if (err != cudaSuccess) {
        return err;
    }
    err = launch_kernel(q8_swiglu_kernel, 148 * 8, 256, 0, stream, gate, up, tokens, tokens_dev, used, ffn, act);
    if (err != cudaSuccess) {
        return err;
    }
    return launch_umma_grouped(stream, scratch, sm_count, w_down, experts * hidden, ffn, act, pairs,
                               tile_tokens, tiles_down, counts + 1, ws.max_down, sorted_pair, proj, hidden,
                               0, (*launches)++, overlap);
}

// The same step with gate and up in one tensor, rows interleaved (row 2r of an expert is its
// gate row r, row 2r + 1 its up row r): one grouped product whose store applies the gated unit
// and writes the half activations, then the down product.  Two tensor-core launches instead of
// three and an elementwise kernel, and no float gate / up round trip.
cudaError_t launch_moe_grouped_fused(cudaStream_t stream, const UmmaScratch &scratch, unsigned int sm_count,
                                     unsigned int *launches, bool overlap, const void *w_gate_up,
                                     const void *w_down, unsigned int experts, unsigned int hidden,
                                     unsigned int ffn, const void *x, const unsigned int *ids,
                                     unsigned int tokens, const unsigned int *tokens_dev, unsigned int used,
                                     unsigned char *workspace, const MoeWorkspace &ws)
{
    const unsigned int pairs = tokens * used;
    const unsigned int tile_tokens = group_tokens();
    unsigned int *sorted_pair = reinterpret_cast<unsigned int *>(workspace + ws.sorted_pair);
    unsigned int *counts = reinterpret_cast<unsigned int *>(workspace + ws.counts);
    GroupTile *tiles_feed = reinterpret_cast<GroupTile *>(workspace + ws.tiles_feed);
    GroupTile *tiles_down = reinterpret_cast<GroupTile *>(workspace + ws.tiles_down);
    __half *x_sorted = reinterpret_cast<__half *>(workspace + ws.x_sorted);
    __half *act = reinterpret_cast<__half *>(workspace + ws.act);
    float *proj = reinterpret_cast<float *>(workspace + ws.proj);

    // the feed table is built over the 2 * ffn interleaved rows of every expert
    cudaError_t err = launch_kernel(q8_group_build_kernel, 1, Q8_GROUP_THREADS, 0, stream, ids, tokens, tokens_dev,
                                    used, experts, 2u * ffn, hidden, sorted_pair, tiles_feed, tiles_down, counts,
                                    tile_tokens);
    if (err != cudaSuccess) {
        return err;
    }
    const unsigned int wave = pairs < 148u * 16u ? pairs : 148u * 16u;
    RowParts rows = {};
    rows.base[0] = x;
    rows.parts = 1u;
    err = launch_kernel(q8_gather_rows_kernel, wave, 128, 0, stream, rows, sorted_pair, tokens,
                        tokens_dev, used, hidden / 8u, reinterpret_cast<uint4 *>(x_sorted));
    if (err != cudaSuccess) {
        return err;
    }
    err = launch_umma_grouped(stream, scratch, sm_count, w_gate_up, experts * 2u * ffn, hidden, x_sorted, pairs,
                              tile_tokens, tiles_feed, counts + 0, ws.max_feed, nullptr, act, ffn, 1,
                              (*launches)++, overlap, kEpilogueSwiglu);
    if (err != cudaSuccess) {
        return err;
    }
    return launch_umma_grouped(stream, scratch, sm_count, w_down, experts * hidden, ffn, act, pairs,
                               tile_tokens, tiles_down, counts + 1, ws.max_down, sorted_pair, proj, hidden,
                               0, (*launches)++, overlap);
}

} // namespace q8
