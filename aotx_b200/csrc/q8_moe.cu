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

static unsigned int group_tokens()
{
    return 64u;
}

// One block.  Counts the pairs of every expert, places each pair in its expert's run of
// `sorted_pair` in ascending order of the pair index (a stable sort: the place of a pair, and
// with it the token tile it lands in and the points where that tile's sums are cut between
// blocks, is a function of the selections alone, so the results repeat bit for bit from run to
// run), and writes the two tile tables.
__global__ void __launch_bounds__(Q8_GROUP_THREADS)
q8_group_build_kernel(const unsigned int *__restrict__ ids, unsigned int tokens_max,
                      const unsigned int *tokens_dev, unsigned int used, unsigned int experts,
                      unsigned int ffn, unsigned int hidden, unsigned int *__restrict__ sorted_pair,
                      GroupTile *__restrict__ tiles_feed, GroupTile *__restrict__ tiles_down,
                      unsigned int *__restrict__ counts, unsigned int tile_tokens)
{
    __shared__ unsigned int count[Q8_GROUP_MAX_EXPERTS];
    __shared__ unsigned int offset[Q8_GROUP_MAX_EXPERTS];
    __shared__ unsigned int cursor[Q8_GROUP_MAX_EXPERTS];
    __shared__ unsigned int feed_base[Q8_GROUP_MAX_EXPERTS];
    __shared__ unsigned int down_base[Q8_GROUP_MAX_EXPERTS];
    __shared__ unsigned int placed;
    // one round of the placement: the expert of every thread's pair, and per warp and expert
    // first the number of its pairs in this round, then the place of the warp's first one
    __shared__ unsigned int round_expert[Q8_GROUP_THREADS];
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
    for (unsigned int e = threadIdx.x; e < experts; e += blockDim.x) {
        count[e] = 0u;
        cursor[e] = 0u;
    }
    __syncthreads();
    // A selection outside the expert table is left out of both passes (its result row is then
    // never written), rather than indexing past the tables.
    for (unsigned int p = threadIdx.x; p < pairs; p += blockDim.x) {
        unsigned int e = ids[p];
        if (e < experts) {
            atomicAdd(&count[e], 1u);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0u) {
        unsigned int at = 0u;
        unsigned int feed = 0u;
        unsigned int down = 0u;
        for (unsigned int e = 0u; e < experts; ++e) {
            offset[e] = at;
            feed_base[e] = feed;
            down_base[e] = down;
            unsigned int tok_tiles = (count[e] + tile_tokens - 1u) / tile_tokens;
            at += count[e];
            feed += tok_tiles * feed_rows;
            down += tok_tiles * down_rows;
        }
        counts[0] = feed;
        counts[1] = down;
        placed = at;
    }
    __syncthreads();
    // Placement, blockDim pairs per round, in order of the pair index: a pair's place is its
    // expert's offset + the pairs of that expert in earlier rounds (cursor) + those in lower
    // warps of this round + those in lower lanes of its own warp.
    for (unsigned int first = 0u; first < pairs; first += blockDim.x) {
        const unsigned int p = first + threadIdx.x;
        unsigned int e = p < pairs ? ids[p] : 0xFFFFFFFFu;
        if (e >= experts) {
            e = 0xFFFFFFFFu;
        }
        round_expert[threadIdx.x] = e;
        for (unsigned int i = lane; i < experts; i += 32u) {
            warp_place[warp][i] = 0u;
        }
        __syncthreads();
        unsigned int below = 0u;
        unsigned int same = 0u;
        if (e != 0xFFFFFFFFu) {
            for (unsigned int i = 0u; i < 32u; ++i) {
                const unsigned int other = round_expert[warp * 32u + i];
                same += other == e ? 1u : 0u;
                below += (other == e && i < lane) ? 1u : 0u;
            }
            if (below == 0u) {
                warp_place[warp][e] = same; // the first lane with this expert speaks for the warp
            }
        }
        __syncthreads();
        for (unsigned int i = threadIdx.x; i < experts; i += blockDim.x) {
            unsigned int running = cursor[i];
            for (unsigned int w = 0u; w < warps; ++w) {
                const unsigned int here = warp_place[w][i];
                warp_place[w][i] = running;
                running += here;
            }
            cursor[i] = running;
        }
        __syncthreads();
        if (e != 0xFFFFFFFFu) {
            sorted_pair[offset[e] + warp_place[warp][e] + below] = p;
        }
        __syncthreads();
    }
    // the places that pairs left out would have taken name no pair (the gather skips them)
    for (unsigned int at = placed + threadIdx.x; at < pairs; at += blockDim.x) {
        sorted_pair[at] = 0xFFFFFFFFu;
    }
    for (unsigned int e = threadIdx.x; e < experts; e += blockDim.x) {
        unsigned int tok_tiles = (count[e] + tile_tokens - 1u) / tile_tokens;
        for (unsigned int tt = 0u; tt < tok_tiles; ++tt) {
            unsigned int tok0 = offset[e] + tt * tile_tokens;
            unsigned int tok_limit = offset[e] + count[e];
            if (tok_limit > tok0 + tile_tokens) {
                tok_limit = tok0 + tile_tokens;
            }
            for (unsigned int r = 0u; r < feed_rows; ++r) {
                GroupTile t;
                t.w_row = e * ffn + r * kRows;
                t.j0 = r * kRows;
                t.j_limit = ffn;
                t.tok0 = tok0;
                t.tok_limit = tok_limit;
                tiles_feed[feed_base[e] + tt * feed_rows + r] = t;
            }
            for (unsigned int r = 0u; r < down_rows; ++r) {
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
__global__ void q8_gather_rows_kernel(const uint4 *__restrict__ x, const unsigned int *__restrict__ sorted_pair,
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
        const unsigned int t = p / used;
        for (unsigned int c = threadIdx.x; c < row_chunks; c += blockDim.x) {
            out[(size_t)i * row_chunks + c] = x[(size_t)t * row_chunks + c];
        }
    }
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
                               const MoeWorkspace &ws)
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
    float *proj = reinterpret_cast<float *>(workspace + ws.proj);

    cudaError_t err = launch_kernel(q8_group_build_kernel, 1, Q8_GROUP_THREADS, 0, stream, ids, tokens, tokens_dev,
                                    used, experts, ffn, hidden, sorted_pair, tiles_feed, tiles_down, counts,
                                    tile_tokens);
    if (err != cudaSuccess) {
        return err;
    }
    const unsigned int wave = pairs < 148u * 16u ? pairs : 148u * 16u;
    err = launch_kernel(q8_gather_rows_kernel, wave, 128, 0, stream, static_cast<const uint4 *>(x), sorted_pair, tokens,
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
    err = launch_kernel(q8_gather_rows_kernel, wave, 128, 0, stream, static_cast<const uint4 *>(x), sorted_pair, tokens,
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
