// Host model of the streaming kernel's division of work, built on the kernel's own helpers
// (unit_range, WorkIter, last_holder from q8_tile.cuh).  For a sweep of shapes and grid sizes
// it checks the properties the device protocol rests on:
//
//   1. every (tile, segment) unit is computed exactly once;
//   2. a block holds at most one piece of a tile whose first segment it does not hold (it has
//      one slot for partial sums and one set of flags), and that piece is its first;
//   3. a piece that starts a tile without finishing it is its block's last piece, so a block
//      only ever waits after it has published its own partial sums: no cycle of waits;
//   4. last_holder() names exactly the blocks that hold the remaining segments of that tile,
//      and they are the blocks directly after the owner;
//   5. no block that takes part is without work;
//   6. the bytes a launch asks L2 for on behalf of the next product (next_unit_pieces) are
//      exactly the weight bytes of the first units of the same block index there.
//
// Prints "ok <cases>" and exits 0, or the first violated property and exits 1.
#include <cstdio>
#include <cstdlib>
#include <utility>
#include <vector>

#include "q8_tile.cuh"

using namespace q8;

struct Piece {
    uint32_t tile, s0, s1;
};

static int fail(const char *what, unsigned long long tiles, uint32_t segs, unsigned int grid, unsigned int b)
{
    std::printf("violated: %s (tiles %llu, segments %u, grid %u, block %u)\n", what, tiles, segs, grid, b);
    return 1;
}

// `dp_waves` whole waves of tiles dealt round-robin ahead of the cut tiles: 0 for the
// decode-regime kernel (everything is cut into units).
static int check(unsigned long long tiles, uint32_t segs, unsigned int grid, bool hybrid)
{
    const uint32_t waves = hybrid ? (uint32_t)(tiles / grid) : 0u;
    const uint32_t dp_tiles = waves * grid;
    const unsigned long long units = (tiles - dp_tiles) * segs;
    const unsigned int blocks = units < grid ? (unsigned int)units : grid;
    std::vector<unsigned int> seen((size_t)(tiles * segs), 0u);
    std::vector<std::vector<Piece>> work(grid);
    for (unsigned int b = 0; b < grid; ++b) {
        WorkIter it;
        it.segs = segs;
        it.u = 0;
        it.u_end = 0;
        if (b < blocks) {
            unit_range(b, blocks, units, &it.u, &it.u_end);
            if (it.u >= it.u_end) {
                return fail("a block in the schedule has no units", tiles, segs, grid, b);
            }
        }
        it.sk_tile0 = dp_tiles;
        it.dp_next = 0;
        it.dp_count = waves;
        it.dp_first = b;
        it.dp_stride = grid;
        Piece p;
        while (it.next(p.tile, p.s0, p.s1)) {
            if (p.tile >= tiles || p.s1 > segs || p.s0 >= p.s1) {
                return fail("piece out of range", tiles, segs, grid, b);
            }
            for (uint32_t s = p.s0; s < p.s1; ++s) {
                seen[(size_t)p.tile * segs + s] += 1u;
            }
            work[b].push_back(p);
        }
    }
    for (size_t i = 0; i < seen.size(); ++i) {
        if (seen[i] != 1u) {
            return fail("a unit is computed zero or several times", tiles, segs, grid, (unsigned int)(i / segs));
        }
    }
    for (unsigned int b = 0; b < grid; ++b) {
        const std::vector<Piece> &pieces = work[b];
        for (size_t i = 0; i < pieces.size(); ++i) {
            const Piece &p = pieces[i];
            const bool whole = p.s0 == 0u && p.s1 == segs;
            const bool owner = p.s0 == 0u;
            if (!owner && i != 0u) {
                return fail("a partial piece is not the block's first piece", tiles, segs, grid, b);
            }
            if (owner && !whole) {
                // In the hybrid order the cut tiles come first and whole tiles follow them, so
                // the waiting piece is the last of the cut pieces; every whole tile after it
                // needs nobody.  Nothing that is published may come after the wait.
                for (size_t later = i + 1; later < pieces.size(); ++later) {
                    if (pieces[later].s0 != 0u || pieces[later].s1 != segs) {
                        return fail("a block waits before it has published", tiles, segs, grid, b);
                    }
                }
                const unsigned long long cut_tile = p.tile - dp_tiles;
                const unsigned long long tile_end = (cut_tile + 1ull) * segs;
                const unsigned int last = last_holder(b, blocks, units, tile_end);
                uint32_t expect = p.s1;
                for (unsigned int cc = b + 1u; cc <= last; ++cc) {
                    if (cc >= blocks || work[cc].empty()) {
                        return fail("last_holder names a block without work", tiles, segs, grid, b);
                    }
                    const Piece &q = work[cc][0];
                    if (q.tile != p.tile || q.s0 != expect) {
                        return fail("a named holder does not continue the tile", tiles, segs, grid, b);
                    }
                    expect = q.s1;
                }
                if (expect != segs) {
                    return fail("the named holders do not finish the tile", tiles, segs, grid, b);
                }
            }
        }
    }
    return 0;
}

// The pieces a launch asks L2 for on behalf of the next product (next_unit_pieces) are exactly
// the bytes that the same block index reads in its first units there: inside the tensor, on
// 16-byte boundaries, each (row, segment) of those units once.
struct RecordEmit {
    std::vector<std::pair<unsigned long long, uint32_t>> *out;
    const unsigned char *base;
    void operator()(const unsigned char *at, uint32_t bytes) const
    {
        out->push_back({(unsigned long long)(at - base), bytes});
    }
};

static int check_next(unsigned int n, unsigned int k, unsigned int tok_tiles, unsigned int grid, unsigned int limit)
{
    static unsigned char anchor[16];
    UmmaArgs args;
    args.next_w = anchor;
    args.next_stride = (unsigned long long)(k / 32u) * 34u;
    args.next_n = n;
    args.next_segs = k / kSegK;
    args.next_tok_tiles = tok_tiles;
    args.next_units = limit;
    const unsigned long long total = args.next_stride * n;
    const unsigned int row_tiles = (n + kRows - 1u) / kRows;
    const unsigned long long units = (unsigned long long)row_tiles * tok_tiles * args.next_segs;
    const unsigned int blocks = units < grid ? (unsigned int)units : grid;
    for (unsigned int b = 0; b < grid; ++b) {
        std::vector<std::pair<unsigned long long, uint32_t>> pieces;
        next_unit_pieces(args, b, grid, RecordEmit{&pieces, anchor});
        if (b >= blocks) {
            if (!pieces.empty()) {
                return fail("a block without work in the next launch asks for bytes", n, k, grid, b);
            }
            continue;
        }
        unsigned long long u0, u1;
        unit_range(b, blocks, units, &u0, &u1);
        if (u1 > u0 + limit) {
            u1 = u0 + limit;
        }
        // expected: every (row, segment) of the units [u0, u1)
        unsigned long long want_bytes = 0, got_bytes = 0;
        for (unsigned long long u = u0; u < u1; ++u) {
            const unsigned int tile = (unsigned int)(u / args.next_segs);
            const unsigned int row0 = (tile / tok_tiles) * kRows;
            const unsigned int rows = n - row0 < kRows ? n - row0 : kRows;
            want_bytes += (unsigned long long)rows * kSegBytes;
        }
        for (const auto &p : pieces) {
            if ((p.first % 16ull) != 0ull || (p.second % 16u) != 0u || p.second == 0u || p.first + p.second > total) {
                return fail("a piece is off the 16-byte grid or outside the tensor", n, k, grid, b);
            }
            // the piece lies in one row and covers whole segments of it
            const unsigned long long row = p.first / args.next_stride;
            const unsigned long long in_row = p.first % args.next_stride;
            if ((in_row % kSegBytes) != 0ull || in_row + p.second > args.next_stride || row >= n) {
                return fail("a piece does not cover whole segments of one row", n, k, grid, b);
            }
            // and those segments belong to this block's units
            for (uint32_t s = 0; s < p.second / kSegBytes; ++s) {
                const unsigned int seg = (unsigned int)(in_row / kSegBytes) + s;
                const unsigned int row_tile = (unsigned int)(row / kRows);
                bool mine = false;
                for (unsigned int tt = 0; tt < tok_tiles && !mine; ++tt) {
                    const unsigned long long u = ((unsigned long long)row_tile * tok_tiles + tt) * args.next_segs + seg;
                    mine = u >= u0 && u < u1;
                }
                if (!mine) {
                    return fail("a piece belongs to another block's units", n, k, grid, b);
                }
            }
            got_bytes += p.second;
        }
        if (got_bytes != want_bytes) {
            return fail("the pieces are not the bytes of the first units", n, k, grid, b);
        }
    }
    return 0;
}

int main()
{
    unsigned long long cases = 0;
    const unsigned int grids[] = {1u, 2u, 3u, 7u, 16u, 37u, 64u, 132u, 147u, 148u, 160u};
    const uint32_t seg_counts[] = {1u, 2u, 3u, 4u, 8u, 16u, 32u, 56u};
    for (unsigned int grid : grids) {
        for (uint32_t segs : seg_counts) {
            for (unsigned long long tiles = 1; tiles <= 700; tiles += (tiles < 40 ? 1 : 13)) {
                for (int hybrid = 0; hybrid < 2; ++hybrid) {
                    if (check(tiles, segs, grid, hybrid != 0) != 0) {
                        return 1;
                    }
                    cases += 1;
                }
            }
        }
    }
    // shapes of the benchmark and the tests: (rows of w, depth, rows of x, token tile)
    const unsigned int shapes[][4] = {{6144, 4096, 32, 32},   {4096, 4096, 32, 32},  {28672, 4096, 32, 32},
                                      {4096, 14336, 32, 32},  {151936, 8192, 8, 16}, {18992, 8192, 8, 16},
                                      {4736, 4096, 300, 128}, {4096, 4096, 2048, 128}, {28672, 4096, 2048, 128},
                                      {130, 256, 1, 16},      {128, 256, 129, 128}};
    for (const auto &shape : shapes) {
        const unsigned long long row_tiles = (shape[0] + kRows - 1u) / kRows;
        const unsigned long long tok_tiles = (shape[2] + shape[3] - 1u) / shape[3];
        for (unsigned int grid : {148u, 132u}) {
            for (int hybrid = 0; hybrid < 2; ++hybrid) {
                if (check(row_tiles * tok_tiles, shape[1] / kSegK, grid, hybrid != 0) != 0) {
                    return 1;
                }
                cases += 1;
            }
        }
    }
    // the next-product pieces: (rows of w, depth, token tiles) x grid x unit limit
    const unsigned int next_shapes[][3] = {{6144, 4096, 1}, {4096, 4096, 1}, {28672, 4096, 1}, {4096, 14336, 1},
                                           {151936, 8192, 1}, {130, 256, 1}, {4736, 4096, 3}, {28672, 4096, 16},
                                           {100, 512, 2}};
    for (const auto &shape : next_shapes) {
        for (unsigned int grid : {148u, 132u, 7u}) {
            for (unsigned int limit : {1u, 6u, 40u}) {
                if (check_next(shape[0], shape[1], shape[2], grid, limit) != 0) {
                    return 1;
                }
                cases += 1;
            }
        }
    }
    std::printf("ok %llu\n", cases);
    return 0;
}
