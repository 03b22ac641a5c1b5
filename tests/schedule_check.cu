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
//   6. the decode kernel's own 32-bit range arithmetic (decode_range, decode_holder in
//      q8_decode.cu) deals every unit once and names the block that holds a unit.
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

// The decode kernel's range arithmetic: the ranges of the blocks tile [0, units) in order, none
// is empty, and decode_holder names the block whose range holds a unit.
static int check_decode(uint32_t units, uint32_t blocks)
{
    uint32_t at = 0;
    for (uint32_t b = 0; b < blocks; ++b) {
        uint32_t begin, end;
        decode_range(b, blocks, units, &begin, &end);
        if (begin != at || end <= begin) {
            return fail("decode ranges do not tile the units", units, 0u, blocks, b);
        }
        for (uint32_t u = begin; u < end; ++u) {
            if (decode_holder(u, blocks, units) != b) {
                return fail("decode_holder names another block", units, u, blocks, b);
            }
        }
        at = end;
    }
    return at == units ? 0 : fail("decode ranges stop short", units, 0u, blocks, 0u);
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
    // the decode kernel's ranges: two blocks per SM and odd grids
    for (uint32_t blocks : {1u, 2u, 7u, 148u, 160u, 264u, 296u}) {
        for (uint32_t units : {1u, 2u, 5u, 147u, 296u, 297u, 512u, 768u, 1792u, 3584u, 37984u}) {
            if (units < blocks) {
                continue;
            }
            if (check_decode(units, blocks) != 0) {
                return 1;
            }
            cases += 1;
        }
    }
    std::printf("ok %llu\n", cases);
    return 0;
}
