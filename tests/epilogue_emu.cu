// The store side of the tensor-core kernels (epilogue_piece in aotx_b200/csrc/q8_tile.cuh) run
// on the host: the function's source is compiled as host code, the four epilogue warps of every
// block run as host threads, all blocks at once (the owner of a cut tile waits for flags that
// later blocks raise), and the few hardware helpers the function calls are stand-ins:
//   tcgen05.ld      -> a read of a host array holding the block's accumulator
//   ld.acquire / st.release / __ldcg / __stcg / atomicOr -> ordinary atomics and loads
//   mbarrier arrive, tcgen05 fences, clock64 -> inert
// The driver below walks each block's share of the units exactly as the kernels' epilogue
// loops do and hands every piece its accumulator, computed on the host in float.  What this
// checks: who owns a cut tile, the partial-sum hand-over between blocks, the row and column
// of every store, rows past the batch, the row map of the grouped mode, and the three store
// modes (plain, add into a float y, gated unit over row pairs).  Not checked: the hardware.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace emu {

struct Index {
    unsigned int x, y, z;
};

class Barrier {
public:
    explicit Barrier(unsigned int count) : count_(count), waiting_(0), generation_(0) {}
    void wait()
    {
        std::unique_lock<std::mutex> lock(mutex_);
        const unsigned int generation = generation_;
        if (++waiting_ == count_) {
            waiting_ = 0;
            generation_ += 1;
            wake_.notify_all();
        } else {
            wake_.wait(lock, [&] { return generation_ != generation; });
        }
    }

private:
    std::mutex mutex_;
    std::condition_variable wake_;
    unsigned int count_, waiting_, generation_;
};

struct Warp {
    Barrier barrier{32};
    uint32_t slot[32];
};

thread_local Index thread_index = {0, 0, 0};
thread_local Index block_index = {0, 0, 0};
thread_local Warp *warp = nullptr;
thread_local const float *accumulator = nullptr; // [128 lanes][columns] of the piece at hand
thread_local unsigned int accumulator_columns = 0;
thread_local unsigned int shift = 0;

inline float shfl_xor(float value, unsigned int mask)
{
    const unsigned int lane = thread_index.x % 32u;
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    warp->slot[lane] = bits;
    warp->barrier.wait();
    bits = warp->slot[lane ^ mask];
    warp->barrier.wait();
    std::memcpy(&value, &bits, 4);
    return value;
}

inline void sync_warp()
{
    warp->barrier.wait();
}

inline float uint_as_float(uint32_t bits)
{
    float value;
    std::memcpy(&value, &bits, 4);
    return value;
}

inline uint32_t float_as_uint(float value)
{
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    return bits;
}

inline long long clock_now()
{
    return 0; // waits in the emulation end because the flags come, never because time ran out
}

inline unsigned int atomic_or(unsigned int *word, unsigned int bits)
{
    return reinterpret_cast<std::atomic<unsigned int> *>(word)->fetch_or(bits);
}

inline float load_global(const float *p)
{
    return *p;
}

inline void store_global(float *p, float v)
{
    *p = v;
}

inline void fence()
{
    std::atomic_thread_fence(std::memory_order_seq_cst);
}

} // namespace emu

#undef __global__
#define __global__
#undef __device__
#define __device__
#undef __host__
#define __host__
#undef __forceinline__
#define __forceinline__ inline
#undef __launch_bounds__
#define __launch_bounds__(...)
#define threadIdx (emu::thread_index)
#define blockIdx (emu::block_index)
#define __shfl_xor_sync(mask, value, lanes) emu::shfl_xor((value), (lanes))
#define __syncwarp() emu::sync_warp()
#define __uint_as_float(bits) emu::uint_as_float(bits)
#define __float_as_uint(value) emu::float_as_uint(value)
#define clock64() emu::clock_now()
// only the store side runs here: the converters' vote is never reached
#define __any_sync(mask, predicate) (predicate)
#define atomicOr(word, bits) emu::atomic_or((word), (bits))
#define __ldg(p) (*(p))
#define __ldcg(p) emu::load_global(p)
#define __stcg(p, v) emu::store_global((p), (v))
#define __threadfence() emu::fence()
#define __cvta_generic_to_shared(p) ((size_t)(p))

// the helpers with inline PTX get other names while the common header is read ...
#define tmem_ld_32x32 ptx_tmem_ld_32x32
#define tmem_ld_32x16 ptx_tmem_ld_32x16
#define tmem_ld_wait ptx_tmem_ld_wait
#define tc_fence_before_sync ptx_tc_fence_before_sync
#define mbar_arrive ptx_mbar_arrive
#define ld_acquire_gpu ptx_ld_acquire_gpu
#define st_release_gpu ptx_st_release_gpu
#define ld_shared_v4 ptx_ld_shared_v4
#define st_shared_b32 ptx_st_shared_b32
#define st_shared_b16 ptx_st_shared_b16
#include "q8_common.cuh"
#undef tmem_ld_32x32
#undef tmem_ld_32x16
#undef tmem_ld_wait
#undef tc_fence_before_sync
#undef mbar_arrive
#undef ld_acquire_gpu
#undef st_release_gpu
#undef ld_shared_v4
#undef st_shared_b32
#undef st_shared_b16

// ... and the stand-ins take the names the tile header calls
namespace q8 {

// a thread reads `count` columns of its own lane of the accumulator (lane base in bits 16..31)
inline void emu_tmem_read(uint32_t taddr, uint32_t *v, unsigned int count)
{
    const unsigned int lane = ((taddr >> 16) & 0xFFFFu) + emu::thread_index.x % 32u;
    const unsigned int column = taddr & 0xFFFFu;
    for (unsigned int i = 0; i < count; ++i) {
        v[i] = emu::float_as_uint(emu::accumulator[(size_t)lane * emu::accumulator_columns + column + i]);
    }
}

inline void tmem_ld_32x32(uint32_t taddr, uint32_t *v)
{
    emu_tmem_read(taddr, v, 32);
}

inline void tmem_ld_32x16(uint32_t taddr, uint32_t *v)
{
    emu_tmem_read(taddr, v, 16);
}

// the row-wise store through a staging buffer is not driven here (no buffer is handed in); the
// whole-kernel emulation (tests/stream_emu.cu) runs it
inline void ld_shared_v4(uint32_t, uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d)
{
    a = b = c = d = 0u;
}
inline void st_shared_b32(uint32_t, uint32_t) {}
inline void st_shared_b16(uint32_t, uint32_t) {}

inline void tmem_ld_wait() {}
inline void tc_fence_before_sync() {}
inline void mbar_arrive(uint32_t) {}

inline uint32_t ld_acquire_gpu(const unsigned int *p)
{
    return reinterpret_cast<const std::atomic<unsigned int> *>(p)->load(std::memory_order_acquire);
}

inline void st_release_gpu(unsigned int *p, uint32_t v)
{
    reinterpret_cast<std::atomic<unsigned int> *>(p)->store(v, std::memory_order_release);
}

} // namespace q8

#include "q8_tile.cuh"

using namespace q8;

// One launch.  x[m][k] and w[n][k] are plain floats here (the epilogue does not care how the
// sums were formed); `mode`: 0 store, 1 add, 2 gated unit; y is float [rows_y][ldy].
// `row_map` (may be null) and `group` (tiles from a table) follow the kernels' grouped mode:
// with group != 0 the table has one entry per row tile of w, all for token rows [0, m).
template <int NTOK>
static void run_launch(const float *w, uint32_t n, uint32_t k, const float *x, uint32_t m, float *y, uint32_t ldy,
                       uint32_t mode, const unsigned int *row_map, uint32_t group, uint32_t grid,
                       unsigned int *status_out)
{
    const uint32_t segs = k / kSegK;
    const uint32_t row_tiles = (n + kRows - 1u) / kRows;
    const uint32_t tok_tiles = group ? 1u : (m + NTOK - 1u) / NTOK;
    std::vector<GroupTile> table;
    if (group) {
        for (uint32_t r = 0; r < row_tiles; ++r) {
            table.push_back({r * kRows, r * kRows, n, 0u, m});
        }
    }
    const unsigned long long units = (unsigned long long)row_tiles * tok_tiles * segs;
    const unsigned int blocks = units < grid ? (unsigned int)units : grid;
    std::vector<float> partial((size_t)grid * kRows * NTOK, 0.0f);
    std::vector<unsigned int> flags((size_t)grid * 4u, 0u);
    unsigned int status = 0;
    UmmaArgs args;
    std::memset(&args, 0, sizeof args);
    args.n = n;
    args.k = k;
    args.m_max = m;
    args.y = y;
    args.partial = partial.data();
    args.flags = flags.data();
    args.status = &status;
    args.tile_floats = (unsigned long long)kRows * NTOK;
    args.group_tiles = group ? table.data() : nullptr;
    args.row_map = row_map;
    args.ldy = ldy;
    args.epilogue = mode;

    std::vector<std::thread> threads;
    std::vector<std::vector<emu::Warp>> warps(blocks);
    for (auto &set : warps) {
        set = std::vector<emu::Warp>(4);
    }
    for (unsigned int b = 0; b < blocks; ++b) {
        for (unsigned int t = 0; t < 128u; ++t) {
            threads.emplace_back([&, b, t] {
                emu::thread_index = {t, 0, 0};
                emu::block_index = {b, 0, 0};
                emu::warp = &warps[b][t / 32u];
                volatile uint32_t abort_flag = 0;
                unsigned long long u, u_end;
                unit_range(b, blocks, units, &u, &u_end);
                std::vector<float> acc((size_t)kRows * NTOK);
                while (u < u_end) {
                    const uint32_t tile = (uint32_t)(u / segs);
                    const uint32_t s0 = (uint32_t)(u % segs);
                    const unsigned long long left = u_end - u;
                    const uint32_t s1 = (segs - s0) < left ? segs : (uint32_t)(s0 + left);
                    // what the MMAs of this piece leave in tensor memory: lane = row of w in the
                    // tile, column = row of x in the token tile, over segments [s0, s1)
                    const uint32_t row0 = (tile / tok_tiles) * kRows;
                    const uint32_t tok0 = (tile % tok_tiles) * NTOK;
                    for (uint32_t lane = 0; lane < kRows; ++lane) {
                        for (uint32_t col = 0; col < (uint32_t)NTOK; ++col) {
                            float sum = 0.0f;
                            const uint32_t j = row0 + lane, i = tok0 + col;
                            if (j < n && i < m) {
                                for (uint32_t c = s0 * kSegK; c < s1 * kSegK; ++c) {
                                    sum += x[(size_t)i * k + c] * w[(size_t)j * k + c];
                                }
                            }
                            acc[(size_t)lane * NTOK + col] = sum;
                        }
                    }
                    emu::accumulator = acc.data();
                    emu::accumulator_columns = NTOK;
                    epilogue_piece<NTOK, float>(args, 0u, t / 32u, t % 32u, tile_place<NTOK>(args, tile, tok_tiles, m), tile, s0, s1, segs, tok_tiles, units,
                                                blocks, m, &abort_flag, 0u);
                    u += (s1 - s0);
                }
            });
        }
    }
    for (std::thread &thread : threads) {
        thread.join();
    }
    *status_out = status;
    for (unsigned int flag : flags) {
        if (flag != 0u) {
            *status_out |= 0x100u; // a flag was left raised: the next launch would misread it
        }
    }
}

extern "C" unsigned int epilogue_emu(const float *w, uint32_t n, uint32_t k, const float *x, uint32_t m, float *y,
                                     uint32_t ldy, uint32_t mode, const unsigned int *row_map, uint32_t group,
                                     uint32_t grid, uint32_t ntok)
{
    unsigned int status = 0xFFFFu;
    if (ntok == 16u) {
        run_launch<16>(w, n, k, x, m, y, ldy, mode, row_map, group, grid, &status);
    } else if (ntok == 32u) {
        run_launch<32>(w, n, k, x, m, y, ldy, mode, row_map, group, grid, &status);
    } else if (ntok == 64u) {
        run_launch<64>(w, n, k, x, m, y, ldy, mode, row_map, group, grid, &status);
    }
    return status;
}
