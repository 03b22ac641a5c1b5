// The decode-regime tensor-core kernel (q8_stream_kernel, aotx_b200/csrc/q8_stream.cu) run on the
// host, whole: its source is compiled as host code with the stand-ins of tests/q8_ptx_emu.cuh in
// place of the inline PTX, a block runs as its 480 threads, and blocks run one after the other
// from the last to the first (the owner of a cut tile waits only for blocks after it, so that
// order never blocks).  The driver builds the kernel's arguments and the two tensor maps as the
// host launch code does and hands back y.  What this checks is the kernel's own logic - the
// roles of the warps and their rings, the byte arithmetic of the dequantisation, the layouts in
// shared and tensor memory, the unit schedule, the stores - against the oracle, on a machine
// without a GPU.  What the hardware really does with the instructions is the GPU tests' matter.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
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
Barrier *block_barrier = nullptr;
Index grid_dim = {1, 1, 1};
Index block_dim = {1, 1, 1};
unsigned int max_delay_us = 0;

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

// __all_sync over the whole warp: true when every lane's predicate is
inline int vote_all(int predicate)
{
    const unsigned int lane = thread_index.x % 32u;
    warp->slot[lane] = predicate ? 1u : 0u;
    warp->barrier.wait();
    int all = 1;
    for (unsigned int i = 0; i < 32u; ++i) {
        all &= warp->slot[i] != 0u;
    }
    warp->barrier.wait();
    return all;
}

// __match_any_sync over the whole warp: the lanes whose value equals this lane's
inline unsigned int match_any(unsigned int value)
{
    const unsigned int lane = thread_index.x % 32u;
    warp->slot[lane] = value;
    warp->barrier.wait();
    unsigned int same = 0u;
    for (unsigned int i = 0; i < 32u; ++i) {
        same |= (warp->slot[i] == value ? 1u : 0u) << i;
    }
    warp->barrier.wait();
    return same;
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

long long cycles_per_us = 400;

// The kernels bound their waits by the SM clock (about two seconds' worth of cycles); here the
// same bound runs out after about ten seconds (cycles_per_us = 400), so that a kernel that has stopped making progress
// ends with its status bits raised, as on the hardware, instead of holding the test.
inline long long clock_now()
{
    const auto now = std::chrono::steady_clock::now().time_since_epoch();
    return (long long)std::chrono::duration_cast<std::chrono::nanoseconds>(now).count() / 1000ll * cycles_per_us;
}

inline unsigned int atomic_add(unsigned int *word, unsigned int value)
{
    return reinterpret_cast<std::atomic<unsigned int> *>(word)->fetch_add(value);
}

inline unsigned int atomic_or(unsigned int *word, unsigned int bits)
{
    return reinterpret_cast<std::atomic<unsigned int> *>(word)->fetch_or(bits);
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
#undef __grid_constant__
#define __grid_constant__
#undef __shared__
#define __shared__
#define threadIdx (emu::thread_index)
#define blockIdx (emu::block_index)
#define gridDim (emu::grid_dim)
#define __shfl_xor_sync(mask, value, lanes) emu::shfl_xor((value), (lanes))
#define __syncwarp() emu::warp->barrier.wait()
#define __all_sync(mask, predicate) emu::vote_all(predicate)
#define __any_sync(mask, predicate) (!emu::vote_all(!(predicate)))
#define __match_any_sync(mask, value) emu::match_any(value)
#define __popc(bits) __builtin_popcount(bits)
#define __syncthreads() emu::block_barrier->wait()
#define __uint_as_float(bits) emu::uint_as_float(bits)
#define __float_as_uint(value) emu::float_as_uint(value)
#define clock64() emu::clock_now()
#define atomicOr(word, bits) emu::atomic_or((word), (bits))
#define __ldcg(p) (*(p))
#define __ldg(p) (*(p))
#define __stcg(p, v) (*(p) = (v))
#define __threadfence() std::atomic_thread_fence(std::memory_order_seq_cst)
#define __threadfence_system() std::atomic_thread_fence(std::memory_order_seq_cst)
#define blockDim (emu::block_dim)
#define atomicAdd(word, value) emu::atomic_add((word), (value))
#define Q8_HOST_EMULATION 1

#include "q8_ptx_emu.cuh"

namespace q8 {
alignas(1024) unsigned char smem_raw_[kEmuSharedBytes];
} // namespace q8

namespace q8emu {
inline unsigned int lane_of_thread()
{
    return emu::thread_index.x % 32u;
}

inline unsigned int warp_of_thread()
{
    return emu::thread_index.x / 32u;
}
} // namespace q8emu

#include "q8_stream.cu"
#include "q8_dispatch.cu"
#include "q8_wide.cu"
#include "q8_decode.cu"

// the routed-expert kernels keep their tables in static shared memory: one block runs at a time,
// so one static copy stands for it
#undef __shared__
#define __shared__ static
#include "q8_moe.cu"

using namespace q8;

// Run `body` as a grid of blocks of `threads` threads, one block at a time, the last block first
// (the owner of a cut tile waits only for blocks after its own, so that order never blocks).
template <typename Body>
static unsigned int run_grid(unsigned int grid, unsigned int threads, Body body, unsigned int grid_x = 0)
{
    unsigned int status = 0;
    grid_x = grid_x == 0u ? grid : grid_x;          // a two-dimensional grid: grid_x blocks per row
    emu::grid_dim = {grid_x, grid / grid_x, 1};
    emu::block_dim = {threads, 1, 1};
    for (unsigned int b = grid; b-- > 0u;) {
        std::memset(q8emu::tensor_memory, 0xEE, sizeof q8emu::tensor_memory);
        std::memset(q8::smem_raw_, 0xDD, q8::kEmuSharedBytes);
        q8emu::barriers.clear();
        emu::Barrier all(threads);
        emu::block_barrier = &all;
        std::vector<emu::Warp> warps(threads / 32u);
        if (q8emu::asynchronous) {
            q8emu::copy_engine.start(17u * b + 1u, emu::max_delay_us);
            q8emu::tensor_pipe.start(31u * b + 2u, emu::max_delay_us);
        }
        std::vector<std::thread> lanes;
        lanes.reserve(threads);
        for (unsigned int t = 0; t < threads; ++t) {
            lanes.emplace_back([&, t, b] {
                emu::thread_index = {t, 0, 0};
                emu::block_index = {b % grid_x, b / grid_x, 0};
                emu::warp = &warps[t / 32u];
                body();
            });
        }
        for (std::thread &lane : lanes) {
            lane.join();
        }
        if (q8emu::asynchronous && q8emu::copy_engine.finish() + q8emu::tensor_pipe.finish() != 0u) {
            status |= 0x200u; // the block ended with a copy or tensor-core work in flight
        }
        if (q8emu::tmem_held.exchange(0u) != 0u) {
            status |= 0x400u; // the block ended holding tensor memory
        }
        if (q8emu::lane_violations.exchange(0u) != 0u) {
            // a use the hardware does not define; which kinds, in bits 16 and up
            status |= 0x800u | (q8emu::violation_kinds.exchange(0u) << 16);
        }
    }
    return status;
}

// What the library's own launch code runs a grid through in this build (q8_launch.h).  Status
// bits of the runs since the last entry point was called collect in `emulated_status`.
static unsigned int emulated_status = 0;

namespace q8 {
void emulate_grid(dim3 grid, unsigned int threads, const std::function<void()> &block_body)
{
    emulated_status |= run_grid(grid.x * grid.y, threads, block_body, grid.x);
}
} // namespace q8

// The two tensor maps as the host launch code encodes them (launch_umma, launch_umma_grouped).
static void make_maps(const unsigned char *w, uint32_t w_rows, uint32_t k, const void *x, uint32_t x_rows,
                      uint32_t x_box_rows, CUtensorMap *tw, CUtensorMap *tx)
{
    static_assert(sizeof(q8emu::TensorMap) <= sizeof(CUtensorMap), "the stand-in fits the real type");
    const uint64_t row_b = (uint64_t)(k / 32u) * 34u;
    q8emu::TensorMap map_w = {w, {row_b / 4u, w_rows}, row_b, {kSegWords, kRows}, 4u, 0u};
    q8emu::TensorMap map_x = {static_cast<const unsigned char *>(x), {k, x_rows}, (uint64_t)k * 2u, {kSubK, x_box_rows}, 2u, 1u};
    std::memset(tw, 0, sizeof *tw);
    std::memset(tx, 0, sizeof *tx);
    std::memcpy(tw, &map_w, sizeof map_w);
    std::memcpy(tx, &map_x, sizeof map_x);
}

// which decode-regime kernel the launches that follow run: 0 the one-block-per-SM kernel
// (q8_stream.cu), 1 the two-blocks-per-SM kernel (q8_decode.cu; token tiles of 16 and 32, one
// token tile, unit schedule - a cluster launch is not modelled)
static unsigned int decode_form = 0;

extern "C" void stream_emu_form(unsigned int form)
{
    decode_form = form;
}

// column-split mode for the launches that follow (UmmaArgs::peers, y_peer, col0): the product's
// n columns are columns [col0, col0 + n) of `count` buffers that are ldy wide; count 0: off
static void *peer_buffer[8];
static unsigned int peer_count = 0, peer_col0 = 0;

extern "C" void stream_emu_peers(unsigned int count, void *const *buffers, unsigned int col0)
{
    peer_count = count;
    peer_col0 = col0;
    for (unsigned int i = 0; i < 8u; ++i) {
        peer_buffer[i] = i < count ? buffers[i] : nullptr;
    }
}

// One launch of the kernel with scratch slots and flags of its own.
template <int NTOK, typename YT>
static unsigned int run_stream(const CUtensorMap &tw, const CUtensorMap &tx, UmmaArgs args, unsigned int grid)
{
    std::vector<float> partial((size_t)grid * kRows * NTOK, 0.0f);
    std::vector<unsigned int> flags((size_t)grid * 4u, 0u);
    unsigned int status = 0;
    args.partial = partial.data();
    args.flags = flags.data();
    args.status = &status;
    args.tile_floats = (unsigned long long)kRows * NTOK;
    unsigned int ended = 0xFFFFu;
    if (decode_form == 0u) {
        ended = run_grid(grid, kThreads, [&] { q8_stream_kernel<NTOK, YT>(tw, tx, args); });
    } else if constexpr (NTOK <= 32) {
        args.split = 0u;
        ended = run_grid(grid, kDecThreads, [&] { q8_decode_kernel<NTOK, YT>(tw, tx, args); });
    }
    status |= ended;
    for (unsigned int flag : flags) {
        if (flag != 0u) {
            status |= 0x100u; // a flag left raised would be misread by the next launch
        }
    }
    return status;
}

template <typename YT>
static unsigned int run_stream_tile(uint32_t ntok, const CUtensorMap &tw, const CUtensorMap &tx, const UmmaArgs &args,
                                    unsigned int grid)
{
    switch (ntok) {
    case 16: return run_stream<16, YT>(tw, tx, args, grid);
    case 32: return run_stream<32, YT>(tw, tx, args, grid);
    case 64: return run_stream<64, YT>(tw, tx, args, grid);
    case 128: return run_stream<128, YT>(tw, tx, args, grid);
    default: return 0xFFFFu;
    }
}

static void set_mode(int asynchronous, uint32_t max_delay_us)
{
    q8emu::asynchronous = asynchronous != 0;
    emu::max_delay_us = max_delay_us;
    q8emu::copies_issued = 0;
}

// One product, arguments as launch_umma fills them.  x: binary16 or bfloat16 [m][k]; y: float
// [m][ldy] (epilogue 0, 1) or [m][n / 2] (epilogue 2).
extern "C" unsigned int stream_emu(const unsigned char *w, uint32_t n, uint32_t k, const void *x, int x_bf16,
                                   uint32_t m, const unsigned int *m_dev, float *y, uint32_t ldy, uint32_t epilogue,
                                   uint32_t grid, uint32_t ntok, int asynchronous, uint32_t max_delay_us)
{
    set_mode(asynchronous, max_delay_us);
    CUtensorMap tw, tx;
    make_maps(w, n, k, x, m, ntok, &tw, &tx);
    const unsigned long long units = (unsigned long long)((n + kRows - 1u) / kRows) * ((m + ntok - 1u) / ntok) * (k / kSegK);
    if (units < grid) {
        grid = (unsigned int)units;
    }
    UmmaArgs args;
    std::memset(&args, 0, sizeof args);
    args.n = n;
    args.k = k;
    args.m_max = m;
    args.m_dev = m_dev;
    args.y = y;
    args.b_bf16 = x_bf16 ? 1u : 0u;
    args.ldy = ldy;
    args.epilogue = epilogue;
    args.peers = peer_count;
    args.col0 = peer_col0;
    for (unsigned int i = 0; i < 8u; ++i) {
        args.y_peer[i] = peer_buffer[i];
    }
    return run_stream_tile<float>(ntok, tw, tx, args, grid);
}

// One product on the prefill-regime kernel (q8_wide.cu: token tiles of 256, whole waves of tiles
// dealt round-robin and the last partial wave cut into units), arguments as launch_umma fills
// them for it.  y: float [m][n].
template <int NTOK, typename Kernel>
static unsigned int run_prefill(Kernel kernel, const CUtensorMap &tw, const CUtensorMap &tx, UmmaArgs args,
                                unsigned int grid)
{
    std::vector<float> partial((size_t)grid * kRows * NTOK, 0.0f);
    std::vector<unsigned int> flags((size_t)grid * 4u, 0u);
    unsigned int status = 0;
    args.partial = partial.data();
    args.flags = flags.data();
    args.status = &status;
    args.tile_floats = (unsigned long long)kRows * NTOK;
    status |= run_grid(grid, kThreads, [&] { kernel(tw, tx, args); });
    for (unsigned int flag : flags) {
        if (flag != 0u) {
            status |= 0x100u;
        }
    }
    return status;
}

extern "C" unsigned int wide_emu(const unsigned char *w, uint32_t n, uint32_t k, const void *x, int x_bf16,
                                 uint32_t m, const unsigned int *m_dev, float *y, uint32_t epilogue, uint32_t grid,
                                 int asynchronous, uint32_t max_delay_us)
{
    const uint32_t ntok = 256u;
    set_mode(asynchronous, max_delay_us);
    CUtensorMap tw, tx;
    make_maps(w, n, k, x, m, ntok, &tw, &tx);
    const unsigned long long units = (unsigned long long)((n + kRows - 1u) / kRows) * ((m + ntok - 1u) / ntok) * (k / kSegK);
    if (units < grid) {
        grid = (unsigned int)units;
    }
    UmmaArgs args;
    std::memset(&args, 0, sizeof args);
    args.n = n;
    args.k = k;
    args.m_max = m;
    args.m_dev = m_dev;
    args.y = y;
    args.b_bf16 = x_bf16 ? 1u : 0u;
    args.ldy = epilogue == kEpilogueSwiglu ? n / 2u : n;
    args.epilogue = epilogue;
    return run_prefill<256>(q8_wide_kernel<float>, tw, tx, args, grid);
}

// Grouped mode, arguments as launch_umma_grouped fills them.
template <typename YT>
static unsigned int run_grouped(const unsigned char *w_stacked, uint32_t total_rows, uint32_t k, const void *x_sorted,
                                uint32_t x_rows, uint32_t ntok, const GroupTile *tiles, const unsigned int *count,
                                uint32_t max_tiles, const unsigned int *row_map, void *y, uint32_t ldy,
                                uint32_t epilogue, uint32_t grid)
{
    if (max_tiles == 0u || x_rows == 0u) {
        return 0u;
    }
    CUtensorMap tw, tx;
    make_maps(w_stacked, total_rows, k, x_sorted, x_rows, ntok, &tw, &tx);
    const unsigned long long units = (unsigned long long)max_tiles * (k / kSegK);
    if (units < grid) {
        grid = (unsigned int)units;
    }
    UmmaArgs args;
    std::memset(&args, 0, sizeof args);
    args.n = total_rows;
    args.k = k;
    args.m_max = x_rows;
    args.y = y;
    args.group_tiles = tiles;
    args.group_count = count;
    args.row_map = row_map;
    args.ldy = ldy;
    args.epilogue = epilogue;
    return run_stream_tile<YT>(ntok, tw, tx, args, grid);
}

// The routed-expert step as launch_moe_grouped (w_gate_up null) and launch_moe_grouped_fused
// (w_gate_up set: gate and up rows interleaved) run it: table build, row gather, grouped products,
// the gated unit.  x: binary16 [tokens][hidden]; ids [tokens][used].  Out: proj float
// [tokens * used][hidden] (row = token * used + rank), act binary16 [tokens * used][ffn] in the
// sorted order, sorted_pair [tokens * used].
extern "C" unsigned int stream_emu_moe(const unsigned char *w_gate, const unsigned char *w_up,
                                       const unsigned char *w_gate_up, const unsigned char *w_down, uint32_t experts,
                                       uint32_t hidden, uint32_t ffn, const void *x, const unsigned int *ids,
                                       uint32_t tokens, const unsigned int *tokens_dev, uint32_t used,
                                       uint32_t tile_tokens, uint32_t grid, float *proj, unsigned short *act,
                                       unsigned int *sorted_pair, int asynchronous, uint32_t max_delay_us)
{
    set_mode(asynchronous, max_delay_us);
    const bool fused = w_gate_up != nullptr;
    const uint32_t pairs = tokens * used;
    const MoeWorkspace ws = moe_workspace_layout(tokens, used, hidden, ffn, experts);
    std::vector<GroupTile> tiles_feed(ws.max_feed), tiles_down(ws.max_down);
    std::vector<unsigned short> x_sorted((size_t)pairs * hidden, 0);
    unsigned int counts[2] = {0u, 0u};
    unsigned int status = 0;
    status |= run_grid(1u, Q8_GROUP_THREADS, [&] {
        q8_group_build_kernel(ids, tokens, tokens_dev, used, experts, fused ? 2u * ffn : ffn, hidden, sorted_pair,
                              tiles_feed.data(), tiles_down.data(), counts, tile_tokens);
    });
    RowParts rows = {};
    rows.base[0] = x;
    rows.parts = 1u;
    status |= run_grid(pairs < 3u ? pairs : 3u, 128u, [&] {
        q8_gather_rows_kernel(rows, sorted_pair, tokens, tokens_dev, used, hidden / 8u,
                              reinterpret_cast<uint4 *>(x_sorted.data()));
    });
    if (fused) {
        status |= run_grouped<__half>(w_gate_up, experts * 2u * ffn, hidden, x_sorted.data(), pairs, tile_tokens,
                                      tiles_feed.data(), counts + 0, ws.max_feed, nullptr, act, ffn, kEpilogueSwiglu,
                                      grid);
    } else {
        std::vector<float> gate((size_t)pairs * ffn, 0.0f), up((size_t)pairs * ffn, 0.0f);
        status |= run_grouped<float>(w_gate, experts * ffn, hidden, x_sorted.data(), pairs, tile_tokens,
                                     tiles_feed.data(), counts + 0, ws.max_feed, nullptr, gate.data(), ffn, 0u, grid);
        status |= run_grouped<float>(w_up, experts * ffn, hidden, x_sorted.data(), pairs, tile_tokens,
                                     tiles_feed.data(), counts + 0, ws.max_feed, nullptr, up.data(), ffn, 0u, grid);
        status |= run_grid(2u, 256u, [&] {
            q8_swiglu_kernel(gate.data(), up.data(), tokens, tokens_dev, used, ffn, reinterpret_cast<__half *>(act));
        });
    }
    status |= run_grouped<float>(w_down, experts * hidden, ffn, act, pairs, tile_tokens, tiles_down.data(),
                                 counts + 1, ws.max_down, sorted_pair, proj, hidden, 0u, grid);
    return status;
}

// The table build alone: sorted pairs, the two tile tables (five words per entry) and their
// entry counts.
extern "C" void stream_emu_group_build(const unsigned int *ids, uint32_t tokens, const unsigned int *tokens_dev,
                                       uint32_t used, uint32_t experts, uint32_t ffn, uint32_t hidden,
                                       uint32_t tile_tokens, unsigned int *sorted_pair, unsigned int *tiles_feed,
                                       unsigned int *tiles_down, unsigned int *counts)
{
    set_mode(0, 0);
    run_grid(1u, Q8_GROUP_THREADS, [&] {
        q8_group_build_kernel(ids, tokens, tokens_dev, used, experts, ffn, hidden, sorted_pair,
                              reinterpret_cast<GroupTile *>(tiles_feed), reinterpret_cast<GroupTile *>(tiles_down),
                              counts, tile_tokens);
    });
}

// Bulk tensor copies issued since the last entry point was called.
extern "C" long long stream_emu_copies()
{
    return q8emu::copies_issued.load();
}

// Fault injection for the bounded waits: copy number `lost_copy` of the next launches never lands
// (-1: none), and the wait bound is `seconds` long.
extern "C" void stream_emu_faults(long long lost_copy, double seconds)
{
    q8emu::lost_copy = lost_copy;
    emu::cycles_per_us = (long long)(4000.0 / seconds);
}
