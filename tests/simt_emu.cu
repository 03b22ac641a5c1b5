// A small host emulator for the kernels that run on the ordinary cores (no tensor memory, no
// bulk copies): the kernel source is compiled as host code, a block runs as blockDim.x host
// threads, and __shfl_*_sync / __syncwarp / __syncthreads are barriers between them, so the
// kernels execute with the warp semantics they rely on.  It lets the tests run, without a GPU,
//   q_dequant_any_kernel, q_gemv_any_kernel            (aotx_b200/csrc/q_generic.cu)
//   q8_gemv_simt_kernel, q8_gemv_simt_fused_kernel     (aotx_b200/csrc/q8_simt_gemv.cuh)
//   q8_dequant_kernel, q8_route_kernel, q8_expert_feed_kernel, q8_expert_down_kernel,
//   q8_expert_sum_kernel                               (aotx_b200/csrc/q8_simt.cu)
// on small shapes and compare them with the oracle.  It checks the kernels' index arithmetic and
// data flow; it says nothing about the hardware.
//
// Built as a shared library by tests/test_simt_emu.py (nvcc, host code only).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

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

struct Block {
    std::vector<Warp> warps;
    Barrier *all;
};

thread_local Index thread_index = {0, 0, 0};
thread_local Index block_index = {0, 0, 0};
thread_local Block *block = nullptr;
Index block_dim = {1, 1, 1};
Index grid_dim = {1, 1, 1};

// every lane of the warp calls these together (full mask), as the kernels under test do
inline uint32_t exchange(uint32_t value, unsigned int from_lane_of_mine(unsigned int))
{
    Warp &warp = block->warps[thread_index.x / 32u];
    const unsigned int lane = thread_index.x % 32u;
    warp.slot[lane] = value;
    warp.barrier.wait();
    const unsigned int source = from_lane_of_mine(lane);
    const uint32_t got = source < 32u ? warp.slot[source] : value;
    warp.barrier.wait();
    return got;
}

thread_local unsigned int shift = 0;

inline float shfl_down(float value, unsigned int delta)
{
    shift = delta;
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    bits = exchange(bits, [](unsigned int lane) { return lane + shift; });
    std::memcpy(&value, &bits, 4);
    return value;
}

inline float shfl_xor(float value, unsigned int mask)
{
    shift = mask;
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    bits = exchange(bits, [](unsigned int lane) { return lane ^ shift; });
    std::memcpy(&value, &bits, 4);
    return value;
}

inline void sync_warp()
{
    block->warps[thread_index.x / 32u].barrier.wait();
}

inline void sync_block()
{
    block->all->wait();
}

inline float uint_as_float(uint32_t bits)
{
    float value;
    std::memcpy(&value, &bits, 4);
    return value;
}

// one rounding each, never contracted into a fused multiply-add
inline float fmul_rn(float a, float b)
{
    volatile float product = a * b;
    return product;
}

inline float fadd_rn(float a, float b)
{
    volatile float sum = a + b;
    return sum;
}

// Run `body` as a grid of `grid` blocks of `threads` threads (a multiple of 32), block by block.
inline void launch(unsigned int grid, unsigned int threads, const std::function<void()> &body)
{
    block_dim = {threads, 1, 1};
    grid_dim = {grid, 1, 1};
    for (unsigned int b = 0; b < grid; ++b) {
        Block shared;
        shared.warps = std::vector<Warp>(threads / 32u);
        Barrier all(threads);
        shared.all = &all;
        std::vector<std::thread> lanes;
        lanes.reserve(threads);
        for (unsigned int t = 0; t < threads; ++t) {
            lanes.emplace_back([&, t, b] {
                thread_index = {t, 0, 0};
                block_index = {b, 0, 0};
                block = &shared;
                body();
            });
        }
        for (std::thread &lane : lanes) {
            lane.join();
        }
    }
}

// the same with a grid of grid.x * grid.y blocks
inline void launch2(Index grid, unsigned int threads, const std::function<void()> &body)
{
    block_dim = {threads, 1, 1};
    grid_dim = grid;
    for (unsigned int by = 0; by < grid.y; ++by) {
        for (unsigned int bx = 0; bx < grid.x; ++bx) {
            Block shared;
            shared.warps = std::vector<Warp>(threads / 32u);
            Barrier all(threads);
            shared.all = &all;
            std::vector<std::thread> lanes;
            lanes.reserve(threads);
            for (unsigned int t = 0; t < threads; ++t) {
                lanes.emplace_back([&, t, bx, by] {
                    thread_index = {t, 0, 0};
                    block_index = {bx, by, 0};
                    block = &shared;
                    body();
                });
            }
            for (std::thread &lane : lanes) {
                lane.join();
            }
        }
    }
}

} // namespace emu

// ---- the kernel sources as host code --------------------------------------------------------
#undef __global__
#define __global__
#undef __grid_constant__
#define __grid_constant__
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
#define blockDim (emu::block_dim)
#define gridDim (emu::grid_dim)
#define __shfl_down_sync(mask, value, delta) emu::shfl_down((value), (delta))
#define __shfl_xor_sync(mask, value, lanes) emu::shfl_xor((value), (lanes))
#define __syncwarp() emu::sync_warp()
#define __syncthreads() emu::sync_block()
#define __uint_as_float(bits) emu::uint_as_float(bits)
#define __int_as_float(bits) emu::uint_as_float((uint32_t)(bits))
#define __fmul_rn(a, b) emu::fmul_rn((a), (b))
#define __fadd_rn(a, b) emu::fadd_rn((a), (b))
#define clock64() 0ll                           /* only the tensor-core kernels wait; none runs here */
#define atomicOr(word, bits) (*(word) |= (bits))
#define Q8_HOST_EMULATION 1

// the stand-ins for the few PTX instructions these kernels reach (byte permute for the exact
// dequantisation); the rest of that header serves the tensor-core kernels' emulation
#include "q8_ptx_emu.cuh"

namespace q8 {
alignas(1024) unsigned char smem_raw_[kEmuSharedBytes];
static float emulated_dynamic_shared[4 * 16384]; // the router kernel's dynamic shared memory
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

// static shared arrays: one block runs at a time, so one static copy stands for the block's
#undef __shared__
#define __shared__ static
#include "q8_simt.cu"
#include "q_generic.cu"

// what the library's own launch code runs a grid through in this build (q8_launch.h)
namespace q8 {
void emulate_grid(dim3 grid, unsigned int threads, const std::function<void()> &block_body)
{
    emu::launch2({grid.x, grid.y, 1}, threads, block_body);
}
} // namespace q8

// ---- entry points for the tests -------------------------------------------------------------
extern "C" void emu_dequant_any(const unsigned char *w, uint32_t type, uint32_t k, uint32_t first_row, uint32_t rows,
                                unsigned short *out, uint32_t grid)
{
    emu::launch(grid, 256, [=] {
        q8::q_dequant_any_kernel(w, type, k, first_row, rows, reinterpret_cast<__half *>(out));
    });
}

// x and y: binary16 in, float out (the reference's types)
extern "C" void emu_gemv_any(const unsigned char *w, uint32_t type, uint32_t n, uint32_t k, const unsigned short *x,
                             uint32_t m, const unsigned int *m_dev, float *y, uint32_t wide_x, uint32_t grid)
{
    emu::launch(grid, QG_WARPS * 32u, [=] {
        q8::q_gemv_any_kernel<__half, float>(w, type, n, k, reinterpret_cast<const __half *>(x), m, m_dev, y,
                                             wide_x);
    });
}

// bfloat16 activations, bfloat16 results
extern "C" void emu_gemv_any_bf16(const unsigned char *w, uint32_t type, uint32_t n, uint32_t k,
                                  const unsigned short *x, uint32_t m, unsigned short *y, uint32_t wide_x,
                                  uint32_t grid)
{
    emu::launch(grid, QG_WARPS * 32u, [=] {
        q8::q_gemv_any_kernel<__nv_bfloat16, __nv_bfloat16>(w, type, n, k, reinterpret_cast<const __nv_bfloat16 *>(x),
                                                            m, nullptr, reinterpret_cast<__nv_bfloat16 *>(y), wide_x);
    });
}

extern "C" void emu_gemv_q8(const unsigned char *w, uint32_t n, uint32_t k, const unsigned short *x, uint32_t m,
                            const unsigned int *m_dev, float *y, uint32_t grid)
{
    emu::launch(grid, Q8_SIMT_WARPS * 32u, [=] {
        q8::q8_gemv_simt_kernel<__half, float>(w, n, k, reinterpret_cast<const __half *>(x), m, m_dev, y);
    });
}

// epilogue 1: y float, added to; epilogue 2: y binary16 [m][n / 2]
extern "C" void emu_gemv_q8_fused(const unsigned char *w, uint32_t n, uint32_t k, const unsigned short *x, uint32_t m,
                                  const unsigned int *m_dev, void *y, uint32_t epilogue, uint32_t grid)
{
    if (epilogue == 1u) {
        emu::launch(grid, Q8_SIMT_WARPS * 32u, [=] {
            q8::q8_gemv_simt_fused_kernel<__half, float>(w, n, k, reinterpret_cast<const __half *>(x), m, m_dev,
                                                         static_cast<float *>(y), epilogue);
        });
    } else {
        emu::launch(grid, Q8_SIMT_WARPS * 32u, [=] {
            q8::q8_gemv_simt_fused_kernel<__half, __half>(w, n, k, reinterpret_cast<const __half *>(x), m, m_dev,
                                                          static_cast<__half *>(y), epilogue);
        });
    }
}

extern "C" void emu_dequant_q8(const unsigned char *w, unsigned long long blocks, unsigned short *out, int wide,
                               uint32_t grid)
{
    emu::launch(grid, 256, [=] { q8::q8_dequant_kernel(w, blocks, reinterpret_cast<__half *>(out), wide); });
}

extern "C" void emu_route(const unsigned short *x, const float *router, uint32_t tokens, const unsigned int *tokens_dev,
                          uint32_t hidden, uint32_t experts, uint32_t used, float *prob, unsigned int *ids,
                          uint32_t grid)
{
    emu::launch(grid, Q8_ROUTE_THREADS, [=] {
        q8::q8_route_kernel(reinterpret_cast<const __half *>(x), router, tokens, tokens_dev, hidden, experts, used,
                            prob, ids);
    });
}

// the per-pair expert products: act binary16 [tokens * used][ffn], proj float [tokens * used][hidden]
extern "C" void emu_expert_pairs(const unsigned char *w_gate, const unsigned char *w_up, const unsigned char *w_down,
                                 uint32_t hidden, uint32_t ffn, const unsigned short *x, const unsigned int *ids,
                                 uint32_t experts, uint32_t tokens, const unsigned int *tokens_dev, uint32_t used,
                                 unsigned short *act, float *proj, uint32_t pair_blocks)
{
    emu::Index feed = {(ffn + Q8_SIMT_WARPS - 1u) / Q8_SIMT_WARPS, pair_blocks, 1};
    emu::Index down = {(hidden + Q8_SIMT_WARPS - 1u) / Q8_SIMT_WARPS, pair_blocks, 1};
    emu::launch2(feed, Q8_SIMT_WARPS * 32u, [=] {
        q8::q8_expert_feed_kernel(w_gate, w_up, hidden, ffn, reinterpret_cast<const __half *>(x), ids, experts, tokens,
                                  tokens_dev, used, reinterpret_cast<__half *>(act));
    });
    emu::launch2(down, Q8_SIMT_WARPS * 32u, [=] {
        q8::q8_expert_down_kernel(w_down, hidden, ffn, reinterpret_cast<const __half *>(act), ids, experts, tokens,
                                  tokens_dev, used, proj);
    });
}

// width 4: 16-byte loads of proj; width 1: any hidden, any alignment
extern "C" void emu_expert_sum(const float *proj, const float *prob, const unsigned int *ids, uint32_t tokens,
                               const unsigned int *tokens_dev, uint32_t hidden, uint32_t experts, uint32_t used,
                               float *out, uint32_t width, uint32_t grid)
{
    q8::ProjParts from = {};
    from.base[0] = proj;
    from.parts = 1u;
    if (width == 4u) {
        emu::launch(grid, 256, [=] {
            q8::q8_expert_sum_kernel<float, 4u>(from, prob, ids, tokens, tokens_dev, hidden, experts, used, out);
        });
    } else {
        emu::launch(grid, 256, [=] {
            q8::q8_expert_sum_kernel<float, 1u>(from, prob, ids, tokens, tokens_dev, hidden, experts, used, out);
        });
    }
}
