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
#define __syncthreads() emu::block_barrier->wait()
#define __uint_as_float(bits) emu::uint_as_float(bits)
#define __float_as_uint(value) emu::float_as_uint(value)
#define clock64() emu::clock_now()
#define atomicOr(word, bits) emu::atomic_or((word), (bits))
#define __ldcg(p) (*(p))
#define __stcg(p, v) (*(p) = (v))
#define __threadfence() std::atomic_thread_fence(std::memory_order_seq_cst)
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
} // namespace q8emu

#include "q8_stream.cu"

using namespace q8;

// the product that follows on the stream, whose first units each block asks the L2 for
struct Next {
    const unsigned char *w;
    uint32_t n, k, m, units_per_block;
};

template <int NTOK, typename YT>
static unsigned int run(const unsigned char *w, uint32_t n, uint32_t k, const void *x, int x_bf16, uint32_t m,
                        const unsigned int *m_dev, void *y, uint32_t ldy, uint32_t epilogue, uint32_t grid,
                        const Next &next)
{
    static_assert(sizeof(q8emu::TensorMap) <= sizeof(CUtensorMap), "the stand-in fits the real type");
    CUtensorMap tw, tx;
    q8emu::TensorMap map_w = {w, {(uint64_t)(k / 32u) * 34u / 4u, n}, (uint64_t)(k / 32u) * 34u, {kSegWords, kRows}, 4u, 0u};
    q8emu::TensorMap map_x = {static_cast<const unsigned char *>(x), {k, m}, (uint64_t)k * 2u, {kSubK, (uint32_t)NTOK}, 2u, 1u};
    std::memcpy(&tw, &map_w, sizeof map_w);
    std::memcpy(&tx, &map_x, sizeof map_x);

    const unsigned long long units = (unsigned long long)((n + kRows - 1u) / kRows) * ((m + NTOK - 1u) / NTOK) * (k / kSegK);
    if (units < grid) {
        grid = (unsigned int)units;
    }
    std::vector<float> partial((size_t)grid * kRows * NTOK, 0.0f);
    std::vector<unsigned int> flags((size_t)grid * 4u, 0u);
    unsigned int status = 0;
    UmmaArgs args;
    std::memset(&args, 0, sizeof args);
    args.n = n;
    args.k = k;
    args.m_max = m;
    args.m_dev = m_dev;
    args.y = y;
    args.partial = partial.data();
    args.flags = flags.data();
    args.status = &status;
    args.tile_floats = (unsigned long long)kRows * NTOK;
    args.b_bf16 = x_bf16 ? 1u : 0u;
    args.ldy = ldy;
    args.epilogue = epilogue;
    if (next.w != nullptr) {
        args.next_w = next.w;
        args.next_stride = (unsigned long long)(next.k / 32u) * 34u;
        args.next_n = next.n;
        args.next_segs = next.k / kSegK;
        args.next_tok_tiles = (next.m + NTOK - 1u) / NTOK;
        args.next_units = next.units_per_block;
    }
    emu::grid_dim = {grid, 1, 1};

    for (unsigned int b = grid; b-- > 0u;) {
        std::memset(q8emu::tensor_memory, 0xEE, sizeof q8emu::tensor_memory);
        std::memset(q8::smem_raw_, 0xDD, q8::kEmuSharedBytes);
        q8emu::barriers.clear();
        emu::Barrier all(kThreads);
        emu::block_barrier = &all;
        std::vector<emu::Warp> warps(kThreads / 32u);
        if (q8emu::asynchronous) {
            q8emu::copy_engine.start(17u * b + 1u, emu::max_delay_us);
            q8emu::tensor_pipe.start(31u * b + 2u, emu::max_delay_us);
        }
        std::vector<std::thread> threads;
        threads.reserve(kThreads);
        for (unsigned int t = 0; t < kThreads; ++t) {
            threads.emplace_back([&, t, b] {
                emu::thread_index = {t, 0, 0};
                emu::block_index = {b, 0, 0};
                emu::warp = &warps[t / 32u];
                q8_stream_kernel<NTOK, YT>(tw, tx, args);
            });
        }
        for (std::thread &thread : threads) {
            thread.join();
        }
        if (q8emu::asynchronous && q8emu::copy_engine.finish() + q8emu::tensor_pipe.finish() != 0u) {
            status |= 0x200u; // the block ended with a copy or tensor-core work in flight
        }
        if (q8emu::tmem_held.exchange(0u) != 0u) {
            status |= 0x400u; // the block ended holding tensor memory
        }
    }
    for (unsigned int flag : flags) {
        if (flag != 0u) {
            status |= 0x100u; // a flag left raised would be misread by the next launch
        }
    }
    return status;
}

static unsigned int stream_emu_tile(const unsigned char *w, uint32_t n, uint32_t k, const void *x, int x_bf16,
                                    uint32_t m, const unsigned int *m_dev, float *y, uint32_t ldy, uint32_t epilogue,
                                    uint32_t grid, uint32_t ntok, const Next &next)
{
    switch (ntok) {
    case 16: return run<16, float>(w, n, k, x, x_bf16, m, m_dev, y, ldy, epilogue, grid, next);
    case 32: return run<32, float>(w, n, k, x, x_bf16, m, m_dev, y, ldy, epilogue, grid, next);
    case 64: return run<64, float>(w, n, k, x, x_bf16, m, m_dev, y, ldy, epilogue, grid, next);
    case 128: return run<128, float>(w, n, k, x, x_bf16, m, m_dev, y, ldy, epilogue, grid, next);
    default: return 0xFFFFu;
    }
}

// x: binary16 or bfloat16 [m][k]; y: float [m][ldy] (epilogue 0, 1) or [m][n / 2] (epilogue 2)
extern "C" unsigned int stream_emu(const unsigned char *w, uint32_t n, uint32_t k, const void *x, int x_bf16,
                                   uint32_t m, const unsigned int *m_dev, float *y, uint32_t ldy, uint32_t epilogue,
                                   uint32_t grid, uint32_t ntok, const unsigned char *next_w, uint32_t next_n,
                                   uint32_t next_k, uint32_t next_m, uint32_t next_units,
                                   unsigned long long *l2_bytes, int asynchronous, uint32_t max_delay_us)
{
    q8emu::asynchronous = asynchronous != 0;
    emu::max_delay_us = max_delay_us;
    q8emu::copies_issued = 0;
    const Next next = {next_w, next_n, next_k, next_m, next_units};
    q8::l2_requests = 0;
    const unsigned int status = stream_emu_tile(w, n, k, x, x_bf16, m, m_dev, y, ldy, epilogue, grid, ntok, next);
    if (l2_bytes != nullptr) {
        *l2_bytes = q8::l2_requests;
    }
    return status;
}

// Fault injection for the bounded waits: copy number `lost_copy` of the next launches never lands
// (-1: none), and the wait bound is `seconds` long.
extern "C" void stream_emu_faults(long long lost_copy, double seconds)
{
    q8emu::lost_copy = lost_copy;
    emu::cycles_per_us = (long long)(4000.0 / seconds);
}
