// Host stand-ins for the instructions of aotx_b200/csrc/q8_ptx.cuh, for the tests' emulation of
// the tensor-core kernels (-DQ8_HOST_EMULATION; tests/stream_emu.cu).  One block runs at a time,
// its threads are host threads; shared memory, tensor memory and the shared-memory barriers are
// plain host state:
//   shared memory   one byte array; a shared-space "address" is an offset into it (plus a base,
//                   so that 0 is never a valid address)
//   tensor memory   128 lanes x 512 columns of 32-bit words
//   mbarrier        arrivals, outstanding copy bytes and a phase count per barrier address
//   bulk tensor copy (TMA)  copies the box, then credits its bytes to the barrier
//   tcgen05.mma     in float, from tensor / shared memory
//   tcgen05.commit  an arrival after everything issued before it
// The copies and the tensor-core work run either at once in the calling thread or, in the
// asynchronous mode, later and in order on a thread of their own per engine (with a random delay
// before each operation), so that a kernel which reused a buffer before the operation reading or
// writing it had finished would compute wrong numbers here as it would on the hardware.
// The operand layouts follow what the kernels were written and verified against on the GPU:
// K-major rows of 128 bytes with the 128-byte swizzle for shared-memory operands, lane = row and
// two 16-bit values per column for a tensor-memory A operand, lane = row and one float per
// column for the accumulator.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <functional>
#include <map>
#include <mutex>
#include <random>
#include <thread>

namespace q8 {
// the kernels declare `extern __shared__ unsigned char smem_raw_[]`: this is that array, defined
// by the program that includes this header
constexpr unsigned int kEmuSharedBytes = 256u * 1024u + 1024u;
extern unsigned char smem_raw_[];
} // namespace q8

namespace q8emu {

constexpr uint32_t kSharedBase = 4096; // shared-space address of byte 0 of the block's shared memory
inline unsigned char *const shared_memory = q8::smem_raw_;
inline uint32_t tensor_memory[128][512];

struct MBarrier {
    uint32_t count = 0, pending = 0, phase = 0;
    int64_t tx = 0;
};

inline std::mutex barrier_mutex;
inline std::map<uint32_t, MBarrier> barriers;

inline unsigned char *shared_at(uint32_t addr)
{
    return shared_memory + (addr - kSharedBase);
}

inline void advance(MBarrier &bar)
{
    if (bar.pending == 0 && bar.tx == 0) {
        bar.phase += 1;
        bar.pending = bar.count;
    }
}

// What the emulated tensor map holds (the driver writes it into the 128 bytes of a CUtensorMap).
struct TensorMap {
    const unsigned char *base;
    uint64_t dims[2];      // elements: inner, outer
    uint64_t stride_bytes; // between outer indices
    uint32_t box[2];       // elements: inner, outer
    uint32_t elem_bytes;
    uint32_t swizzle128;   // rows of the box are 128 bytes and stored with the 128-byte swizzle
};

// cuTensorMapEncodeTiled for two dimensions: the description goes into the 128 bytes of the map.
// Refuses what the driver refuses: a base or a row stride off a 16-byte boundary, a box whose
// rows are not a multiple of 16 bytes, a box side above 256, rows of a swizzled box that are not
// 128 bytes.
inline CUresult encode_tiled(CUtensorMap *map, CUtensorMapDataType type, cuuint32_t rank, void *base,
                             const cuuint64_t *dims, const cuuint64_t *strides, const cuuint32_t *box,
                             const cuuint32_t *element_strides, CUtensorMapInterleave, CUtensorMapSwizzle swizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill)
{
    static_assert(sizeof(TensorMap) <= sizeof(CUtensorMap), "the stand-in fits the real type");
    uint32_t bytes = 0;
    if (type == CU_TENSOR_MAP_DATA_TYPE_UINT32) {
        bytes = 4;
    } else if (type == CU_TENSOR_MAP_DATA_TYPE_FLOAT16 || type == CU_TENSOR_MAP_DATA_TYPE_BFLOAT16) {
        bytes = 2;
    }
    const bool swizzled = swizzle == CU_TENSOR_MAP_SWIZZLE_128B;
    if (map == nullptr || rank != 2u || bytes == 0u || (reinterpret_cast<uintptr_t>(base) & 15u) != 0u
        || (strides[0] & 15u) != 0u || ((uint64_t)box[0] * bytes) % 16u != 0u || box[0] > 256u || box[1] > 256u
        || box[0] == 0u || box[1] == 0u || element_strides[0] != 1u || element_strides[1] != 1u
        || (swizzle != CU_TENSOR_MAP_SWIZZLE_NONE && !swizzled) || (swizzled && box[0] * bytes != 128u)
        || dims[0] == 0u || dims[1] == 0u) {
        return CUDA_ERROR_INVALID_VALUE;
    }
    TensorMap described = {static_cast<const unsigned char *>(base), {dims[0], dims[1]}, strides[0], {box[0], box[1]},
                           bytes, swizzled ? 1u : 0u};
    std::memset(map, 0, sizeof *map);
    std::memcpy(map, &described, sizeof described);
    return CUDA_SUCCESS;
}

inline float half_bits_to_float(uint16_t bits)
{
    return __half2float(__ushort_as_half(bits));
}

inline float bf16_bits_to_float(uint16_t bits)
{
    uint32_t wide = (uint32_t)bits << 16;
    float value;
    std::memcpy(&value, &wide, 4);
    return value;
}

inline unsigned int lane_of_thread();
inline unsigned int warp_of_thread();
// Uses that the hardware does not define or faults on, counted: a warp reading or writing
// tensor-memory lanes outside its own quarter (warp w of a block reaches lanes 32 (w mod 4) .. + 31
// only) or columns outside the block's allocation; a bulk tensor copy whose inner coordinate is
// not a multiple of 16 bytes or whose destination is not on a 128-byte (1024 with the swizzle)
// boundary; an L2 request that is not 16-byte aligned and sized.
inline std::atomic<unsigned int> lane_violations{0};
// which kinds were seen: 1 lanes, 2 columns of a load or store, 4 a bulk tensor copy, 8 an L2
// request, 16 columns of an MMA's accumulator
inline std::atomic<unsigned int> violation_kinds{0};
inline std::atomic<uint32_t> tmem_first_column{0};

// An engine that runs operations in the order they were issued, some time after the issue.
class Engine {
public:
    void start(unsigned int seed, unsigned int max_delay_us)
    {
        stop_ = false;
        rng_.seed(seed);
        max_delay_us_ = max_delay_us;
        worker_ = std::thread([this] { run(); });
    }
    void push(std::function<void()> op)
    {
        {
            std::lock_guard<std::mutex> lock(mutex_);
            queue_.push_back(std::move(op));
        }
        wake_.notify_one();
    }
    // Ends the thread after the queue has drained; returns how many operations were still
    // waiting or running when the call came (a block must not end with work in flight).
    size_t finish()
    {
        size_t in_flight;
        {
            std::lock_guard<std::mutex> lock(mutex_);
            in_flight = queue_.size() + (busy_ ? 1u : 0u);
            stop_ = true;
        }
        wake_.notify_one();
        worker_.join();
        return in_flight;
    }

private:
    void run()
    {
        for (;;) {
            std::function<void()> op;
            {
                std::unique_lock<std::mutex> lock(mutex_);
                wake_.wait(lock, [this] { return stop_ || !queue_.empty(); });
                if (queue_.empty()) {
                    return;
                }
                op = std::move(queue_.front());
                queue_.pop_front();
                busy_ = true;
            }
            if (max_delay_us_ != 0u) {
                const unsigned int wait = rng_() % (max_delay_us_ + 1u);
                if (wait != 0u) {
                    std::this_thread::sleep_for(std::chrono::microseconds(wait));
                }
            }
            op();
            {
                std::lock_guard<std::mutex> lock(mutex_);
                busy_ = false;
            }
        }
    }
    std::mutex mutex_;
    std::condition_variable wake_;
    std::deque<std::function<void()>> queue_;
    std::thread worker_;
    std::minstd_rand rng_;
    unsigned int max_delay_us_ = 0;
    bool stop_ = false, busy_ = false;
};

inline Engine copy_engine, tensor_pipe;
inline bool asynchronous = false;

// Fault injection on the host: the copy with this number (counted over the launch, from 0) never
// lands - its bytes are not credited - so the waits that depend on it must run out.
inline long long lost_copy = -1;
inline std::atomic<long long> copies_issued{0};
// Columns of tensor memory the running block holds (it must hand them back before it ends).
inline std::atomic<uint32_t> tmem_held{0};

inline void issue(Engine &engine, std::function<void()> op)
{
    if (asynchronous) {
        engine.push(std::move(op));
    } else {
        op();
    }
}

} // namespace q8emu

namespace q8 {

inline uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    const uint64_t both = ((uint64_t)b << 32) | a;
    uint32_t out = 0;
    for (int i = 0; i < 4; ++i) {
        const uint32_t pick = (sel >> (4 * i)) & 0xFu;
        uint32_t byte = (uint32_t)(both >> (8 * (pick & 7u))) & 0xFFu;
        if (pick & 8u) {
            byte = (byte & 0x80u) ? 0xFFu : 0x00u;
        }
        out |= byte << (8 * i);
    }
    return out;
}

inline uint32_t cvt_bf16x2_rn(float high, float low)
{
    const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rn(high));
    const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rn(low));
    return (hi << 16) | lo;
}

inline uint32_t cvt_f16x2_rn_sat(float high, float low)
{
    auto one = [](float v) -> uint32_t {
        if (v > 65504.0f) {
            v = 65504.0f;
        } else if (v < -65504.0f) {
            v = -65504.0f;
        }
        return __half_as_ushort(__float2half_rn(v));
    };
    return (one(high) << 16) | one(low);
}

inline uint32_t smem_u32(const void *p)
{
    return (uint32_t)(static_cast<const unsigned char *>(p) - q8emu::shared_memory) + q8emu::kSharedBase;
}

inline void ld_shared_v4(uint32_t addr, uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d)
{
    uint32_t w[4];
    std::memcpy(w, q8emu::shared_at(addr), 16);
    a = w[0], b = w[1], c = w[2], d = w[3];
}

inline void st_shared_b32(uint32_t addr, uint32_t value)
{
    std::memcpy(q8emu::shared_at(addr), &value, 4);
}

inline void st_shared_b16(uint32_t addr, uint32_t value)
{
    const uint16_t low = (uint16_t)value;
    std::memcpy(q8emu::shared_at(addr), &low, 2);
}

inline void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    const uint32_t w[4] = {a, b, c, d};
    std::memcpy(q8emu::shared_at(addr), w, 16);
}

inline void mbar_init(uint32_t bar, uint32_t count)
{
    std::lock_guard<std::mutex> lock(q8emu::barrier_mutex);
    q8emu::MBarrier fresh;
    fresh.count = fresh.pending = count;
    q8emu::barriers[bar] = fresh;
}

inline void mbar_init_fence() {}

inline void mbar_arrive(uint32_t bar)
{
    std::lock_guard<std::mutex> lock(q8emu::barrier_mutex);
    q8emu::MBarrier &b = q8emu::barriers.at(bar);
    b.pending -= 1;
    q8emu::advance(b);
}

inline void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    std::lock_guard<std::mutex> lock(q8emu::barrier_mutex);
    q8emu::MBarrier &b = q8emu::barriers.at(bar);
    b.tx += bytes;
    b.pending -= 1;
    q8emu::advance(b);
}

inline uint32_t mbar_try_wait(uint32_t bar, uint32_t parity)
{
    bool done;
    {
        std::lock_guard<std::mutex> lock(q8emu::barrier_mutex);
        done = (q8emu::barriers.at(bar).phase & 1u) != parity;
    }
    if (!done) {
        std::this_thread::yield();
    }
    return done ? 1u : 0u;
}

inline uint32_t mbar_test_wait(uint32_t bar, uint32_t parity)
{
    return mbar_try_wait(bar, parity);
}

inline void fence_proxy_async_smem() {}
inline void tma_prefetch_desc(const void *) {}

inline void emu_tma_load_2d(uint32_t dst, const q8emu::TensorMap &map, uint32_t bar, int c0, int c1)
{
    const uint32_t row_bytes = map.box[0] * map.elem_bytes;
    for (uint32_t r = 0; r < map.box[1]; ++r) {
        const long long row = (long long)c1 + r;
        for (uint32_t e = 0; e < map.box[0]; ++e) {
            const long long col = (long long)c0 + e;
            uint32_t offset = r * row_bytes + e * map.elem_bytes;
            if (map.swizzle128) {
                offset ^= (r & 7u) << 4;
            }
            unsigned char *to = q8emu::shared_at(dst) + offset;
            if (row >= 0 && col >= 0 && (uint64_t)row < map.dims[1] && (uint64_t)col < map.dims[0]) {
                std::memcpy(to, map.base + (uint64_t)row * map.stride_bytes + (uint64_t)col * map.elem_bytes,
                            map.elem_bytes);
            } else {
                std::memset(to, 0, map.elem_bytes); // out of range reads as zero
            }
        }
    }
    std::lock_guard<std::mutex> lock(q8emu::barrier_mutex);
    q8emu::MBarrier &b = q8emu::barriers.at(bar);
    b.tx -= (int64_t)row_bytes * map.box[1];
    q8emu::advance(b);
}

inline void tma_load_2d(uint32_t dst, const void *tmap, uint32_t bar, int c0, int c1)
{
    const q8emu::TensorMap map = *static_cast<const q8emu::TensorMap *>(tmap);
    if (((long long)c0 * (long long)map.elem_bytes) % 16 != 0 || dst % (map.swizzle128 ? 1024u : 128u) != 0u
        || c1 < 0) {
        q8emu::lane_violations += 1u;
        q8emu::violation_kinds |= 4u;
    }
    if (q8emu::copies_issued.fetch_add(1) == q8emu::lost_copy) {
        return;
    }
    q8emu::issue(q8emu::copy_engine, [=] { emu_tma_load_2d(dst, map, bar, c0, c1); });
}

inline void tmem_alloc(uint32_t smem_result, uint32_t columns)
{
    // the allocation sits at the top of the 512 columns, so a kernel that takes fewer than all of
    // them gets a base that is not zero (as a second block on the SM would) and must add it
    const uint32_t base = 512u - columns;
    if (q8emu::lane_of_thread() == 0u) {
        q8emu::tmem_held += columns;
        q8emu::tmem_first_column = base;
    }
    std::memcpy(q8emu::shared_at(smem_result), &base, 4);
}

inline void tmem_relinquish() {}
inline void tmem_dealloc(uint32_t, uint32_t columns)
{
    if (q8emu::lane_of_thread() == 0u) {
        q8emu::tmem_held -= columns;
    }
}
inline void tc_fence_before_sync() {}
inline void tc_fence_after_sync() {}

// D (+)= A * B for one 128 x N x 16 step.  `a_value(row, kk)` gives the A operand.
template <typename AValue>
inline void emu_mma(uint32_t d_tmem, AValue a_value, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    const uint32_t n = ((idesc >> 17) & 0x3Fu) << 3;
    const bool b_bf16 = ((idesc >> 10) & 1u) != 0u;
    const uint32_t d_col = d_tmem & 0xFFFFu;
    if (d_col < q8emu::tmem_first_column.load() || d_col + n > 512u) {
        q8emu::lane_violations += 1u;
        q8emu::violation_kinds |= 16u;
    }
    const uint32_t b_start = (uint32_t)(b_desc & 0x3FFFu) << 4;
    for (uint32_t row = 0; row < 128u; ++row) {
        float a[16];
        for (uint32_t kk = 0; kk < 16u; ++kk) {
            a[kk] = a_value(row, kk);
        }
        for (uint32_t col = 0; col < n; ++col) {
            float sum = 0.0f;
            for (uint32_t kk = 0; kk < 16u; ++kk) {
                // K-major row of 128 bytes, groups of 8 rows 1024 bytes apart, 128-byte swizzle
                uint32_t addr = b_start + (col >> 3) * 1024u + (col & 7u) * 128u + kk * 2u;
                addr ^= ((addr >> 7) & 7u) << 4;
                uint16_t bits;
                std::memcpy(&bits, q8emu::shared_at(addr), 2);
                const float b = b_bf16 ? q8emu::bf16_bits_to_float(bits) : q8emu::half_bits_to_float(bits);
                sum += a[kk] * b;
            }
            float total = sum;
            if (accumulate) {
                float before;
                std::memcpy(&before, &q8emu::tensor_memory[row][d_col + col], 4);
                total += before;
            }
            std::memcpy(&q8emu::tensor_memory[row][d_col + col], &total, 4);
        }
    }
}

inline void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    q8emu::issue(q8emu::tensor_pipe, [=] {
        const uint32_t a_col = a_tmem & 0xFFFFu;
        const bool a_bf16 = ((idesc >> 7) & 1u) != 0u;
        emu_mma(d_tmem, [&](uint32_t row, uint32_t kk) {
            const uint32_t word = q8emu::tensor_memory[row][a_col + kk / 2u];
            const uint16_t bits = (uint16_t)(kk & 1u ? word >> 16 : word & 0xFFFFu);
            return a_bf16 ? q8emu::bf16_bits_to_float(bits) : q8emu::half_bits_to_float(bits);
        }, b_desc, idesc, accumulate);
    });
}

inline void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    q8emu::issue(q8emu::tensor_pipe, [=] {
        const uint32_t a_start = (uint32_t)(a_desc & 0x3FFFu) << 4;
        const bool a_bf16 = ((idesc >> 7) & 1u) != 0u;
        emu_mma(d_tmem, [&](uint32_t row, uint32_t kk) {
            uint32_t addr = a_start + (row >> 3) * 1024u + (row & 7u) * 128u + kk * 2u;
            addr ^= ((addr >> 7) & 7u) << 4;
            uint16_t bits;
            std::memcpy(&bits, q8emu::shared_at(addr), 2);
            return a_bf16 ? q8emu::bf16_bits_to_float(bits) : q8emu::half_bits_to_float(bits);
        }, b_desc, idesc, accumulate);
    });
}

inline void umma_commit(uint32_t bar)
{
    q8emu::issue(q8emu::tensor_pipe, [=] { mbar_arrive(bar); });
}

// thread t of the warp reads / writes lane (base lane + t)
inline void emu_tmem_access(uint32_t taddr, uint32_t *v, const uint32_t *from, unsigned int count)
{
    const unsigned int lane = ((taddr >> 16) & 0xFFFFu) + q8emu::lane_of_thread();
    const unsigned int column = taddr & 0xFFFFu;
    if (((taddr >> 16) & 0xFFFFu) != 32u * (q8emu::warp_of_thread() & 3u)) {
        q8emu::lane_violations += 1u;
        q8emu::violation_kinds |= 1u;
    }
    if (column < q8emu::tmem_first_column.load() || column + count > 512u) {
        q8emu::lane_violations += 1u;
        q8emu::violation_kinds |= 2u;
    }
    for (unsigned int i = 0; i < count; ++i) {
        if (from != nullptr) {
            q8emu::tensor_memory[lane][column + i] = from[i];
        } else {
            v[i] = q8emu::tensor_memory[lane][column + i];
        }
    }
}

inline void tmem_ld_32x32(uint32_t taddr, uint32_t *v)
{
    emu_tmem_access(taddr, v, nullptr, 32);
}

inline void tmem_ld_32x16(uint32_t taddr, uint32_t *v)
{
    emu_tmem_access(taddr, v, nullptr, 16);
}

inline void tmem_ld_32x8(uint32_t taddr, uint32_t *v)
{
    emu_tmem_access(taddr, v, nullptr, 8);
}

inline void tmem_st_32x32(uint32_t taddr, const uint32_t *v)
{
    emu_tmem_access(taddr, nullptr, v, 32);
}

inline void tmem_st_wait() {}
inline void tmem_ld_wait() {}
inline void grid_launch_dependents() {}
inline void grid_dependency_wait() {}
inline void named_bar_sync(uint32_t, uint32_t) {}

inline uint32_t ld_acquire_gpu(const unsigned int *p)
{
    return reinterpret_cast<const std::atomic<unsigned int> *>(p)->load(std::memory_order_acquire);
}

inline uint32_t ld_acquire_sys(const unsigned int *p)
{
    return reinterpret_cast<const std::atomic<unsigned int> *>(p)->load(std::memory_order_acquire);
}

inline void st_release_sys(unsigned int *p, uint32_t v)
{
    reinterpret_cast<std::atomic<unsigned int> *>(p)->store(v, std::memory_order_release);
}

inline void st_release_gpu(unsigned int *p, uint32_t v)
{
    reinterpret_cast<std::atomic<unsigned int> *>(p)->store(v, std::memory_order_release);
}

// Clusters are not modelled: the emulated blocks run one after another, so the library never
// picks a cluster launch in this build, and a block is a cluster of its own.
inline uint32_t cluster_ctarank() { return 0u; }
inline uint32_t cluster_nctarank() { return 1u; }
inline void cluster_arrive_release() {}
inline void cluster_wait_acquire() {}
inline uint32_t mapa_shared(uint32_t addr, uint32_t) { return addr; }

inline void st_shared_cluster_f32(uint32_t addr, float v)
{
    std::memcpy(q8emu::shared_at(addr), &v, sizeof v);
}

inline void st_shared_cluster_v4_f32(uint32_t addr, float a, float b, float c, float d)
{
    const float w[4] = {a, b, c, d};
    std::memcpy(q8emu::shared_at(addr), w, sizeof w);
}

inline void st_shared_cluster_v2_f32(uint32_t addr, float a, float b)
{
    const float w[2] = {a, b};
    std::memcpy(q8emu::shared_at(addr), w, sizeof w);
}

inline float ld_shared_f32(uint32_t addr)
{
    float v;
    std::memcpy(&v, q8emu::shared_at(addr), sizeof v);
    return v;
}

} // namespace q8
