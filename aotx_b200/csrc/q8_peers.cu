// The barrier between the GPUs of a column-split product: after a rank has stored its slice of y
// into every rank's buffer (aotx_q8_matmul_peers), nobody may read y before every rank has done
// so.  Each rank owns an array of `peers` flag words that the other ranks can store into through
// peer-mapped addresses; arriving means writing the step number into one's own word of every
// rank's array, and the barrier is passed when all words of the own array have reached that
// number.  Ordinary stores and loads at system scope: no multicast, no library on the path.  The
// wait is bounded like every wait of this library: when it runs out the kernel raises
// Q8_DEV_FLAG_TIMEOUT in the status word and ends, so a rank that never arrives costs the others
// two seconds and an error code, not the GPU.
//
// The step number lives in device memory (one word per rank, counted up by the kernel), so a
// call captured in a CUDA graph arrives with a new number on every replay.  The reference is
// single-GPU and has no counterpart.
#include "q8_common.cuh"
#include "q8_launch.h"

namespace q8 {

struct PeerFlags {
    unsigned int *of_rank[8]; // the flag array of every rank, as this GPU addresses it
};

__global__ void q8_peer_barrier_kernel(PeerFlags flags, unsigned int peers, unsigned int rank,
                                       unsigned int *step_word, unsigned int *status)
{
    __shared__ unsigned int step_shared;
    // Launched with the programmatic attribute, this kernel starts while the product before it
    // still runs and lets the product after it start as well (that one streams weights and
    // touches nothing else before its own wait): the launch gaps either side of the barrier and
    // the next product's pipeline fill overlap the wait for the peers.  Everything this kernel
    // does comes after the work before it has completed.
    grid_launch_dependents();
    grid_dependency_wait();
    if (threadIdx.x == 0) {
        step_shared = *step_word + 1u;
    }
    __syncthreads();
    const unsigned int step = step_shared;
    const unsigned int peer = threadIdx.x;
    if (peer < peers) {
        // everything this GPU stored before (the slices of y) becomes visible before the word
        __threadfence_system();
        st_release_sys(flags.of_rank[peer] + rank, step);
        const unsigned int *mine = flags.of_rank[rank] + peer;
        const long long begin = clock64();
        // wrap-safe "has reached": the words only ever count up, one barrier at a time
        while ((int)(ld_acquire_sys(mine) - step) < 0) {
            if (clock64() - begin > Q8_WAIT_CYCLES) {
                atomicOr(status, Q8_DEV_FLAG_TIMEOUT);
                break;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        *step_word = step;
    }
}

cudaError_t launch_peer_barrier(cudaStream_t stream, void *const *flag_arrays, unsigned int peers,
                                unsigned int rank, unsigned int *step_word, unsigned int *status, bool overlap)
{
    PeerFlags flags = {};
    for (unsigned int i = 0; i < 8u; ++i) {
        flags.of_rank[i] = i < peers ? static_cast<unsigned int *>(flag_arrays[i]) : nullptr;
    }
#ifndef Q8_HOST_EMULATION
    if (overlap) {
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(1, 1, 1);
        config.blockDim = dim3(32, 1, 1);
        config.stream = stream;
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[0].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        return cudaLaunchKernelEx(&config, q8_peer_barrier_kernel, flags, peers, rank, step_word, status);
    }
#endif
    (void)overlap;
    return launch_kernel(q8_peer_barrier_kernel, dim3(1, 1, 1), 32u, 0, stream, flags, peers, rank, step_word,
                         status);
}

} // namespace q8
