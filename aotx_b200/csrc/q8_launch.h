// Internal launch interface between the C-ABI layer and the kernel files.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef Q8_HOST_EMULATION
#include <functional>
#endif

namespace q8 {

// Every kernel of the library is launched through this one function (or, for the tensor-core
// kernels with their launch attributes, through launch_tile_kernel in q8_tile.cuh).  In the
// tests' host emulation (-DQ8_HOST_EMULATION: the kernels compiled as host code) the same call
// runs the grid's blocks as host threads, so the host side of the library - argument checks,
// tensor maps, grids, workspaces - is the code that ships in both.
#ifdef Q8_HOST_EMULATION
void emulate_grid(dim3 grid, unsigned int threads, const std::function<void()> &block_body);
#endif

template <typename... Params, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(Params...), dim3 grid, unsigned int threads, size_t shared_bytes,
                                 cudaStream_t stream, Args... args)
{
#ifdef Q8_HOST_EMULATION
    (void)shared_bytes;
    (void)stream;
    emulate_grid(grid, threads, [&] { kernel(args...); });
    return cudaSuccess;
#else
    kernel<<<grid, threads, shared_bytes, stream>>>(args...);
    return cudaGetLastError();
#endif
}

// Raise a kernel's dynamic shared-memory limit once per device (the attribute is per device).
// `two_per_sm`: also ask for all of the SM's configurable memory as shared memory, so that two
// blocks of the kernel fit on one SM.
template <typename Kernel>
inline cudaError_t allow_shared_memory(Kernel kernel, unsigned int bytes, unsigned long long *done_mask,
                                       bool two_per_sm = false)
{
#ifdef Q8_HOST_EMULATION
    (void)kernel;
    (void)bytes;
    (void)done_mask;
    (void)two_per_sm;
    return cudaSuccess;
#else
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) {
        return err;
    }
    const unsigned long long bit = 1ull << (device & 63);
    if ((*done_mask & bit) == 0ull) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (err == cudaSuccess && two_per_sm) {
            err = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                       cudaSharedmemCarveoutMaxShared);
        }
        if (err != cudaSuccess) {
            return err;
        }
        *done_mask |= bit;
    }
    return cudaSuccess;
#endif
}

// y dtype codes as in the public header: 0 float, 1 half, 2 bfloat16.

// What a product does with a finished sum (the epilogue codes of the public header).
constexpr unsigned int kEpilogueStore = 0u;
constexpr unsigned int kEpilogueAdd = 1u;    // y is float and the sum is added to it
constexpr unsigned int kEpilogueSwiglu = 2u; // rows 2p, 2p+1 of w are gate and up of column p

cudaError_t launch_dequant(cudaStream_t stream, const void *w, unsigned int k, unsigned int first_row,
                           unsigned int rows, void *out);

// `epilogue`: 0 store, 1 add into a float y, 2 silu(gate) * up over row pairs of w into a y of
// n / 2 columns (the same three modes as the tensor-core kernel, see q8_tile.cuh).
cudaError_t launch_gemv_simt(cudaStream_t stream, const void *w, unsigned int n, unsigned int k,
                             const void *x, int x_bf16, unsigned int m, const unsigned int *m_dev,
                             void *y, int y_dtype, unsigned int epilogue = 0u);

// Every other block type of the model file (q_generic.cu, decoder in q_blocks.cuh).
bool block_type_known(unsigned int type);
unsigned int block_type_run(unsigned int type); // k must be a multiple of this; 0 for an unknown type
cudaError_t launch_dequant_any(cudaStream_t stream, const void *w, unsigned int type, unsigned int k,
                               unsigned int first_row, unsigned int rows, void *out);
cudaError_t launch_gemv_any(cudaStream_t stream, const void *w, unsigned int type, unsigned int n,
                            unsigned int k, const void *x, int x_bf16, unsigned int m,
                            const unsigned int *m_dev, void *y, int y_dtype);

cudaError_t launch_route(cudaStream_t stream, const void *x, const float *router, unsigned int tokens,
                         const unsigned int *tokens_dev, unsigned int hidden, unsigned int experts,
                         unsigned int used, float *prob, unsigned int *ids);

// Expert parallel (several GPUs, each holding a run of the experts; q8_api.cu aotx_q8_moe_ep).
// Where the rows of x of all GPUs' tokens lie: rows_per_part rows in each of `parts` arrays
// (own and peer-mapped); parts <= 1: one array.
struct RowParts {
    const void *base[8];
    unsigned int parts;
    unsigned int rows_per_part;
};
// Where the projections of this GPU's pairs lie: in the array of the GPU that holds the pair's
// expert (the experts dealt to `parts` GPUs, the first `extra` of them holding share + 1, the
// others share), at row first_pair + pair; parts <= 1: one array, first_pair 0.
struct ProjParts {
    const float *base[8];
    unsigned int parts;
    unsigned int share;
    unsigned int extra;
    unsigned int first_pair;
};

cudaError_t launch_expert_pairs_simt(cudaStream_t stream, const void *w_gate, const void *w_up,
                                     const void *w_down, unsigned int hidden, unsigned int ffn,
                                     const void *x, const unsigned int *ids, unsigned int experts,
                                     unsigned int tokens, const unsigned int *tokens_dev, unsigned int used,
                                     void *act, float *proj);

cudaError_t launch_expert_sum(cudaStream_t stream, const float *proj, const float *prob,
                              const unsigned int *ids, unsigned int tokens,
                              const unsigned int *tokens_dev, unsigned int hidden, unsigned int experts,
                              unsigned int used, void *out, int out_dtype);
cudaError_t launch_expert_sum_parts(cudaStream_t stream, const ProjParts &proj, const float *prob,
                                    const unsigned int *ids, unsigned int tokens,
                                    const unsigned int *tokens_dev, unsigned int hidden, unsigned int experts,
                                    unsigned int used, void *out, int out_dtype);

// The streaming tensor-core product.  Scratch, in two sets that alternate between launches:
// `partial` holds one float tile of 128 x token_tile per block of the grid, `flags` four words
// per block (zero between launches); `status` is one word that kernels only ever OR bits into.
struct UmmaScratch {
    float *partial;
    unsigned int *flags;
    unsigned int *status;
    unsigned int blocks;          // blocks the scratch was sized for
    unsigned long long tile_floats; // floats per block in `partial`
    // room for a binary16 copy of bfloat16 activations (batches of 33 to 128 rows: one pass
    // over x before the product instead of a rewrite of every x tile by every block); may be null
    void *x16 = nullptr;
    unsigned long long x16_bytes = 0;
};

// Column-split output: the product is columns [col0, col0 + n) of a y with row stride ldy,
// stored into every buffer of y_peer (own and peer-mapped).
struct PeerOut {
    void *y_peer[8];
    unsigned int peers;
    unsigned int col0;
    unsigned int ldy;
};

// The barrier between the ranks of a column-split product (q8_peers.cu): flag_arrays[r] is rank
// r's array of `peers` words as this GPU addresses it, step_word this rank's own counter.
cudaError_t launch_peer_barrier(cudaStream_t stream, void *const *flag_arrays, unsigned int peers,
                                unsigned int rank, unsigned int *step_word, unsigned int *status,
                                bool overlap = false);

// Returns cudaErrorNotSupported when the shape is outside what the kernel takes
// (k % 256 != 0, unaligned pointers); the caller then uses the general kernel.
cudaError_t launch_umma(cudaStream_t stream, const UmmaScratch &scratch, unsigned int sm_count,
                        const void *w, unsigned int n, unsigned int k, const void *x, int x_bf16,
                        unsigned int m, const unsigned int *m_dev, void *y, int y_dtype, unsigned int set,
                        bool overlap, const PeerOut *out = nullptr, unsigned int epilogue = 0u);

// Grouped mode of the decode-regime kernel: tiles from a device table (see q8_tile.cuh).
struct GroupTile;
cudaError_t launch_umma_grouped(cudaStream_t stream, const UmmaScratch &scratch, unsigned int sm_count,
                                const void *w_stacked, unsigned int total_rows, unsigned int k,
                                const void *x_sorted, unsigned int x_rows, unsigned int ntok,
                                const GroupTile *tiles, const unsigned int *count_dev, unsigned int max_tiles,
                                const unsigned int *row_map, void *y, unsigned int ldy, int y_dtype,
                                unsigned int set, bool overlap, unsigned int epilogue = 0u);

// Routed experts as grouped products (q8_moe.cu).  Offsets are bytes into the workspace.
struct MoeWorkspace {
    size_t act, proj, sorted_pair, counts, tiles_feed, tiles_down, x_sorted, gate, up, bytes;
    unsigned int max_feed, max_down;
};
MoeWorkspace moe_workspace_layout(unsigned int tokens, unsigned int used, unsigned int hidden,
                                  unsigned int ffn, unsigned int experts);
bool moe_grouped_supports(const void *w_gate, const void *w_up, const void *w_down, const void *x,
                          unsigned int hidden, unsigned int ffn, unsigned int experts);
cudaError_t launch_moe_grouped(cudaStream_t stream, const UmmaScratch &scratch, unsigned int sm_count,
                               unsigned int *launches, bool overlap, const void *w_gate, const void *w_up,
                               const void *w_down, unsigned int experts, unsigned int hidden,
                               unsigned int ffn, const void *x, const unsigned int *ids, unsigned int tokens,
                               const unsigned int *tokens_dev, unsigned int used, unsigned char *workspace,
                               const MoeWorkspace &ws, const RowParts *x_parts = nullptr, float *proj_out = nullptr);

cudaError_t launch_moe_grouped_fused(cudaStream_t stream, const UmmaScratch &scratch, unsigned int sm_count,
                                     unsigned int *launches, bool overlap, const void *w_gate_up,
                                     const void *w_down, unsigned int experts, unsigned int hidden,
                                     unsigned int ffn, const void *x, const unsigned int *ids,
                                     unsigned int tokens, const unsigned int *tokens_dev, unsigned int used,
                                     unsigned char *workspace, const MoeWorkspace &ws);

// ids_all[q * count + i] = ids_of_rank[q][i] - first_expert for the `parts` arrays of `count`
// selections each: an expert of another GPU becomes a number that names no local expert.
cudaError_t launch_collect_ids(cudaStream_t stream, const unsigned int *const *ids_of_rank, unsigned int parts,
                               unsigned int count, unsigned int first_expert, unsigned int *ids_all);

bool umma_supports(const void *w, unsigned int n, unsigned int k, const void *x, unsigned int m);

unsigned int umma_token_tile(unsigned int m);

} // namespace q8
