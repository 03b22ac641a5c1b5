/* aotx_q8_b200 - C ABI of the B200-native Q8_0 weight-matrix path.
 *
 * A drop-in for the matrix kernels of AOTX's model module.  Every entry point takes plain
 * pointers to device memory that the caller owns, enqueues its work on the caller's stream
 * and returns without synchronising, so it can be called inside a stream capture exactly
 * where the reference launches its own kernels.  Nothing is allocated by a call: scratch
 * memory lives in the context (made once, outside any capture) or is passed in.
 *
 * Weight layout (unchanged from the model file; reference cuda/model/matrix.cuh:6-7,26,77-82):
 * w[n][k] row-major, each row k/32 blocks of 34 bytes = little-endian binary16 scale then 32
 * signed bytes.  `type` is the model file's block type id (reference cuda/model/model.cuh:24-36).
 * 8 (Q8_0) is the path this library is built for: every entry point takes it, on the
 * tensor-core kernels where the shape allows.  aotx_q8_dequant and aotx_q8_matmul also take the
 * other types the reference's kernels read - F32 0, F16 1, Q4_0 2, Q4_1 3, Q5_0 6, Q5_1 7,
 * Q2_K 10, Q3_K 11, Q4_K 12, Q5_K 13, Q6_K 14 - through one decoder on the ordinary cores (rows
 * of whole blocks: k a multiple of 32, of 256 for the K types); any other id is
 * AOTX_Q8_ERR_TYPE.
 *
 * Return value: 0 on success, one of the AOTX_Q8_ERR_* codes otherwise.  On an error nothing
 * is enqueued and no output is written (the reference's kernels likewise write nothing for a
 * type they do not know: cuda/model/dequant.cu:24-25, cuda/model/gemm.cuh:236-237).
 *
 * Devices and threads: a context belongs to the device it was made for; the caller keeps that
 * device current in the calling thread and passes one of its streams, as the reference does
 * for its own launches.  A context keeps a launch counter and alternating scratch sets, so
 * calls on one context come from one thread at a time, and products on one context that run
 * on different streams at the same time need a context each (they would share the scratch).
 *
 * Paths are relative to the reference's source root.
 */
#ifndef AOTX_Q8_B200_H
#define AOTX_Q8_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AOTX_Q8_OK 0
#define AOTX_Q8_ERR_ARGUMENT 1    /* null pointer, k not a multiple of 32, bad dtype, misaligned */
#define AOTX_Q8_ERR_TYPE 2        /* block type other than Q8_0 */
#define AOTX_Q8_ERR_CUDA 3        /* a CUDA call failed; see aotx_q8_last_cuda_error */
#define AOTX_Q8_ERR_UNSUPPORTED 4 /* forced kernel family cannot take this shape */
#define AOTX_Q8_ERR_WORKSPACE 5   /* workspace null or too small */
#define AOTX_Q8_ERR_DEVICE 6      /* a device-side wait ran out (see aotx_q8_device_status) */

#define AOTX_Q8_TYPE_Q8_0 8u

/* element types of activations and outputs */
#define AOTX_Q8_F32 0
#define AOTX_Q8_F16 1
#define AOTX_Q8_BF16 2

/* kernel family, for aotx_q8_set_path */
#define AOTX_Q8_PATH_AUTO 0    /* tensor-core streaming kernel where it applies, else general */
#define AOTX_Q8_PATH_GENERAL 1 /* the any-shape kernel on the ordinary cores */
#define AOTX_Q8_PATH_TENSOR 2  /* the tcgen05 streaming kernel; ERR_UNSUPPORTED if it cannot run */

/* what a product does with a finished sum, for aotx_q8_matmul_fused */
#define AOTX_Q8_EPILOGUE_STORE 0  /* y[i][j] = sum: aotx_q8_matmul */
#define AOTX_Q8_EPILOGUE_ADD 1    /* y[i][j] = y[i][j] + sum, y float: the residual add */
#define AOTX_Q8_EPILOGUE_SWIGLU 2 /* y[i][p] = silu(sum over row 2p) * (sum over row 2p + 1) */

/* bits of the device status word */
#define AOTX_Q8_DEVICE_BARRIER_TIMEOUT 1u
#define AOTX_Q8_DEVICE_FLAG_TIMEOUT 2u

typedef struct aotx_q8_ctx aotx_q8_ctx;

/* Make / release the per-device context: SM count, the scratch tiles and flags of the
 * streaming kernel (about 40 MB) and a device status word.  Call outside stream capture.
 * No counterpart in the reference, whose kernels need no scratch; it takes the place of the
 * buffers that cuda/model/model_host.cu:95-153 makes before its capture starts. */
int aotx_q8_init(aotx_q8_ctx **ctx, int device);
int aotx_q8_destroy(aotx_q8_ctx *ctx);

/* Choose the kernel family for later calls on this context (tests and measurements). */
int aotx_q8_set_path(aotx_q8_ctx *ctx, int path);

/* Let consecutive products on one stream overlap (default on).  The tensor-core kernels are
 * launched as programmatic dependents: the blocks of a product may start, and stream weight
 * bytes, while the work before it on the stream is still finishing; they wait for that work
 * before they read x or the live batch or write y.  The weight tensor itself must therefore
 * not be written by the operation just before the product on the same stream; switch the
 * overlap off around such a sequence.  No counterpart in the reference. */
int aotx_q8_set_overlap(aotx_q8_ctx *ctx, int enabled);

/* The last CUDA error code an entry point of this context saw (cudaError_t as int). */
int aotx_q8_last_cuda_error(const aotx_q8_ctx *ctx);

/* Synchronise the device and read the status word that kernels raise instead of hanging;
 * 0 means every bounded wait completed.  `clear` != 0 zeroes it afterwards, and after a wait
 * that ran out also resets the hand-over state between blocks that such a launch can leave
 * behind: after AOTX_Q8_ERR_DEVICE call this with `clear` != 0 before the next product. */
int aotx_q8_device_status(aotx_q8_ctx *ctx, uint32_t *status, int clear);

/* Rows [first_row, first_row + rows) of w as binary16: out[r][j] = half(float(q) * float(d)),
 * bit-exact; for the other block types half(v) with v the correctly rounded float of the
 * format's expression (one fused multiply-add after exact products), as the reference's
 * readers form it (cuda/model/matrix.cuh:163-245, 255-340).  Replaces aotx_model_dequant (cuda/model/dequant.cu:26-70; declaration
 * cuda/model/model.cuh:112-116). */
int aotx_q8_dequant(aotx_q8_ctx *ctx, void *stream, const void *w, uint32_t type, uint32_t k,
                    uint32_t first_row, uint32_t rows, void *out_f16);

/* y[i][j] = sum_c x[i][c] * w[j][c], float sums, for i < m and j < n; no other element of y
 * is written.  x is [m][k] of x_dtype (F16 or BF16), y is [m][n] of y_dtype.
 * BF16 activations enter the tensor-core kernel as binary16: exact for magnitudes from 2^-14
 * to 65504, rounded below that range and saturated above it (activations after a norm layer
 * are far inside it); the general kernel reads them as they are.
 * If m_dev is not null it points to a device word holding the live batch; the product then
 * covers min(*m_dev, m) rows, read on the device at run time, so one captured node serves
 * every batch up to m.  With x F16, y F32 and m_dev this is the whole of
 * aotx_model_matrix's work (cuda/model/graph_host.cu:20-40): it stands in for
 * aotx_model_gemm (cuda/model/gemm.cu:7-14), aotx_model_gemv (cuda/model/gemv.cu:7-11),
 * aotx_model_line and aotx_model_product (cuda/model/product.cu:24-49) and the PTX module
 * aotx_gemv_q8 (ptx/gemv_q8.ptx:18-223). */
int aotx_q8_matmul(aotx_q8_ctx *ctx, void *stream, const void *w, uint32_t type, uint32_t n,
                   uint32_t k, const void *x, int x_dtype, uint32_t m, const uint32_t *m_dev,
                   void *y, int y_dtype);

/* The product with the step that follows it in a layer folded into its store, so that the
 * float result never makes a round trip through memory and one launch goes away:
 *   AOTX_Q8_EPILOGUE_ADD     y is the float residual stream and the product is added to it,
 *                            y[i][j] = fadd(y[i][j], sum): the O and down projections followed
 *                            by aotx_model_residual (cuda/model/norm.cu:78-89;
 *                            cuda/model/graph_host.cu:86,96).  y_dtype must be F32.
 *   AOTX_Q8_EPILOGUE_SWIGLU  w holds gate and up rows interleaved (row 2p = gate row p,
 *                            row 2p + 1 = up row p; n even counts both), y is [m][n / 2] and
 *                            y[i][p] = silu(gate sum) * (up sum), silu(g) = g / (1 + expf(-g)),
 *                            rounded once to y_dtype: the gate and up projections followed by
 *                            aotx_model_swiglu (cuda/model/norm.cu:92-105;
 *                            cuda/model/graph_host.cu:88-92).  With y_dtype F16 this is the
 *                            reference's `act` buffer.
 * AOTX_Q8_EPILOGUE_ADD forms the same float sums as aotx_q8_matmul on the same shape and adds
 * each once, so it equals the two-step form bit for bit.  AOTX_Q8_EPILOGUE_SWIGLU runs over a
 * tensor of twice the rows, which moves the points where long rows are cut between blocks, so
 * its gate and up sums can differ from the separate products' in the last bits of a float (the
 * activations then differ by at most a binary16 rounding step).
 * AOTX_Q8_EPILOGUE_STORE is aotx_q8_matmul itself.  Every shape is served (tensor-core
 * kernel or general kernel, as for aotx_q8_matmul). */
int aotx_q8_matmul_fused(aotx_q8_ctx *ctx, void *stream, const void *w, uint32_t type, uint32_t n,
                         uint32_t k, const void *x, int x_dtype, uint32_t m, const uint32_t *m_dev,
                         void *y, int y_dtype, int epilogue);

/* Router of a routed-expert layer: prob[t][e] = softmax over all experts of
 * router[e] . x[t] (float router rows, binary16 x), ids[t][r] = the expert of rank r < used,
 * ties to the lower index.  experts <= 256; hidden <= 10240 (the kernel keeps four rows of x
 * as floats in shared memory), more returns AOTX_Q8_ERR_UNSUPPORTED.  Replaces
 * aotx_model_expert_route (cuda/model/experts.cu:10-75). */
int aotx_q8_moe_route(aotx_q8_ctx *ctx, void *stream, const void *x_f16, const float *router,
                      uint32_t tokens, const uint32_t *tokens_dev, uint32_t hidden,
                      uint32_t experts, uint32_t used, float *prob, uint32_t *ids);

/* Bytes of workspace aotx_q8_moe_ffn needs for this shape. */
size_t aotx_q8_moe_workspace_bytes(uint32_t tokens, uint32_t used, uint32_t hidden, uint32_t ffn);

/* The routed feed-forward step for given selections.  For each token t and rank r in
 * ascending order, with e = ids[t][r]: gate = x[t] . Wg[e], up = x[t] . Wu[e],
 * act = half(silu(gate) * up), proj = act . Wd[e]; out[t] = the rank-ordered sum of
 * float(proj * prob[t][e]) (product and sum rounded separately).  Wg, Wu are
 * [experts][ffn][hidden], Wd is [experts][hidden][ffn], all Q8_0.  Replaces the loop of
 * aotx_model_capture_experts (cuda/model/experts_host.cu:99-111): aotx_model_expert_matrix
 * (cuda/model/expert_matrix.cu:8-63), aotx_model_swiglu (cuda/model/norm.cu:92-105) and
 * aotx_model_expert_add (cuda/model/experts.cu:77-98).
 * A selection ids[t][r] >= experts names no expert: it is left out of the products and adds
 * nothing to out[t] (the reference's selections come from its own router and are always in the
 * table; here they come from the caller, and no value of them may make a kernel read outside
 * the tensors). */
int aotx_q8_moe_ffn(aotx_q8_ctx *ctx, void *stream, const void *w_gate, const void *w_up,
                    const void *w_down, uint32_t type, uint32_t experts, uint32_t hidden,
                    uint32_t ffn, const void *x_f16, const float *prob, const uint32_t *ids,
                    uint32_t tokens, const uint32_t *tokens_dev, uint32_t used, void *out,
                    int out_dtype, void *workspace, size_t workspace_bytes);

/* aotx_q8_moe_ffn with gate and up of every expert in one tensor, rows interleaved:
 * w_gate_up is [experts][2 * ffn][hidden] with row 2r of an expert its gate row r and row
 * 2r + 1 its up row r.  One grouped product applies the gated unit in its store and writes the
 * binary16 activations, the down product follows: two tensor-core launches where aotx_q8_moe_ffn
 * has three and an elementwise kernel (result equal up to the float summation order of the gate
 * and up sums, see aotx_q8_matmul_fused).  Needs the shapes of the
 * grouped kernels (hidden and ffn multiples of 256, 16-byte aligned tensors), else
 * AOTX_Q8_ERR_UNSUPPORTED.  Workspace as for aotx_q8_moe_ffn. */
int aotx_q8_moe_ffn_fused(aotx_q8_ctx *ctx, void *stream, const void *w_gate_up, const void *w_down,
                          uint32_t type, uint32_t experts, uint32_t hidden, uint32_t ffn,
                          const void *x_f16, const float *prob, const uint32_t *ids, uint32_t tokens,
                          const uint32_t *tokens_dev, uint32_t used, void *out, int out_dtype,
                          void *workspace, size_t workspace_bytes);

/* The rank-ordered weighted sum alone: proj is float [tokens][used][hidden] (the output of
 * the selected experts, rank-major inside a token); out[t] = fmul(proj[t][0], p0), then for each
 * later rank fadd(out[t], fmul(proj[t][r], pr)), pr = prob[t][ids[t][r]].  Bit-exact with
 * aotx_model_expert_add run for rank 0..used-1 (cuda/model/experts.cu:77-98). */
int aotx_q8_moe_combine(aotx_q8_ctx *ctx, void *stream, const float *proj, const float *prob,
                        const uint32_t *ids, uint32_t tokens, const uint32_t *tokens_dev,
                        uint32_t hidden, uint32_t experts, uint32_t used, void *out, int out_dtype);

/* Column-split product for several GPUs of one box: w holds this GPU's n rows of a wider tensor,
 * the result is columns [col0, col0 + n) of y[m][ldy], and every tile is stored into all of
 * y_peers[0..peers) - this GPU's copy of y and the peers' copies, given as device addresses
 * that this GPU can store through (peer-mapped or symmetric memory).  The gather of the
 * column slices thus happens in the kernel's own stores; the caller only has to order the
 * GPUs afterwards (a barrier) before anyone reads y.  Only the tensor-core kernels serve it
 * (k % 256 == 0, 16-byte aligned w and x); peers <= 8.  The reference is single-GPU and has no
 * counterpart. */
int aotx_q8_matmul_peers(aotx_q8_ctx *ctx, void *stream, const void *w, uint32_t type, uint32_t n,
                         uint32_t k, const void *x, int x_dtype, uint32_t m, const uint32_t *m_dev,
                         void *const *y_peers, uint32_t peers, uint32_t ldy, uint32_t col0, int y_dtype);

/* The barrier that ends a column-split step, the library's own: flag_arrays[r] is rank r's array
 * of `peers` 32-bit words (zero at the start; device memory that every rank can store into, as
 * this GPU addresses it), step_word a word of this rank's own device memory (zero at the start)
 * that the call counts up, so that a call captured in a CUDA graph arrives with a new number on
 * every replay.  One small kernel: it writes the step number into this rank's word of every
 * rank's array (ordinary system-scope stores, after a system-scope fence over what this GPU
 * stored before) and waits until all words of its own array have reached it.  The wait is
 * bounded (about two seconds of SM clock): when it runs out, AOTX_Q8_DEVICE_FLAG_TIMEOUT is
 * raised in the context's status word and the kernel ends.  Every rank calls it the same number
 * of times.  No counterpart in the reference (single GPU). */
int aotx_q8_peer_barrier(aotx_q8_ctx *ctx, void *stream, void *const *flag_arrays, uint32_t peers,
                         uint32_t rank, uint32_t *step_word);

/* aotx_q8_matmul_peers followed by aotx_q8_peer_barrier on the same stream: one call per rank
 * and step for a projection split by output columns (LM head, 70B-class FFN).  After it, on
 * every rank, y holds all columns.  This is the form that replaces "product, then all-gather of
 * the slices": the gather happens in the kernel's own stores, over NVLink, while the weights
 * stream.  No counterpart in the reference. */
int aotx_q8_matmul_colsplit(aotx_q8_ctx *ctx, void *stream, const void *w, uint32_t type, uint32_t n,
                            uint32_t k, const void *x, int x_dtype, uint32_t m, const uint32_t *m_dev,
                            void *const *y_peers, void *const *flag_arrays, uint32_t peers, uint32_t rank,
                            uint32_t ldy, uint32_t col0, int y_dtype, uint32_t *step_word);

/* The routed-expert step over several GPUs of one box (expert parallel), one call per rank and
 * step.  The experts are dealt to the ranks in runs (rank r holds experts [r * E / peers ...) as
 * aotx_gguf_row_range deals rows: the first E % peers ranks hold one more); w_gate / w_up /
 * w_down are this rank's experts only.  Every rank has `tokens` tokens of its own:
 * x_of_rank[q] ([tokens][hidden] binary16) and ids_of_rank[q] ([tokens][used], expert numbers
 * of the whole table) are rank q's activations and selections, proj_of_rank[q]
 * ([peers * tokens * used][hidden] float) the array in which rank q leaves the projections of
 * its experts - all as this GPU addresses them (peer-mapped or symmetric memory; q == rank:
 * this GPU's own).  prob ([tokens][experts_total]) and out ([tokens][hidden]) are this rank's.
 *
 * The call is the single-GPU step with the exchange folded into its kernels: after the
 * library's barrier (every rank's x and ids are in place) the gather that sorts the rows by
 * expert reads each row straight from the memory of the GPU that holds the token, the grouped
 * products run on the pairs that name one of this rank's experts, a second barrier follows, and
 * the rank-ordered weighted sum reads each pair's projection straight from the GPU that
 * computed it.  A row of x crosses NVLink once per remote pair, a projection once; there is no
 * staging buffer, no padding, no library collective and no count ever comes to the host, so the
 * step is a fixed sequence of kernels (CUDA-graph capturable).  The result equals the
 * single-GPU step's to float rounding (an expert sees the same pairs in the same order; where a
 * tile's depth is cut between blocks differs with the number of local experts).  flag_arrays /
 * step_word: as for aotx_q8_peer_barrier (two barriers per call).  Workspace:
 * aotx_q8_moe_ep_workspace_bytes.  Needs the tensor-core path (hidden, ffn multiples of 256).
 * No counterpart in the reference (single GPU). */
size_t aotx_q8_moe_ep_workspace_bytes(uint32_t tokens, uint32_t used, uint32_t hidden, uint32_t ffn,
                                      uint32_t peers);
int aotx_q8_moe_ep(aotx_q8_ctx *ctx, void *stream, const void *w_gate, const void *w_up, const void *w_down,
                   uint32_t type, uint32_t experts_total, uint32_t hidden, uint32_t ffn,
                   const void *const *x_of_rank, const uint32_t *const *ids_of_rank, const float *prob,
                   uint32_t tokens, uint32_t used, float *const *proj_of_rank, void *const *flag_arrays,
                   uint32_t peers, uint32_t rank, uint32_t *step_word, void *out, int out_dtype,
                   void *workspace, size_t workspace_bytes);

/* The product without a context, for callers that cannot allocate device memory (a frozen
 * memory plan, a process whose device footprint must not grow, a plug-in that only gets a
 * stream and buffers).  Same arguments and result as aotx_q8_matmul; the scratch the kernel
 * needs is a fixed array inside the library (about 5.3 MB on every GPU that loads it, held
 * until the process exits), which limits a call to m <= 64 rows of x: more returns
 * AOTX_Q8_ERR_WORKSPACE and enqueues nothing.  It calls no cudaMalloc or cudaFree.  The first
 * call on each device looks the array up (cudaGetSymbolAddress): make that call before any
 * stream capture.  All calls share the array and clear the part that must start at zero; two
 * calls that overlap on the GPU (different streams, no ordering) race on it.  First calls made
 * from several host threads at once are safe (the look-up is under a lock).  The other block
 * types are served too (they use no scratch).
 * It has no counterpart in the reference. */
int aotx_q8_matmul_static(void *stream, const void *w, uint32_t type, uint32_t n, uint32_t k,
                          const void *x, int x_dtype, uint32_t m, const uint32_t *m_dev, void *y,
                          int y_dtype);

/* The status word of the fixed array on the current device, the counterpart of
 * aotx_q8_device_status for aotx_q8_matmul_static: synchronises the device, copies the word to
 * *status (0 = every wait of every static call ended in time) and, with clear != 0, resets the
 * word and the hand-over flags a cut-short launch may have left.  Allocates nothing.  Returns
 * AOTX_Q8_ERR_DEVICE when the word is not zero.  No counterpart in the reference. */
int aotx_q8_static_status(uint32_t *status, int clear);

#ifdef __cplusplus
}
#endif

#endif
