// C++ host shim: the reference's matrix seam on top of the C ABI.
//
// The reference's layer capture code calls one host function per projection,
//     aotx_model_matrix(hold, w, type, n, k, x, m, y, which)
// (cuda/model/graph_host.h:47-52, body cuda/model/graph_host.cu:20-40), while a stream
// capture is open on hold->stream.  In the prefill graph it launches one tensor-core kernel;
// in the decode graph it adds three nodes (PTX module, memory-bound kernel, tensor-core
// kernel) that each read the live batch from a device word and exit when it is not theirs.
// Here both cases are one call of aotx_q8_matmul: the streaming kernel serves every batch
// and reads the live batch itself.
//
// The argument meaning and the error behaviour follow the reference: errors stop the
// program and name the call (cuda/boot/check.h:14-34); a block type the kernels do not
// serve writes nothing.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include "aotx_q8_b200.h"

// Which batch word a matrix node reads (cuda/model/forward.cuh; cuda/model/decode_module_host.cu:19-40).
#define AOTX_B200_BATCH_TOKENS 0u
#define AOTX_B200_BATCH_ROWS 1u

// The part of the reference's per-role state (cuda/model/graph_host.h:14-39) that the matrix
// seam reads, plus the context of this library.
struct aotx_b200_hold {
    aotx_q8_ctx *q8;               // made by aotx_q8_init before the capture starts
    cudaStream_t stream;           // the stream under capture
    unsigned int decode;           // 1 while the decode graph is captured: batch comes from a device word
    const unsigned int *batch[2];  // device addresses of the live batch: [tokens, rows]
};

static inline void aotx_b200_check(int code, const char *call)
{
    if (code == AOTX_Q8_OK) {
        return;
    }
    std::fprintf(stderr, "%s: aotx_q8 error %d\n", call, code);
    std::exit(1);
}

// Put one matrix product in the capture.  `m` is the batch of the prefill graph, or the
// largest batch of the decode graph, as in the reference.
static inline void aotx_model_matrix(aotx_b200_hold *hold, const void *w, unsigned int type,
                                     unsigned int n, unsigned int k, const half *x, unsigned int m,
                                     float *y, unsigned int which)
{
    const unsigned int *live = hold->decode != 0u ? hold->batch[which & 1u] : nullptr;
    int code = aotx_q8_matmul(hold->q8, (void *)hold->stream, w, type, n, k, x, AOTX_Q8_F16, m, live, y,
                              AOTX_Q8_F32);
    if (code == AOTX_Q8_ERR_TYPE) {
        return; /* the reference's kernels write nothing for a type they do not read */
    }
    aotx_b200_check(code, "aotx_model_matrix");
}

// The product of the O or down projection followed by the residual add, as one node:
// resid[i][j] += sum (aotx_model_matrix(..., work->proj, ...) then aotx_model_residual,
// cuda/model/graph_host.cu:84-86, 93-96; cuda/model/norm.cu:78-89).
static inline void aotx_model_matrix_residual(aotx_b200_hold *hold, const void *w, unsigned int type,
                                              unsigned int n, unsigned int k, const half *x, unsigned int m,
                                              float *resid, unsigned int which)
{
    const unsigned int *live = hold->decode != 0u ? hold->batch[which & 1u] : nullptr;
    int code = aotx_q8_matmul_fused(hold->q8, (void *)hold->stream, w, type, n, k, x, AOTX_Q8_F16, m, live,
                                    resid, AOTX_Q8_F32, AOTX_Q8_EPILOGUE_ADD);
    if (code == AOTX_Q8_ERR_TYPE) {
        return;
    }
    aotx_b200_check(code, "aotx_model_matrix_residual");
}

// Gate and up projections and the gated unit as one node: `w_gate_up` holds the two tensors'
// rows interleaved (2 * ffn rows), act[i][p] = half(silu(gate) * up)
// (cuda/model/graph_host.cu:88-92; cuda/model/norm.cu:92-105).
static inline void aotx_model_matrix_swiglu(aotx_b200_hold *hold, const void *w_gate_up, unsigned int type,
                                            unsigned int ffn, unsigned int k, const half *x, unsigned int m,
                                            half *act, unsigned int which)
{
    const unsigned int *live = hold->decode != 0u ? hold->batch[which & 1u] : nullptr;
    int code = aotx_q8_matmul_fused(hold->q8, (void *)hold->stream, w_gate_up, type, 2u * ffn, k, x, AOTX_Q8_F16,
                                    m, live, act, AOTX_Q8_F16, AOTX_Q8_EPILOGUE_SWIGLU);
    if (code == AOTX_Q8_ERR_TYPE) {
        return;
    }
    aotx_b200_check(code, "aotx_model_matrix_swiglu");
}

// Rows of a tensor as halves (the reference launches aotx_model_dequant directly:
// tests/matrix_test.cu:363; cuda/model/model.cuh:112-116).
static inline void aotx_model_dequant_rows(aotx_b200_hold *hold, const void *w, unsigned int type,
                                           unsigned int k, unsigned int first_row, unsigned int rows,
                                           half *out)
{
    int code = aotx_q8_dequant(hold->q8, (void *)hold->stream, w, type, k, first_row, rows, out);
    if (code == AOTX_Q8_ERR_TYPE) {
        return;
    }
    aotx_b200_check(code, "aotx_model_dequant");
}
