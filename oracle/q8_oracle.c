/* CPU oracle for the Q8_0 weight-matrix path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the host-side checking code that the AOTX reference keeps
 * in its own device tests.  It is the checker for the CUDA kernels of this repository: only
 * the test suite, the smoke check and the CPU-baseline leg of the benchmark may link or call
 * it.  The product library never does, and has no CPU path of its own.
 *
 * Parity pin: every function below is compared, in the CPU test suite, with the reference's
 * own host functions compiled from the reference's sources (the `_ref` library that the
 * recipe beside this file builds), and with the closed-form known-answer vector of
 * tests/embedded_modules_test.cu:22-51.
 *
 * Each function cites the reference lines it follows (paths relative to the reference root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define Q8O_BLOCK 32u       /* weights of one block:  cuda/model/matrix.cuh:25 */
#define Q8O_BLOCK_BYTES 34u /* fp16 scale + 32 int8: cuda/model/matrix.cuh:6-7,26 */

/* ---------------------------------------------------------------------------------------
 * IEEE binary16 / bfloat16 conversions (round to nearest even, subnormals kept).  The
 * reference uses the CUDA host functions __float2half / __half2float for these.
 * ------------------------------------------------------------------------------------- */
uint16_t q8o_f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, sizeof x);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mag = x & 0x7FFFFFFFu;
    if (mag > 0x7F800000u) {
        return (uint16_t)(sign | 0x7E00u | ((mag >> 13) & 0x3FFu));
    }
    if (mag >= 0x477FF000u) { /* 65520 and above, and infinity, round to infinity */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (mag < 0x38800000u) { /* below 2^-14: the result is a subnormal half or zero */
        uint32_t e = mag >> 23;
        if (e < 102u) { /* below 2^-25: rounds to zero */
            return (uint16_t)sign;
        }
        uint32_t m = (mag & 0x7FFFFFu) | 0x800000u;
        uint32_t shift = 126u - e; /* 14 .. 24 */
        uint32_t q = m >> shift;
        uint32_t rest = m & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1u);
        if (rest > half || (rest == half && (q & 1u))) {
            q += 1u;
        }
        return (uint16_t)(sign | q);
    }
    uint32_t v = mag - 0x38000000u;
    uint32_t lsb = (v >> 13) & 1u;
    v += 0xFFFu + lsb;
    return (uint16_t)(sign | (v >> 13));
}

float q8o_f16_to_f32(uint16_t h)
{
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = ((uint32_t)h >> 10) & 0x1Fu;
    uint32_t m = (uint32_t)h & 0x3FFu;
    uint32_t x;
    if (e == 0u) {
        if (m == 0u) {
            x = sign;
        } else {
            int shift = 0;
            while ((m & 0x400u) == 0u) {
                m <<= 1;
                ++shift;
            }
            m &= 0x3FFu;
            x = sign | ((uint32_t)(113 - shift) << 23) | (m << 13);
        }
    } else if (e == 31u) {
        x = sign | 0x7F800000u | (m << 13);
    } else {
        x = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &x, sizeof f);
    return f;
}

uint16_t q8o_f32_to_bf16(float f)
{
    uint32_t x;
    memcpy(&x, &f, sizeof x);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) {
        return (uint16_t)((x >> 16) | 0x40u);
    }
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

float q8o_bf16_to_f32(uint16_t h)
{
    uint32_t x = (uint32_t)h << 16;
    float f;
    memcpy(&f, &x, sizeof f);
    return f;
}

/* ---------------------------------------------------------------------------------------
 * The reference's fixture generator: splitmix64 and the unit draw.
 * tests/matrix_test.cu:60-72.
 * ------------------------------------------------------------------------------------- */
uint64_t q8o_next(uint64_t *state)
{
    uint64_t z = (*state += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

float q8o_unit(uint64_t *state)
{
    uint32_t bits = (uint32_t)(q8o_next(state) >> 40);
    return (float)bits / 8388608.0f - 1.0f;
}

/* Bytes of one row of k weights.  cuda/model/matrix.cuh:77-82. */
uint64_t q8o_row_bytes(uint32_t k)
{
    return (uint64_t)(k / Q8O_BLOCK) * Q8O_BLOCK_BYTES;
}

/* A tensor of random blocks, each with its own scale and values.
 * tests/matrix_test.cu:133-154 (the Q8_0 arm). */
void q8o_build(uint8_t *w, uint32_t n, uint32_t k, uint64_t seed)
{
    uint64_t stride = q8o_row_bytes(k);
    uint64_t state = seed;
    memset(w, 0, (size_t)(stride * n));
    for (uint32_t r = 0; r < n; ++r) {
        uint8_t *row = w + stride * r;
        for (uint32_t b = 0; b < k / Q8O_BLOCK; ++b) {
            float scale = 0.004f + 0.03f * (q8o_unit(&state) * 0.5f + 0.5f);
            uint16_t packed = q8o_f32_to_f16(scale);
            uint8_t *one = row + (size_t)b * Q8O_BLOCK_BYTES;
            one[0] = (uint8_t)(packed & 0xFFu);
            one[1] = (uint8_t)(packed >> 8);
            for (uint32_t i = 0; i < Q8O_BLOCK; ++i) {
                int q = (int)(q8o_next(&state) % 255u) - 127;
                one[2u + i] = (uint8_t)(int8_t)q;
            }
        }
    }
}

/* The rows of x, each value a half of a unit draw.  tests/matrix_test.cu:203-216. */
void q8o_input(uint16_t *x, uint32_t m, uint32_t k, uint64_t seed)
{
    uint64_t state = seed;
    for (size_t i = 0; i < (size_t)m * k; ++i) {
        x[i] = q8o_f32_to_f16(q8o_unit(&state));
    }
}

/* One dequantised weight as the bits of a half: half(float(q) * float(scale)), one
 * rounding.  cuda/model/matrix.cuh:413-422; host twin tests/matrix_test.cu:84-92. */
uint16_t q8o_weight_bits(const uint8_t *row, uint32_t j)
{
    const uint8_t *one = row + (size_t)(j / Q8O_BLOCK) * Q8O_BLOCK_BYTES;
    uint16_t scale = (uint16_t)((uint16_t)one[0] | ((uint16_t)one[1] << 8));
    int q = (int)(int8_t)one[2u + (j % Q8O_BLOCK)];
    return q8o_f32_to_f16((float)q * q8o_f16_to_f32(scale));
}

float q8o_weight(const uint8_t *row, uint32_t j)
{
    return q8o_f16_to_f32(q8o_weight_bits(row, j));
}

/* Rows [first, first+rows) of w as halves.  cuda/model/dequant.cu:9-22. */
void q8o_dequant(const uint8_t *w, uint32_t k, uint32_t first, uint32_t rows, uint16_t *out)
{
    uint64_t stride = q8o_row_bytes(k);
    for (uint32_t r = 0; r < rows; ++r) {
        const uint8_t *row = w + stride * (uint64_t)(first + r);
        for (uint32_t j = 0; j < k; ++j) {
            out[(size_t)r * k + j] = q8o_weight_bits(row, j);
        }
    }
}

static float q8o_x_value(const uint16_t *x, size_t at, int x_is_bf16)
{
    return x_is_bf16 ? q8o_bf16_to_f32(x[at]) : q8o_f16_to_f32(x[at]);
}

/* The reference product in double: y[i][j] = sum over c, in ascending c, of
 * double(float(x[i][c])) * double(weight(j, c)).  With swap the weight tensor is turned
 * (needs n == k).  tests/matrix_test.cu:224-239.  The rows of w are split over `threads`
 * host threads; every sum keeps the reference's order, so the result does not depend on
 * the thread count. */
void q8o_product(const uint8_t *w, uint32_t n, uint32_t k, const uint16_t *x, int x_is_bf16,
                 uint32_t m, double *y, int swap, int threads)
{
    uint64_t stride = q8o_row_bytes(k);
    if (threads < 1) {
        threads = 1;
    }
#ifdef _OPENMP
#pragma omp parallel num_threads(threads)
#endif
    {
        float *line = (float *)malloc((size_t)k * sizeof *line);
#ifdef _OPENMP
#pragma omp for schedule(static)
#endif
        for (int64_t j = 0; j < (int64_t)n; ++j) {
            for (uint32_t c = 0; c < k; ++c) {
                const uint8_t *row = w + stride * (uint64_t)(swap ? c : (uint32_t)j);
                line[c] = q8o_weight(row, swap ? (uint32_t)j : c);
            }
            for (uint32_t i = 0; i < m; ++i) {
                double sum = 0.0;
                for (uint32_t c = 0; c < k; ++c) {
                    sum += (double)q8o_x_value(x, (size_t)i * k + c, x_is_bf16)
                         * (double)line[c];
                }
                y[(size_t)i * n + (size_t)j] = sum;
            }
        }
        free(line);
    }
}

/* The reference's comparison: |got - want| over the larger of |want| and rms(want); a value
 * that is not finite is wrong.  Returns the count over tol.  tests/matrix_test.cu:246-274. */
uint32_t q8o_diff(const float *got, const double *want, size_t count, double tol,
                  double *worst)
{
    double sum = 0.0;
    for (size_t i = 0; i < count; ++i) {
        sum += want[i] * want[i];
    }
    double rms = sqrt(sum / (double)count);
    uint32_t bad = 0;
    double high = 0.0;
    for (size_t i = 0; i < count; ++i) {
        double base = fabs(want[i]);
        if (base < rms) {
            base = rms;
        }
        double rel = (base > 0.0) ? fabs((double)got[i] - want[i]) / base : 0.0;
        if (!isfinite((double)got[i])) {
            rel = INFINITY;
        }
        if (rel > high) {
            high = rel;
        }
        if (rel > tol) {
            bad += 1u;
        }
    }
    *worst = high;
    return bad;
}

/* The spot check of a large product: `count` sampled results against a dot product of the
 * same bytes, base max(|sum|, 1e-3 * sqrt(k * sum of squares)).
 * tests/matrix_test.cu:279-312.  `sample_seed` is the reference's 0x243F6A8885A308D3 ^
 * 0x5A5A5A5A when the caller wants the same samples. */
uint32_t q8o_spot(const uint8_t *w, uint32_t n, uint32_t k, const uint16_t *x, int x_is_bf16,
                  uint32_t m, const float *y, uint32_t count, uint64_t sample_seed, double tol,
                  double *worst)
{
    uint64_t stride = q8o_row_bytes(k);
    uint64_t state = sample_seed;
    uint32_t bad = 0;
    double high = 0.0;
    for (uint32_t s = 0; s < count; ++s) {
        uint32_t i = (uint32_t)(q8o_next(&state) % m);
        uint32_t j = (uint32_t)(q8o_next(&state) % n);
        const uint8_t *row = w + stride * (uint64_t)j;
        double sum = 0.0;
        double square = 0.0;
        for (uint32_t c = 0; c < k; ++c) {
            double one = (double)q8o_x_value(x, (size_t)i * k + c, x_is_bf16)
                       * (double)q8o_weight(row, c);
            sum += one;
            square += one * one;
        }
        double base = fabs(sum);
        double spread = sqrt(square * (double)k);
        if (base < spread * 1e-3) {
            base = spread * 1e-3;
        }
        double got = (double)y[(size_t)i * n + j];
        double rel = isfinite(got) ? fabs(got - sum) / base : INFINITY;
        if (rel > high) {
            high = rel;
        }
        if (rel > tol) {
            bad += 1u;
        }
    }
    *worst = high;
    return bad;
}

/* The acceptance bound this repository is held to for products:
 * max |got - want| <= 1e-2 * max |want| + 1e-3.  Returns 1 when it holds. */
int q8o_within_bound(const float *got, const double *want, size_t count, double *max_err,
                     double *bound)
{
    double high = 0.0;
    double top = 0.0;
    int finite = 1;
    for (size_t i = 0; i < count; ++i) {
        double err = fabs((double)got[i] - want[i]);
        if (!isfinite((double)got[i])) {
            finite = 0;
        }
        if (err > high) {
            high = err;
        }
        if (fabs(want[i]) > top) {
            top = fabs(want[i]);
        }
    }
    *max_err = high;
    *bound = 1e-2 * top + 1e-3;
    return finite && high <= *bound;
}

/* ---------------------------------------------------------------------------------------
 * Routed experts.
 * ------------------------------------------------------------------------------------- */

/* Router: logits = F32 router rows . half x, full softmax with the maximum taken away, the
 * rank of expert e = count of experts with a larger probability, or an equal one and a
 * lower index; ids[t][rank] = e for rank < used.  Kernel: cuda/model/experts.cu:10-75.
 * The arithmetic here is the double-precision host check of tests/expert_test.cu:113-153;
 * the kernel's own float probabilities must sit within 2e-6 of these. */
void q8o_route(const uint16_t *x, const float *router, uint32_t tokens, uint32_t hidden,
               uint32_t experts, uint32_t used, double *prob, uint32_t *ids)
{
    double *logit = (double *)malloc((size_t)experts * sizeof *logit);
    for (uint32_t t = 0; t < tokens; ++t) {
        double top = -INFINITY;
        double total = 0.0;
        for (uint32_t e = 0; e < experts; ++e) {
            double dot = 0.0;
            for (uint32_t d = 0; d < hidden; ++d) {
                dot += (double)router[(size_t)e * hidden + d]
                     * (double)q8o_f16_to_f32(x[(size_t)t * hidden + d]);
            }
            logit[e] = dot;
            if (dot > top) {
                top = dot;
            }
        }
        double *p = prob + (size_t)t * experts;
        for (uint32_t e = 0; e < experts; ++e) {
            p[e] = exp(logit[e] - top);
            total += p[e];
        }
        for (uint32_t e = 0; e < experts; ++e) {
            p[e] /= total;
        }
        for (uint32_t e = 0; e < experts; ++e) {
            uint32_t rank = 0;
            for (uint32_t o = 0; o < experts; ++o) {
                rank += (p[o] > p[e]) || (p[o] == p[e] && o < e);
            }
            if (rank < used) {
                ids[(size_t)t * used + rank] = e;
            }
        }
    }
    free(logit);
}

/* The same selection rule applied to float probabilities that the caller already holds
 * (for example the ones a device kernel produced).  cuda/model/experts.cu:63-72. */
void q8o_rank(const float *prob, uint32_t tokens, uint32_t experts, uint32_t used,
              uint32_t *ids)
{
    for (uint32_t t = 0; t < tokens; ++t) {
        const float *p = prob + (size_t)t * experts;
        for (uint32_t e = 0; e < experts; ++e) {
            uint32_t rank = 0;
            for (uint32_t o = 0; o < experts; ++o) {
                rank += (p[o] > p[e]) || (p[o] == p[e] && o < e);
            }
            if (rank < used) {
                ids[(size_t)t * used + rank] = e;
            }
        }
    }
}

/* Per token and rank: a one-row product on the slice of the token's expert.  The slice of
 * expert e of a [experts][n][k] tensor starts e * n * row_bytes(k) bytes in.
 * Kernel: cuda/model/expert_matrix.cu:8-27; host check tests/expert_test.cu:309-319, which
 * also sums |product| for its bound 2e-6 * magnitude + 2e-5. */
void q8o_expert_matrix(const uint8_t *w, uint32_t n, uint32_t k, const uint16_t *x,
                       const uint32_t *ids, uint32_t used, uint32_t rank, uint32_t tokens,
                       double *y, double *magnitude)
{
    uint64_t stride = q8o_row_bytes(k);
    for (uint32_t t = 0; t < tokens; ++t) {
        uint32_t e = ids[(size_t)t * used + rank];
        for (uint32_t row = 0; row < n; ++row) {
            const uint8_t *line = w + ((uint64_t)e * n + row) * stride;
            double want = 0.0;
            double mag = 0.0;
            for (uint32_t d = 0; d < k; ++d) {
                const uint8_t *one = line + (size_t)(d / Q8O_BLOCK) * Q8O_BLOCK_BYTES;
                uint16_t scale = (uint16_t)((uint16_t)one[0] | ((uint16_t)one[1] << 8));
                double weight = (double)q8o_f16_to_f32(scale)
                              * (double)(int)(int8_t)one[2u + d % Q8O_BLOCK];
                double product = weight * (double)q8o_f16_to_f32(x[(size_t)t * k + d]);
                want += product;
                mag += fabs(product);
            }
            y[(size_t)t * n + row] = want;
            if (magnitude != NULL) {
                magnitude[(size_t)t * n + row] = mag;
            }
        }
    }
}

/* The ordered weighted sum of the selected experts' outputs: for rank 0 the sum is
 * float(proj * p); for every later rank it is float(sum + float(proj * p)), the product and
 * the sum rounded separately.  proj holds [used][tokens][hidden].
 * Kernel: cuda/model/experts.cu:77-98; host twin tests/expert_test.cu:164-178. */
void q8o_ordered_sum(const float *proj, const float *prob, const uint32_t *ids,
                     uint32_t tokens, uint32_t hidden, uint32_t experts, uint32_t used,
                     float *sum)
{
    for (uint32_t r = 0; r < used; ++r) {
        for (uint32_t t = 0; t < tokens; ++t) {
            float weight = prob[(size_t)t * experts + ids[(size_t)t * used + r]];
            for (uint32_t d = 0; d < hidden; ++d) {
                size_t at = (size_t)t * hidden + d;
                volatile float product = proj[((size_t)r * tokens + t) * hidden + d] * weight;
                volatile float total = (r == 0u) ? product : sum[at] + product;
                sum[at] = total;
            }
        }
    }
}

/* The whole routed feed-forward step for given selections: for rank 0..used-1 in order,
 * gate = x.Wg[e], up = x.Wu[e], act = half(silu(gate) * up) with silu(g) = g / (1 + exp(-g)),
 * proj = act.Wd[e], then the ordered weighted sum above.
 * cuda/model/experts_host.cu:99-111; cuda/model/norm.cu:92-105; cuda/model/experts.cu:77-98.
 * Products are in double over the half-rounded weights, like the product reference; gate
 * and up are rounded to float before the activation, as the kernels hand them on as float.
 * `out` is float [tokens][hidden]; `act_out` (optional) is half bits [used][tokens][ffn]. */
void q8o_moe_ffn(const uint8_t *w_gate, const uint8_t *w_up, const uint8_t *w_down,
                 uint32_t experts, uint32_t hidden, uint32_t ffn, const uint16_t *x,
                 const float *prob, const uint32_t *ids, uint32_t tokens, uint32_t used,
                 float *out, uint16_t *act_out, int threads)
{
    uint64_t stride_in = q8o_row_bytes(hidden);
    uint64_t stride_down = q8o_row_bytes(ffn);
    if (threads < 1) {
        threads = 1;
    }
    float *proj = (float *)malloc((size_t)used * tokens * hidden * sizeof *proj);
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
#endif
    for (int64_t t = 0; t < (int64_t)tokens; ++t) {
        float *xv = (float *)malloc((size_t)hidden * sizeof *xv);
        float *act = (float *)malloc((size_t)ffn * sizeof *act);
        for (uint32_t d = 0; d < hidden; ++d) {
            xv[d] = q8o_f16_to_f32(x[(size_t)t * hidden + d]);
        }
        for (uint32_t r = 0; r < used; ++r) {
            uint32_t e = ids[(size_t)t * used + r];
            for (uint32_t f = 0; f < ffn; ++f) {
                const uint8_t *gate_row = w_gate + ((uint64_t)e * ffn + f) * stride_in;
                const uint8_t *up_row = w_up + ((uint64_t)e * ffn + f) * stride_in;
                double gate = 0.0;
                double up = 0.0;
                for (uint32_t d = 0; d < hidden; ++d) {
                    gate += (double)xv[d] * (double)q8o_weight(gate_row, d);
                    up += (double)xv[d] * (double)q8o_weight(up_row, d);
                }
                float g = (float)gate;
                float unit = g / (1.0f + expf(-g));
                uint16_t bits = q8o_f32_to_f16(unit * (float)up);
                act[f] = q8o_f16_to_f32(bits);
                if (act_out != NULL) {
                    act_out[((size_t)r * tokens + (size_t)t) * ffn + f] = bits;
                }
            }
            for (uint32_t d = 0; d < hidden; ++d) {
                const uint8_t *down_row = w_down + ((uint64_t)e * hidden + d) * stride_down;
                double sum = 0.0;
                for (uint32_t f = 0; f < ffn; ++f) {
                    sum += (double)act[f] * (double)q8o_weight(down_row, f);
                }
                proj[((size_t)r * tokens + (size_t)t) * hidden + d] = (float)sum;
            }
        }
        free(xv);
        free(act);
    }
    q8o_ordered_sum(proj, prob, ids, tokens, hidden, experts, used, out);
    free(proj);
}

int q8o_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
