// The reference's matrix seam, called from C++ the way the reference calls it.
//
// include/aotx_b200_seam.hpp re-states aotx_model_matrix (cuda/model/graph_host.h:47-52) on
// top of the C ABI.  This program drives it like the reference's own matrix test
// (tests/matrix_test.cu: seeded fixture, device run, host product in double, the
// error-over-max(|want|, rms) measure, a guard value in the rows that must stay untouched)
// and like its layer capture (cuda/model/graph_host.cu:20-40: the call sits inside an open
// stream capture; in the decode graph the batch is a device word that changes between
// replays of one graph).
//
// Prints one line per case and "pass" at the end; exits 1 on the first failure.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "aotx_b200_seam.hpp"

#ifdef SEAM_DRY_RUN
#include "seam_dry.h" // host stand-ins for the device, see there
#endif

#define CHECK_CUDA(call)                                                                       \
    do {                                                                                       \
        cudaError_t err_ = (call);                                                             \
        if (err_ != cudaSuccess) {                                                             \
            std::fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(err_));                 \
            std::exit(1);                                                                      \
        }                                                                                      \
    } while (0)

static const float kGuard = -12345.0f;

struct Mixer {
    uint64_t state;
    uint64_t next()
    {
        uint64_t z = (state += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    float unit() { return (float)(next() >> 40) / 16777216.0f; } // [0, 1)
};

// w[n][k] in the model file's layout: per 32 weights a binary16 scale, then 32 signed bytes.
static std::vector<unsigned char> make_weights(Mixer &mix, unsigned int n, unsigned int k)
{
    std::vector<unsigned char> w((size_t)n * (k / 32u) * 34u);
    unsigned char *at = w.data();
    for (size_t b = 0; b < (size_t)n * (k / 32u); ++b, at += 34) {
        __half d = __float2half(0.002f + 0.03f * mix.unit());
        std::memcpy(at, &d, 2);
        for (int i = 0; i < 32; ++i) {
            at[2 + i] = (unsigned char)(mix.next() >> 56);
        }
    }
    return w;
}

static std::vector<__half> make_input(Mixer &mix, unsigned int m, unsigned int k)
{
    std::vector<__half> x((size_t)m * k);
    for (auto &v : x) {
        v = __float2half(2.0f * mix.unit() - 1.0f);
    }
    return x;
}

static std::vector<double> host_product(const std::vector<unsigned char> &w, unsigned int n, unsigned int k,
                                        const std::vector<__half> &x, unsigned int m)
{
    std::vector<float> wf((size_t)n * k);
    for (size_t b = 0; b < (size_t)n * (k / 32u); ++b) {
        __half d;
        std::memcpy(&d, &w[b * 34u], 2);
        for (int i = 0; i < 32; ++i) {
            // the value the kernels multiply with: half(float(q) * float(d))
            wf[b * 32u + i] = __half2float(__float2half((float)(signed char)w[b * 34u + 2u + i] * __half2float(d)));
        }
    }
    std::vector<double> want((size_t)m * n);
    for (unsigned int i = 0; i < m; ++i) {
        for (unsigned int j = 0; j < n; ++j) {
            double sum = 0.0;
            for (unsigned int c = 0; c < k; ++c) {
                sum += (double)__half2float(x[(size_t)i * k + c]) * (double)wf[(size_t)j * k + c];
            }
            want[(size_t)i * n + j] = sum;
        }
    }
    return want;
}

// The reference's measure: an entry is wrong when its error exceeds 1e-2 of the larger of
// |want| and the root mean square of the expected rows.
static unsigned int count_wrong(const std::vector<float> &got, const std::vector<double> &want, unsigned int rows,
                                unsigned int n, double *worst)
{
    double square = 0.0;
    for (size_t i = 0; i < (size_t)rows * n; ++i) {
        square += want[i] * want[i];
    }
    const double rms = rows == 0u ? 0.0 : std::sqrt(square / ((double)rows * n));
    unsigned int wrong = 0;
    *worst = 0.0;
    for (size_t i = 0; i < (size_t)rows * n; ++i) {
        double scale = std::fabs(want[i]) > rms ? std::fabs(want[i]) : rms;
        double err = std::fabs((double)got[i] - want[i]) / (scale > 0.0 ? scale : 1.0);
        if (!(err <= 1e-2)) {
            wrong += 1;
        }
        if (err > *worst) {
            *worst = err;
        }
    }
    return wrong;
}

static unsigned int count_touched(const std::vector<float> &got, unsigned int first_row, unsigned int rows,
                                  unsigned int n)
{
    unsigned int touched = 0;
    for (size_t i = (size_t)first_row * n; i < (size_t)rows * n; ++i) {
        if (got[i] != kGuard) {
            touched += 1;
        }
    }
    return touched;
}

static void fill_guard(float *y_dev, size_t count, cudaStream_t stream)
{
    std::vector<float> guard(count, kGuard);
    CHECK_CUDA(cudaMemcpyAsync(y_dev, guard.data(), count * sizeof(float), cudaMemcpyHostToDevice, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
}

struct Case {
    unsigned int n, k, m;
};

int main()
{
    aotx_b200_hold hold;
    std::memset(&hold, 0, sizeof(hold));
    aotx_b200_check(aotx_q8_init(&hold.q8, 0), "aotx_q8_init");
    CHECK_CUDA(cudaStreamCreate(&hold.stream));
    Mixer mix{0x243F6A8885A308D3ull};

    // ---- prefill form: the batch is a host number, the call runs directly on the stream.
    // 80 x 128 is the reference's small case (rows of 136 bytes: the any-shape kernel);
    // the others take the tensor-core kernel at one and at several token tiles.
    const Case direct[] = {{80u, 128u, 3u}, {384u, 1024u, 17u}, {640u, 512u, 130u}, {256u, 768u, 300u}};
    for (const Case &c : direct) {
        std::vector<unsigned char> w = make_weights(mix, c.n, c.k);
        std::vector<__half> x = make_input(mix, c.m, c.k);
        void *w_dev = nullptr;
        half *x_dev = nullptr;
        float *y_dev = nullptr;
        const unsigned int rows = c.m + 2u;
        CHECK_CUDA(cudaMalloc(&w_dev, w.size()));
        CHECK_CUDA(cudaMalloc((void **)&x_dev, x.size() * sizeof(__half)));
        CHECK_CUDA(cudaMalloc((void **)&y_dev, (size_t)rows * c.n * sizeof(float)));
        CHECK_CUDA(cudaMemcpy(w_dev, w.data(), w.size(), cudaMemcpyHostToDevice));
        CHECK_CUDA(cudaMemcpy(x_dev, x.data(), x.size() * sizeof(__half), cudaMemcpyHostToDevice));
        fill_guard(y_dev, (size_t)rows * c.n, hold.stream);
        hold.decode = 0u;
        aotx_model_matrix(&hold, w_dev, AOTX_Q8_TYPE_Q8_0, c.n, c.k, x_dev, c.m, y_dev, AOTX_B200_BATCH_TOKENS);
        CHECK_CUDA(cudaStreamSynchronize(hold.stream));
        std::vector<float> got((size_t)rows * c.n);
        CHECK_CUDA(cudaMemcpy(got.data(), y_dev, got.size() * sizeof(float), cudaMemcpyDeviceToHost));
        std::vector<double> want = host_product(w, c.n, c.k, x, c.m);
        double worst = 0.0;
        unsigned int wrong = count_wrong(got, want, c.m, c.n, &worst);
        unsigned int touched = count_touched(got, c.m, rows, c.n);
        std::printf("direct %u x %u, batch %u: wrong %u, worst %.3e, guard rows touched %u\n", c.n, c.k, c.m,
                    wrong, worst, touched);
        if (wrong != 0u || touched != 0u) {
            return 1;
        }
        // a block type without a layout must leave y alone (cuda/model/gemm.cuh:236-237)
        fill_guard(y_dev, (size_t)rows * c.n, hold.stream);
        aotx_model_matrix(&hold, w_dev, 9u /* a block type without a layout */, c.n, c.k, x_dev, c.m, y_dev,
                          AOTX_B200_BATCH_TOKENS);
        CHECK_CUDA(cudaStreamSynchronize(hold.stream));
        CHECK_CUDA(cudaMemcpy(got.data(), y_dev, got.size() * sizeof(float), cudaMemcpyDeviceToHost));
        if (count_touched(got, 0u, rows, c.n) != 0u) {
            std::printf("unknown type wrote to y\n");
            return 1;
        }
        CHECK_CUDA(cudaFree(w_dev));
        CHECK_CUDA(cudaFree(x_dev));
        CHECK_CUDA(cudaFree(y_dev));
    }

    // ---- decode form: one captured graph, the batch is a device word read at run time.
    {
        const unsigned int n = 512u, k = 1024u, m_max = 32u;
        std::vector<unsigned char> w = make_weights(mix, n, k);
        std::vector<__half> x = make_input(mix, m_max, k);
        std::vector<double> want = host_product(w, n, k, x, m_max);
        void *w_dev = nullptr;
        half *x_dev = nullptr;
        float *y_dev = nullptr;
        unsigned int *batch_dev = nullptr;
        CHECK_CUDA(cudaMalloc(&w_dev, w.size()));
        CHECK_CUDA(cudaMalloc((void **)&x_dev, x.size() * sizeof(__half)));
        CHECK_CUDA(cudaMalloc((void **)&y_dev, (size_t)m_max * n * sizeof(float)));
        CHECK_CUDA(cudaMalloc((void **)&batch_dev, 2 * sizeof(unsigned int)));
        CHECK_CUDA(cudaMemcpy(w_dev, w.data(), w.size(), cudaMemcpyHostToDevice));
        CHECK_CUDA(cudaMemcpy(x_dev, x.data(), x.size() * sizeof(__half), cudaMemcpyHostToDevice));
        hold.decode = 1u;
        hold.batch[AOTX_B200_BATCH_TOKENS] = batch_dev;
        hold.batch[AOTX_B200_BATCH_ROWS] = batch_dev + 1;

        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        CHECK_CUDA(cudaStreamBeginCapture(hold.stream, cudaStreamCaptureModeGlobal));
        aotx_model_matrix(&hold, w_dev, AOTX_Q8_TYPE_Q8_0, n, k, x_dev, m_max, y_dev, AOTX_B200_BATCH_TOKENS);
        CHECK_CUDA(cudaStreamEndCapture(hold.stream, &graph));
        CHECK_CUDA(cudaGraphInstantiate(&exec, graph, 0));

        const unsigned int batches[] = {1u, 7u, 32u, 0u, 16u, 40u /* above the captured size: clamps */};
        for (unsigned int live : batches) {
            const unsigned int words[2] = {live, live};
            fill_guard(y_dev, (size_t)m_max * n, hold.stream);
            CHECK_CUDA(cudaMemcpyAsync(batch_dev, words, sizeof(words), cudaMemcpyHostToDevice, hold.stream));
            CHECK_CUDA(cudaGraphLaunch(exec, hold.stream));
            CHECK_CUDA(cudaStreamSynchronize(hold.stream));
            std::vector<float> got((size_t)m_max * n);
            CHECK_CUDA(cudaMemcpy(got.data(), y_dev, got.size() * sizeof(float), cudaMemcpyDeviceToHost));
            const unsigned int rows = live < m_max ? live : m_max;
            double worst = 0.0;
            unsigned int wrong = count_wrong(got, want, rows, n, &worst);
            unsigned int touched = count_touched(got, rows, m_max, n);
            std::printf("captured %u x %u, live batch %u: wrong %u, worst %.3e, rows past the batch touched %u\n",
                        n, k, live, wrong, worst, touched);
            if (wrong != 0u || touched != 0u) {
                return 1;
            }
        }
        CHECK_CUDA(cudaGraphExecDestroy(exec));
        CHECK_CUDA(cudaGraphDestroy(graph));
        CHECK_CUDA(cudaFree(w_dev));
        CHECK_CUDA(cudaFree(x_dev));
        CHECK_CUDA(cudaFree(y_dev));
        CHECK_CUDA(cudaFree(batch_dev));
    }

    uint32_t status = 0;
    aotx_b200_check(aotx_q8_device_status(hold.q8, &status, 0), "aotx_q8_device_status");
    CHECK_CUDA(cudaStreamDestroy(hold.stream));
    aotx_q8_destroy(hold.q8);
    std::printf("pass\n");
    return 0;
}
