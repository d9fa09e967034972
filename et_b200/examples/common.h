// Shared pieces of the three example drivers: argument parsing, seeded input, timing.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <encoder/encoder.h>
#include <test/utils.h>

struct DriverArgs {
    int seq_len = 128, nhead = 12, d_model = 768, batch = 1, iters = 20;
    float sparsity = 0.5f;
};

inline bool parse_args(int argc, char** argv, DriverArgs& a) {
    if (argc < 5) {
        std::puts("Usage: ./exec seq_len head_number d_model sparsity [batch] [iterations]");
        return false;
    }
    a.seq_len = std::atoi(argv[1]);
    a.nhead = std::atoi(argv[2]);
    a.d_model = std::atoi(argv[3]);
    a.sparsity = (float)std::atof(argv[4]);
    if (argc > 5) a.batch = std::atoi(argv[5]);
    if (argc > 6) a.iters = std::atoi(argv[6]);
    return a.seq_len > 0 && a.nhead > 0 && a.d_model > 0 && a.d_model % (16 * a.nhead) == 0 && a.batch > 0 &&
           a.iters > 0;
}

inline half* device_input(size_t n, uint64_t seed) {
    std::vector<half> h(n);
    for (auto& v : h) v = __float2half(et_test::gaussian(seed));
    half* d = nullptr;
    cudaChk(cudaMalloc(&d, n * sizeof(half)));
    cudaChk(cudaMemcpy(d, h.data(), n * sizeof(half), cudaMemcpyHostToDevice));
    return d;
}

// Runs `step` a few times untimed, then `iters` times between CUDA events; prints the figures and checks that
// the output is finite.
template <typename Step>
int time_and_report(const char* name, const DriverArgs& a, half* out, Step step) {
    for (int i = 0; i < 3; ++i) step();
    cudaEvent_t e0, e1;
    cudaChk(cudaEventCreate(&e0));
    cudaChk(cudaEventCreate(&e1));
    cudaChk(cudaEventRecord(e0));
    for (int i = 0; i < a.iters; ++i) step();
    cudaChk(cudaEventRecord(e1));
    cudaChk(cudaEventSynchronize(e1));
    float ms = 0.f;
    cudaChk(cudaEventElapsedTime(&ms, e0, e1));
    const size_t n = (size_t)a.batch * a.seq_len * a.d_model;
    std::vector<half> h(n);
    cudaChk(cudaMemcpy(h.data(), out, n * sizeof(half), cudaMemcpyDeviceToHost));
    size_t bad = 0;
    double sum_abs = 0;
    for (auto v : h) {
        const float f = __half2float(v);
        if (!(f == f) || f > 65000.f || f < -65000.f) ++bad;
        sum_abs += f < 0 ? -f : f;
    }
    const double us = 1e3 * ms / a.iters;
    std::printf("%s: seq_len %d heads %d d_model %d sparsity %.2f batch %d: %.1f us/layer, %.0f sequences/s, "
                "mean |out| %.4f, non-finite %zu\n",
                name, a.seq_len, a.nhead, a.d_model, a.sparsity, a.batch, us, a.batch / (us * 1e-6), sum_abs / n, bad);
    return bad == 0 ? 0 : 2;
}
