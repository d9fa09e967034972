// Driver of the tile-pruned encoder layer: the workload of the reference's encoder_tile_test
// (test/tile_test.cu:9-42), with the same four positional arguments, seeded inputs, a result check and timing.
#include "common.h"

int main(int argc, char** argv) {
    DriverArgs a;
    if (!parse_args(argc, argv, a)) return -1;
    et_test::weight_std() = 0.02f;
    et_test::bernoulli() = true;
    const int tokens = a.batch * a.seq_len, d = a.d_model;
    auto q = gen_tile_linear(d, d, tokens, a.sparsity);
    auto k = gen_tile_linear(d, d, tokens, a.sparsity);
    auto v = gen_tile_linear(d, d, tokens, a.sparsity);
    auto o = gen_tile_linear(d, d, tokens, a.sparsity);
    auto mlp1 = gen_tile_linear(d, 4 * d, tokens, a.sparsity, true);
    auto mlp2 = gen_tile_linear(4 * d, d, tokens, a.sparsity);
    std::vector<half> mask((size_t)a.seq_len * a.seq_len, __float2half(0.f));
    std::vector<half> gamma(d, __float2half(1.f)), beta(d, __float2half(0.f));
    half* buffer = nullptr;
    cudaChk(cudaMalloc(&buffer, Encoder_tile::buffer_size(d, a.seq_len, a.nhead)));
    Encoder_tile encoder(d, a.seq_len, a.nhead, buffer, std::move(q), std::move(k), std::move(v), std::move(o),
                         std::move(mlp1), std::move(mlp2), gamma.data(), beta.data(), gamma.data(), beta.data(),
                         mask.data());
    half* in = device_input((size_t)tokens * d, 7);
    half* out = nullptr;
    cudaChk(cudaMalloc(&out, (size_t)tokens * d * sizeof(half)));
    void* scratch = nullptr;
    const size_t scratch_bytes = Encoder_base::batch_buffer_size(d, tokens, a.batch, a.seq_len, a.nhead);
    cudaChk(cudaMalloc(&scratch, scratch_bytes));
    std::vector<int> lens(a.batch, a.seq_len);
    if (a.batch == 1) encoder.run(out, in);   // the reference's single-sequence entry, once
    return time_and_report("encoder_tile_test", a, out, [&] {
        encoder.run_batch(out, in, lens.data(), a.batch, scratch, scratch_bytes);
    });
}
