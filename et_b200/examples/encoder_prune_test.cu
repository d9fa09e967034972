// Driver of the attention-aware pruned encoder layer: the workload of the reference's encoder_prune_test
// (test/prune_test.cu:9-40). Q, K, V are row-pruned at `sparsity` (Q and K keep the same rows; pass a 7th
// argument "v" to prune only V as the reference's constructor does); the FFN and output linears are
// tile-pruned at 0.75.
#include <cstring>
#include "common.h"

int main(int argc, char** argv) {
    DriverArgs a;
    if (!parse_args(argc, argv, a)) return -1;
    const bool v_only = argc > 7 && std::strcmp(argv[7], "v") == 0;
    et_test::weight_std() = 0.02f;
    et_test::bernoulli() = true;
    const int tokens = a.batch * a.seq_len, d = a.d_model;
    const float ffn_sparsity = 0.75f;
    auto o = gen_tile_linear(d, d, tokens, ffn_sparsity);
    auto mlp1 = gen_tile_linear(d, 4 * d, tokens, ffn_sparsity, true);
    auto mlp2 = gen_tile_linear(4 * d, d, tokens, ffn_sparsity);
    std::vector<half> mask((size_t)a.seq_len * a.seq_len, __float2half(0.f));
    std::vector<half> gamma(d, __float2half(1.f)), beta(d, __float2half(0.f));
    Encoder_prune* encoder = nullptr;
    if (v_only) {
        auto q = gen_tile_linear(d, d, tokens, ffn_sparsity);
        auto k = gen_tile_linear(d, d, tokens, ffn_sparsity);
        auto v = gen_row_linear(d, d, tokens, a.sparsity, a.nhead);
        encoder = new Encoder_prune(d, a.seq_len, a.nhead, nullptr, std::move(q), std::move(k), std::move(v),
                                    std::move(o), std::move(mlp1), std::move(mlp2), gamma.data(), beta.data(),
                                    gamma.data(), beta.data(), mask.data());
    } else {
        const uint64_t row_seed = et_test::seed();
        auto q = gen_row_linear(d, d, tokens, a.sparsity, a.nhead);
        et_test::seed() = row_seed;            // K keeps the rows Q keeps
        auto k = gen_row_linear(d, d, tokens, a.sparsity, a.nhead);
        auto v = gen_row_linear(d, d, tokens, a.sparsity, a.nhead);
        encoder = new Encoder_prune(d, a.seq_len, a.nhead, nullptr, std::move(q), std::move(k), std::move(v),
                                    std::move(o), std::move(mlp1), std::move(mlp2), gamma.data(), beta.data(),
                                    gamma.data(), beta.data(), mask.data());
    }
    half* in = device_input((size_t)tokens * d, 7);
    half* out = nullptr;
    cudaChk(cudaMalloc(&out, (size_t)tokens * d * sizeof(half)));
    void* scratch = nullptr;
    const size_t scratch_bytes = Encoder_base::batch_buffer_size(d, tokens, a.batch, a.seq_len, a.nhead);
    cudaChk(cudaMalloc(&scratch, scratch_bytes));
    std::vector<int> lens(a.batch, a.seq_len);
    const int rc = time_and_report(v_only ? "encoder_prune_test (V pruned)" : "encoder_prune_test (Q,K,V pruned)", a, out,
                                   [&] { encoder->run_batch(out, in, lens.data(), a.batch, scratch, scratch_bytes); });
    delete encoder;
    return rc;
}
