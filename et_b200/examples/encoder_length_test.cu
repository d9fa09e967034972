// Driver of the sequence-aware encoder: the workload of the reference's encoder_length_test
// (test/length_test.cu:9-39). `seq_len` is the maximum length; with batch > 1 the lengths are drawn uniformly
// from [32, seq_len] with a seed and the batch runs packed (no padding), then padded to seq_len for comparison.
#include "common.h"

int main(int argc, char** argv) {
    DriverArgs a;
    if (!parse_args(argc, argv, a)) return -1;
    et_test::weight_std() = 0.02f;
    et_test::bernoulli() = true;
    const int d = a.d_model;
    std::vector<int> lens(a.batch, a.seq_len);
    uint64_t s = 99;
    if (a.batch > 1)
        for (auto& l : lens) {
            s += 0x9e3779b97f4a7c15ull;
            uint64_t z = (s ^ (s >> 30)) * 0xbf58476d1ce4e5b9ull;
            const int lo = a.seq_len < 32 ? 1 : 32;
            l = lo + (int)((z >> 33) % (uint64_t)(a.seq_len - lo + 1));
        }
    int tokens = 0;
    for (int l : lens) tokens += l;
    const int padded = a.batch * a.seq_len;
    auto q = gen_tile_linear(d, d, tokens, a.sparsity);
    auto k = gen_tile_linear(d, d, tokens, a.sparsity);
    auto v = gen_tile_linear(d, d, tokens, a.sparsity);
    auto o = gen_tile_linear(d, d, tokens, a.sparsity);
    auto mlp1 = gen_tile_linear(d, 4 * d, tokens, a.sparsity, true);
    auto mlp2 = gen_tile_linear(4 * d, d, tokens, a.sparsity);
    std::vector<half> gamma(d, __float2half(1.f)), beta(d, __float2half(0.f));
    Encoder_length encoder(d, a.seq_len, a.nhead, nullptr, std::move(q), std::move(k), std::move(v), std::move(o),
                           std::move(mlp1), std::move(mlp2), gamma.data(), beta.data(), gamma.data(), beta.data(),
                           nullptr);
    half* in = device_input((size_t)padded * d, 7);
    half* out = nullptr;
    cudaChk(cudaMalloc(&out, (size_t)padded * d * sizeof(half)));
    void* scratch = nullptr;
    const size_t scratch_bytes = et_encoder_batch_buffer_size(2, d, padded, a.batch, a.seq_len, a.nhead);
    cudaChk(cudaMalloc(&scratch, scratch_bytes));
    DriverArgs packed = a;
    std::printf("lengths: %d sequences, %d tokens packed, %d padded\n", a.batch, tokens, padded);
    // report() reads batch*seq_len*d_model values: for the packed run only `tokens` rows are written, the rest
    // of `out` is cleared first so the check stays meaningful
    cudaChk(cudaMemset(out, 0, (size_t)padded * d * sizeof(half)));
    int rc = time_and_report("encoder_length_test (packed, length-driven)", packed, out, [&] {
        encoder.run_batch(out, in, lens.data(), a.batch, scratch, scratch_bytes);
    });
    std::vector<int> full(a.batch, a.seq_len);
    rc |= time_and_report("encoder_length_test (padded to seq_len, key padding)", a, out, [&] {
        encoder.run_batch(out, in, full.data(), a.batch, scratch, scratch_bytes, nullptr, lens.data());
    });
    return rc;
}
