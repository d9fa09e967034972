// Encoder_base / Encoder_tile / Encoder_prune / Encoder_length with the reference's constructor and run()
// signatures (encoder/encoder.h:7-134) over the C-ABI encoder handle of libet_b200.so.
// LayerNorm vectors and the mask are HOST pointers (copied); `buffer` is a DEVICE scratch owned by the caller
// of at least buffer_size(...) bytes; the linears are consumed (moved from).
#pragma once
#include <cstddef>
#include <vector>
#include "Linear.h"
#include "utils.h"

class Encoder_base {
  public:
    static constexpr int buffer_num = 5;

  protected:
    et_encoder* enc_ = nullptr;
    int d_model, seq_len, nheads;

    Encoder_base(int d_model_, int seq_len_, int nheads_) : d_model(d_model_), seq_len(seq_len_), nheads(nheads_) {}

  public:
    Encoder_base(const Encoder_base&) = delete;
    Encoder_base& operator=(const Encoder_base&) = delete;
    virtual ~Encoder_base() { et_encoder_destroy(enc_); }
    et_encoder* handle() { return enc_; }

    // One sequence of seq_len tokens; out may alias in. Runs on the default stream without host synchronisation.
    virtual void run(half* out, half* in) {
        et_shim::require_ok(et_encoder_run(enc_, out, in, et_shim::stream_of(nullptr)), "Encoder::run");
    }
    // Extension: `batch` packed sequences of seq_lens[b] tokens each (host array); scratch is a device buffer
    // of batch_buffer_size(...) bytes.
    void run_batch(half* out, half* in, const int* seq_lens, int batch, void* scratch, size_t scratch_bytes,
                   cudaStream_t stream = nullptr, const int* valid_lens = nullptr) {
        et_shim::require_ok(et_encoder_run_batch(enc_, out, in, seq_lens, valid_lens, batch, scratch, scratch_bytes,
                                                 et_shim::stream_of(stream)),
                            "Encoder::run_batch");
    }
    static size_t buffer_size(int d_model_, int seq_len_, int nheads_) {
        return et_encoder_buffer_size(0, d_model_, seq_len_, nheads_);
    }
    static size_t batch_buffer_size(int d_model_, int total_tokens, int batch, int max_len, int nheads_) {
        return et_encoder_batch_buffer_size(0, d_model_, total_tokens, batch, max_len, nheads_);
    }
};

class Encoder_tile : public Encoder_base {
  public:
    Encoder_tile(int d_model_, int seq_len_, int nheads_, half* buffer_, Linear_tile&& Q_linear_,
                 Linear_tile&& K_linear_, Linear_tile&& V_linear_, Linear_tile&& O_linear_,
                 Linear_tile&& MLP1_linear_, Linear_tile&& MLP2_linear_, half* ln_gamma_1, half* ln_beta_1,
                 half* ln_gamma_2, half* ln_beta_2, half* mask_)
        : Encoder_base(d_model_, seq_len_, nheads_) {
        assert(MLP1_linear_.is_gelu);
        et_shim::require_ok(et_encoder_tile_create(&enc_, 0, d_model_, seq_len_, nheads_, buffer_, Q_linear_.handle(),
                                                   K_linear_.handle(), V_linear_.handle(), O_linear_.handle(),
                                                   MLP1_linear_.handle(), MLP2_linear_.handle(), ln_gamma_1,
                                                   ln_beta_1, ln_gamma_2, ln_beta_2, mask_),
                            "Encoder_tile");
    }
};

class Encoder_prune : public Encoder_base {
  public:
    // The reference's form: only V is row-pruned.
    Encoder_prune(int d_model_, int seq_len_, int nheads_, half* buffer_, Linear_tile&& Q_linear_,
                  Linear_tile&& K_linear_, Linear_row&& V_linear_, Linear_tile&& O_linear_,
                  Linear_tile&& MLP1_linear_, Linear_tile&& MLP2_linear_, half* ln_gamma_1, half* ln_beta_1,
                  half* ln_gamma_2, half* ln_beta_2, half* mask_)
        : Encoder_base(d_model_, seq_len_, nheads_) {
        assert(MLP1_linear_.is_gelu);
        et_shim::require_ok(et_encoder_prune_create(&enc_, d_model_, seq_len_, nheads_, buffer_, Q_linear_.handle(),
                                                    K_linear_.handle(), V_linear_.handle(), O_linear_.handle(),
                                                    MLP1_linear_.handle(), MLP2_linear_.handle(), ln_gamma_1,
                                                    ln_beta_1, ln_gamma_2, ln_beta_2, mask_),
                            "Encoder_prune");
    }
    // Extension: Q, K and V row-pruned; Q and K must keep the same rows.
    Encoder_prune(int d_model_, int seq_len_, int nheads_, half* buffer_, Linear_row&& Q_linear_,
                  Linear_row&& K_linear_, Linear_row&& V_linear_, Linear_tile&& O_linear_,
                  Linear_tile&& MLP1_linear_, Linear_tile&& MLP2_linear_, half* ln_gamma_1, half* ln_beta_1,
                  half* ln_gamma_2, half* ln_beta_2, half* mask_)
        : Encoder_base(d_model_, seq_len_, nheads_) {
        assert(MLP1_linear_.is_gelu);
        et_shim::require_ok(et_encoder_prune_qkv_create(&enc_, d_model_, seq_len_, nheads_, buffer_,
                                                        Q_linear_.handle(), K_linear_.handle(), V_linear_.handle(),
                                                        O_linear_.handle(), MLP1_linear_.handle(),
                                                        MLP2_linear_.handle(), ln_gamma_1, ln_beta_1, ln_gamma_2,
                                                        ln_beta_2, mask_),
                            "Encoder_prune");
    }
};

class Encoder_length : public Encoder_base {
  public:
    Encoder_length(int d_model_, int seq_len_, int nheads_, half* buffer_, Linear_tile&& Q_linear_,
                   Linear_tile&& K_linear_, Linear_tile&& V_linear_, Linear_tile&& O_linear_,
                   Linear_tile&& MLP1_linear_, Linear_tile&& MLP2_linear_, half* ln_gamma_1, half* ln_beta_1,
                   half* ln_gamma_2, half* ln_beta_2, half* mask_)
        : Encoder_base(d_model_, seq_len_, nheads_) {
        assert(MLP1_linear_.is_gelu);
        et_shim::require_ok(et_encoder_tile_create(&enc_, 2, d_model_, seq_len_, nheads_, buffer_, Q_linear_.handle(),
                                                   K_linear_.handle(), V_linear_.handle(), O_linear_.handle(),
                                                   MLP1_linear_.handle(), MLP2_linear_.handle(), ln_gamma_1,
                                                   ln_beta_1, ln_gamma_2, ln_beta_2, mask_),
                            "Encoder_length");
    }
    // Scores materialised in HBM (the reference's structure) instead of the default on-the-fly attention.
    void materialize_scores(bool on) {
        et_shim::require_ok(et_encoder_set_materialize_scores(enc_, on ? 1 : 0), "Encoder_length");
    }
    static size_t buffer_size(int d_model_, int seq_len_, int nheads_) {
        return et_encoder_buffer_size(2, d_model_, seq_len_, nheads_);
    }
};

// Extension (no counterpart in the reference, whose callers run one layer object once, test/tile_test.cu:36-41):
// a stack of layers run back to back on packed tokens with model-owned scratch, replayed as one CUDA graph.
// The layers are consumed: after add() the encoder object is an empty shell and must not be run.
class Encoder_stack {
    et_model* model_ = nullptr;
    std::vector<et_encoder*> pending_;

  public:
    Encoder_stack() = default;
    Encoder_stack(const Encoder_stack&) = delete;
    Encoder_stack& operator=(const Encoder_stack&) = delete;
    ~Encoder_stack() { et_model_destroy(model_); }

    // Layers in order; call before the first run_batch().
    void add(Encoder_base& layer) { pending_.push_back(layer.handle()); }

    void run_batch(half* out, half* in, const int* seq_lens, int batch, cudaStream_t stream = nullptr,
                   const int* valid_lens = nullptr) {
        if (!model_) et_shim::require_ok(et_model_create(&model_, pending_.data(), (int)pending_.size()), "Encoder_stack");
        et_shim::require_ok(et_model_run_batch(model_, out, in, seq_lens, valid_lens, batch, et_shim::stream_of(stream)),
                            "Encoder_stack::run_batch");
    }
    void reserve(int total_tokens, int batch, int max_len) {
        if (!model_) et_shim::require_ok(et_model_create(&model_, pending_.data(), (int)pending_.size()), "Encoder_stack");
        et_shim::require_ok(et_model_reserve(model_, total_tokens, batch, max_len), "Encoder_stack::reserve");
    }
};
