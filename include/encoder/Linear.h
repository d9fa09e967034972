// Linear_tile and Linear_row with the reference's constructors, public members and run() signatures
// (encoder/Linear.h:4-72), as owners of the C-ABI weight handles of libet_b200.so.
#pragma once
#include <utility>
#include "../kernels/kernels.h"
#include "utils.h"

// 16x16 tile-pruned linear. All pointer arguments of the constructor are HOST pointers and are copied.
class Linear_tile {
    et_tile_weight* handle_ = nullptr;
    int in_feat, out_feat, size;

  public:
    const bool is_gelu;

    Linear_tile(int in_feat_, int out_feat_, int size_, int ntile, half* data_, int* row_ptr_, int* row_offset_,
                half* bias_, bool is_gelu_ = false)
        : in_feat(in_feat_), out_feat(out_feat_), size(size_), is_gelu(is_gelu_) {
        et_shim::require_ok(et_tile_weight_create(&handle_, in_feat_, out_feat_, size_, ntile, data_, row_ptr_,
                                                  row_offset_, bias_),
                            "Linear_tile");
    }
    Linear_tile(const Linear_tile&) = delete;
    Linear_tile& operator=(const Linear_tile&) = delete;
    Linear_tile(Linear_tile&& other) noexcept
        : handle_(other.handle_), in_feat(other.in_feat), out_feat(other.out_feat), size(other.size),
          is_gelu(other.is_gelu) {
        other.handle_ = nullptr;
    }
    ~Linear_tile() { et_tile_weight_destroy(handle_); }

    void run(half* out, half* in, cudaStream_t stream) {
        et_shim::require_ok(et_tile_linear(handle_, out, in, size, is_gelu ? 1 : 0, et_shim::stream_of(stream)), "Linear_tile::run");
    }
    // Extension: any token count (packed batch).
    void run(half* out, half* in, int tokens, cudaStream_t stream) {
        et_shim::require_ok(et_tile_linear(handle_, out, in, tokens, is_gelu ? 1 : 0, et_shim::stream_of(stream)), "Linear_tile::run");
    }
    et_tile_weight* handle() { return handle_; }
};

// Row-pruned linear: only the output features listed in row_id are kept.
class Linear_row {
    et_row_weight* handle_ = nullptr;

  public:
    // Device-side views of the index arrays, with the get() the reference's encoder calls on them.
    struct DeviceInts {
        int* ptr = nullptr;
        int* get() const { return ptr; }
    };
    int in_feat, out_feat, size, nhead;
    DeviceInts row_id;    // sorted kept rows (device)
    DeviceInts head_ptr;  // nhead+1 prefix counts (device)
    int nrow = 0;         // kept rows rounded up to 16: the output pitch
    int row_id_size = 0;

    Linear_row(int in_feat_, int out_feat_, int size_, half* weight_, int* row_id_, int row_id_size_, half* bias_,
               int nhead_)
        : in_feat(in_feat_), out_feat(out_feat_), size(size_), nhead(nhead_) {
        et_shim::require_ok(et_row_weight_create(&handle_, in_feat_, out_feat_, size_, weight_, row_id_,
                                                 row_id_size_, bias_, nhead_),
                            "Linear_row");
        const int *rid = nullptr, *hp = nullptr;
        et_shim::require_ok(et_row_weight_meta(handle_, &nrow, &row_id_size, &rid, &hp, nullptr), "Linear_row");
        row_id.ptr = const_cast<int*>(rid);
        head_ptr.ptr = const_cast<int*>(hp);
    }
    Linear_row(const Linear_row&) = delete;
    Linear_row& operator=(const Linear_row&) = delete;
    Linear_row(Linear_row&& other) noexcept
        : handle_(other.handle_), in_feat(other.in_feat), out_feat(other.out_feat), size(other.size),
          nhead(other.nhead), row_id(other.row_id), head_ptr(other.head_ptr), nrow(other.nrow),
          row_id_size(other.row_id_size) {
        other.handle_ = nullptr;
    }
    ~Linear_row() { et_row_weight_destroy(handle_); }

    // The handle selects nothing here (no cuBLAS); the work goes to the default stream.
    void run(half* out, half* in, cublasHandle_t /*handle*/) {
        et_shim::require_ok(et_row_linear(handle_, out, in, size, et_shim::stream_of(nullptr)), "Linear_row::run");
    }
    void run(half* out, half* in, int tokens, cudaStream_t stream) {
        et_shim::require_ok(et_row_linear(handle_, out, in, tokens, et_shim::stream_of(stream)), "Linear_row::run");
    }
    et_row_weight* handle() { return handle_; }
};
