// extern "C" entry points that are thin adapters over the host-side C++ of this library.
#include "common.h"
#include "handles.h"
#include "tile_gemm.h"


extern "C" int et_tile_weight_create(et_tile_weight** out, int in_feat, int out_feat, int size,
                                     int ntile, const void* data_host, const int* row_ptr_host,
                                     const int* row_offset_host, const void* bias_host) {
    ET_REQUIRE(out, "et_tile_weight_create: null output");
    *out = nullptr;
    et::TileWeight* w = nullptr;
    int rc = et::tile_weight_pack(&w, in_feat, out_feat, size, ntile,
                                  static_cast<const half*>(data_host), row_ptr_host,
                                  row_offset_host, static_cast<const half*>(bias_host), 0);
    if (rc) return rc;
    *out = new et_tile_weight{w};
    return ET_OK;
}
extern "C" int et_tile_weight_destroy(et_tile_weight* w) {
    if (!w) return ET_OK;
    et::tile_weight_free(w->w);
    delete w;
    return ET_OK;
}
extern "C" int et_tile_linear(const et_tile_weight* w, void* Y, const void* X, int tokens, int gelu,
                              void* stream) {
    ET_REQUIRE(w, "et_tile_linear: null weight");
    return et::tile_linear_run(w->w, static_cast<half*>(Y), static_cast<const half*>(X), tokens,
                               gelu, static_cast<cudaStream_t>(stream));
}
extern "C" int et_tile_weight_check(const et_tile_weight* w, int* code) {
    ET_REQUIRE(w && code, "et_tile_weight_check: null pointer");
    int rc = et::tile_weight_error(w->w, code);
    if (rc) return rc;
    if (*code) {
        et::set_error("tile linear: device wait %d gave up", *code);
        return ET_ERR_DEVICE_TIMEOUT;
    }
    return ET_OK;
}
extern "C" int et_tile_weight_info(const et_tile_weight* w, int* info) {
    ET_REQUIRE(w && info, "et_tile_weight_info: null pointer");
    et::tile_weight_info(w->w, info);
    return ET_OK;
}
extern "C" int et_tile_spmm_bias(void* Y, const void* X, const int* W_row_ptr,
                                 const int* W_row_offset, const void* W_data, int M, int N, int K,
                                 const void* bias, int gelu, void* stream) {
    ET_REQUIRE(Y && X, "et_tile_spmm_bias: null pointer");
    return et::tile_spmm_raw(static_cast<half*>(Y), static_cast<const half*>(X), W_row_ptr,
                             W_row_offset, static_cast<const half*>(W_data), M, N, K,
                             static_cast<const half*>(bias), gelu, static_cast<cudaStream_t>(stream));
}
namespace et { void row_spmm_cache_clear(); }
extern "C" int et_tile_spmm_cache_clear(void) {
    et::tile_spmm_cache_clear();
    et::row_spmm_cache_clear();
    return ET_OK;
}

extern "C" int et_set_tuning_goal(int goal) {
    if (goal != 0 && goal != 1) return et::fail(ET_ERR_INVALID, "et_set_tuning_goal: goal must be 0 (latency) or 1 (throughput)");
    et::tile_gemm_set_goal(goal);
    return ET_OK;
}

namespace et { void attention_tc_set_scores_fp32(int on); int attention_tc_scores_fp32(); }
extern "C" int et_set_attention_scores_fp32(int on) {
    if (on != 0 && on != 1) return et::fail(ET_ERR_INVALID, "et_set_attention_scores_fp32: 0 (fp16 scores) or 1 (fp32 scores)");
    et::attention_tc_set_scores_fp32(on);
    return ET_OK;
}
extern "C" int et_attention_scores_fp32(void) { return et::attention_tc_scores_fp32(); }

// Not part of the public header: used by profiling builds of the library only.
extern "C" int et_debug_set_gemm_profile_buffer(void* dev_buf) {
    et::tile_gemm_set_profile_buffer(static_cast<long long*>(dev_buf));
    return ET_OK;
}

namespace et { void attention_tc_set_profile_buffer(long long* dev_buf); }
extern "C" int et_debug_set_attention_profile_buffer(void* dev_buf) {
    et::attention_tc_set_profile_buffer(static_cast<long long*>(dev_buf));
    return ET_OK;
}
