// Fused additive mask + row softmax over attention score matrices, in place.
// Replaces the mask/softmax half of kernels/attention.cu:273-323 (scores read from HBM) and
// the device function kernels/attention.cu:10-48 of the reference.
//
// Bandwidth kernel: 4*L*L bytes per score matrix (fp16 read + write); the [L x L] mask is
// shared by every matrix and stays in L2. One warp per row, 16-byte accesses, the row held in
// registers, fp32 max / sum, true row max (a fully masked row yields zeros), ex2 with log2(e)
// folded into the argument. Keys at index >= valid_len are excluded and written as zero.
#include "common.h"

namespace et {

// 2^x on the special-function unit; inputs here are <= 0 or -inf, results flush to zero below 2^-126.
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int CH, int R>  // CH 16-byte chunks per lane (L <= CH*256); R rows per warp and iteration
__global__ void __launch_bounds__(256) softmax_mask_vec(half* __restrict__ scores,
                                                        const half* __restrict__ mask, long nrow,
                                                        int L, int valid) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long nwarp = ((long)gridDim.x * blockDim.x) >> 5;
    const int nchunk = L >> 3;
    constexpr float kLog2e = 1.4426950408889634f;
    for (long row0 = warp * R; row0 < nrow; row0 += nwarp * R) {
        uint4 sv[R][CH], mv[R][CH];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const long row = row0 + r;
            const uint4* sr = reinterpret_cast<const uint4*>(scores + row * L);
            const uint4* mr = mask ? reinterpret_cast<const uint4*>(mask + (size_t)(row % L) * L) : nullptr;
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                const int c = lane + 32 * i;
                sv[r][i] = make_uint4(0, 0, 0, 0);
                mv[r][i] = make_uint4(0, 0, 0, 0);
                if (row < nrow && c < nchunk) {
                    sv[r][i] = __ldcs(sr + c);
                    if (mr) mv[r][i] = __ldg(mr + c);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const long row = row0 + r;
            float v[CH][8];
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                const int c = lane + 32 * i;
                const half2* sh = reinterpret_cast<const half2*>(&sv[r][i]);
                const half2* mh = reinterpret_cast<const half2*>(&mv[r][i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 a = __half22float2(sh[j]), m = __half22float2(mh[j]);
                    const int k = c * 8 + 2 * j;
                    v[i][2 * j] = (c < nchunk && k < valid) ? a.x + m.x : -INFINITY;
                    v[i][2 * j + 1] = (c < nchunk && k + 1 < valid) ? a.y + m.y : -INFINITY;
                    mx = fmaxf(mx, fmaxf(v[i][2 * j], v[i][2 * j + 1]));
                }
            }
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
            const float shift = (mx == -INFINITY) ? 0.f : mx * kLog2e;
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < CH; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[i][j] = ex2_fast(v[i][j] * kLog2e - shift);
                    sum += v[i][j];
                }
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
            const float inv = sum > 0.f ? 1.0f / sum : 0.f;
            if (row < nrow) {
                uint4* sw = reinterpret_cast<uint4*>(scores + row * L);
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    const int c = lane + 32 * i;
                    if (c < nchunk) {
                        uint4 o;
                        half2* oh = reinterpret_cast<half2*>(&o);
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            oh[j] = __floats2half2_rn(v[i][2 * j] * inv, v[i][2 * j + 1] * inv);
                        __stcs(sw + c, o);
                    }
                }
            }
        }
    }
}

// Any L and alignment: one warp per row, three passes.
__global__ void __launch_bounds__(256) softmax_mask_generic(half* __restrict__ scores,
                                                            const half* __restrict__ mask,
                                                            long nrow, int L, int valid) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long nwarp = ((long)gridDim.x * blockDim.x) >> 5;
    constexpr float kLog2e = 1.4426950408889634f;
    for (long row = warp; row < nrow; row += nwarp) {
        half* s = scores + row * L;
        const half* m = mask ? mask + (size_t)(row % L) * L : nullptr;
        float mx = -INFINITY;
        for (int k = lane; k < valid; k += 32)
            mx = fmaxf(mx, __half2float(s[k]) + (m ? __half2float(m[k]) : 0.f));
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float shift = (mx == -INFINITY) ? 0.f : mx * kLog2e;
        float sum = 0.f;
        for (int k = lane; k < valid; k += 32)
            sum += exp2f((__half2float(s[k]) + (m ? __half2float(m[k]) : 0.f)) * kLog2e - shift);
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float inv = sum > 0.f ? 1.0f / sum : 0.f;
        for (int k = lane; k < L; k += 32) {
            float p = 0.f;
            if (k < valid)
                p = exp2f((__half2float(s[k]) + (m ? __half2float(m[k]) : 0.f)) * kLog2e - shift) *
                    inv;
            s[k] = __float2half_rn(p);
        }
    }
}

}  // namespace et

extern "C" int et_softmax_mask(void* scores, const void* mask, int nmat, int seq_len,
                               int valid_len, void* stream) {
    using namespace et;
    ET_REQUIRE(scores, "et_softmax_mask: null scores");
    ET_REQUIRE(nmat >= 0 && seq_len > 0, "et_softmax_mask: bad dimensions");
    ET_REQUIRE(valid_len >= 0 && valid_len <= seq_len, "et_softmax_mask: valid_len out of range");
    if (nmat == 0) return ET_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    half* s = static_cast<half*>(scores);
    const half* m = static_cast<const half*>(mask);
    const long nrow = (long)nmat * seq_len;
    long blocks = (nrow + 15) / 16;          // 8 warps per block, 2 rows per warp and iteration
    const long cap = (long)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    const bool vec = seq_len % 8 == 0 && seq_len <= 2048 && aligned16(s) && (!m || aligned16(m));
    if (vec) {
        const int ch = (seq_len / 8 + 31) / 32;
        switch (ch) {
            case 1: launch_pdl(softmax_mask_vec<1, 2>, dim3((unsigned)blocks), dim3(256), 0, st, s, m, nrow, seq_len, valid_len); break;
            case 2: launch_pdl(softmax_mask_vec<2, 2>, dim3((unsigned)blocks), dim3(256), 0, st, s, m, nrow, seq_len, valid_len); break;
            case 3:
            case 4: launch_pdl(softmax_mask_vec<4, 2>, dim3((unsigned)blocks), dim3(256), 0, st, s, m, nrow, seq_len, valid_len); break;
            default: launch_pdl(softmax_mask_vec<8, 1>, dim3((unsigned)blocks), dim3(256), 0, st, s, m, nrow, seq_len, valid_len); break;
        }
    } else {
        launch_pdl(softmax_mask_generic, dim3((unsigned)blocks), dim3(256), 0, st, s, m, nrow, seq_len, valid_len);
    }
    return cuda_status(cudaGetLastError(), "et_softmax_mask launch");
}
