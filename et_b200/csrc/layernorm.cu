// Residual add + LayerNorm, in place: in_out <- LN(in_out + skip) * gamma + beta.
// Replaces kernels/skip_layernorm.cu:4-112 of the reference (both its kernels).
//
// Bandwidth kernel: 6*size bytes per row (read x, read skip, write). One warp owns a row, reads
// it with 16-byte loads into registers, reduces with shuffles only (no shared memory, no block
// barrier), does all arithmetic in fp32 (sum, two-pass variance, eps 1e-6 as the reference) and
// writes 16 bytes per lane. gamma/beta are re-read per row through the read-only cache.
#include "common.h"

namespace et {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

template <int CH>  // 16-byte chunks per lane; covers size <= CH*256
__global__ void __launch_bounds__(256, (CH <= 4 ? 3 : 1)) skip_layernorm_vec(half* __restrict__ in_out,
                                                          const half* __restrict__ skip,
                                                          const half* __restrict__ gamma,
                                                          const half* __restrict__ beta, int num,
                                                          int size) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int nwarp = (gridDim.x * blockDim.x) >> 5;
    const int nchunk = size >> 3;
    const float inv_n = 1.0f / (float)size;
    for (int row = warp; row < num; row += nwarp) {
        uint4* xr = reinterpret_cast<uint4*>(in_out + (size_t)row * size);
        const uint4* sr = reinterpret_cast<const uint4*>(skip + (size_t)row * size);
        uint4 xv[CH], sv[CH];
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const int c = lane + 32 * i;
            if (c < nchunk) {
                xv[i] = xr[c];
                sv[i] = skip ? __ldcs(sr + c) : make_uint4(0u, 0u, 0u, 0u);   // no residual: plain LayerNorm of the row
            }
        }
        float v[CH][8];
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const int c = lane + 32 * i;
            const half2* xh = reinterpret_cast<const half2*>(&xv[i]);
            const half2* sh = reinterpret_cast<const half2*>(&sv[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 a = __half22float2(xh[j]), s = __half22float2(sh[j]);
                v[i][2 * j] = c < nchunk ? a.x + s.x : 0.f;
                v[i][2 * j + 1] = c < nchunk ? a.y + s.y : 0.f;
                sum += v[i][2 * j] + v[i][2 * j + 1];
            }
        }
        const float mean = warp_sum(sum) * inv_n;
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const int c = lane + 32 * i;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float d = v[i][j] - mean;
                sq += c < nchunk ? d * d : 0.f;
            }
        }
        const float rstd = rsqrtf(warp_sum(sq) * inv_n + 1e-6f);
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const int c = lane + 32 * i;
            if (c < nchunk) {
                const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + c);
                const uint4 b = __ldg(reinterpret_cast<const uint4*>(beta) + c);
                const half2* gh = reinterpret_cast<const half2*>(&g);
                const half2* bh = reinterpret_cast<const half2*>(&b);
                uint4 o;
                half2* oh = reinterpret_cast<half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 gg = __half22float2(gh[j]), bb = __half22float2(bh[j]);
                    oh[j] = __floats2half2_rn((v[i][2 * j] - mean) * rstd * gg.x + bb.x,
                                              (v[i][2 * j + 1] - mean) * rstd * gg.y + bb.y);
                }
                xr[c] = o;
            }
        }
    }
}

// Any even size, any alignment of 4 bytes: one warp per row, three passes over the row.
__global__ void __launch_bounds__(256) skip_layernorm_generic(half* __restrict__ in_out,
                                                              const half* __restrict__ skip,
                                                              const half* __restrict__ gamma,
                                                              const half* __restrict__ beta,
                                                              int num, int size) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int nwarp = (gridDim.x * blockDim.x) >> 5;
    const float inv_n = 1.0f / (float)size;
    for (int row = warp; row < num; row += nwarp) {
        half* x = in_out + (size_t)row * size;
        const half* s = skip + (size_t)row * size;
        float sum = 0.f;
        for (int i = lane; i < size; i += 32) sum += __half2float(x[i]) + (skip ? __half2float(s[i]) : 0.f);
        const float mean = warp_sum(sum) * inv_n;
        float sq = 0.f;
        for (int i = lane; i < size; i += 32) {
            const float d = __half2float(x[i]) + (skip ? __half2float(s[i]) : 0.f) - mean;
            sq += d * d;
        }
        const float rstd = rsqrtf(warp_sum(sq) * inv_n + 1e-6f);
        for (int i = lane; i < size; i += 32) {
            const float v = __half2float(x[i]) + (skip ? __half2float(s[i]) : 0.f);
            x[i] = __float2half_rn((v - mean) * rstd * __half2float(gamma[i]) +
                                   __half2float(beta[i]));
        }
    }
}

}  // namespace et

namespace et {
// in_out <- LN(in_out + skip) * gamma + beta; skip == nullptr leaves the residual out (the layer stack's last
// LayerNorm when the others are folded into the linears).
int layernorm_launch(half* x, const half* s, const half* g, const half* b, int num, int size, cudaStream_t st);
}

extern "C" int et_skip_layernorm(void* in_out, const void* skip, const void* gamma,
                                 const void* beta, int num, int size, void* stream) {
    ET_REQUIRE(in_out && skip && gamma && beta, "et_skip_layernorm: null pointer");
    ET_REQUIRE(num >= 0 && size > 0, "et_skip_layernorm: bad dimensions");
    return et::layernorm_launch(static_cast<half*>(in_out), static_cast<const half*>(skip), static_cast<const half*>(gamma),
                                static_cast<const half*>(beta), num, size, static_cast<cudaStream_t>(stream));
}

int et::layernorm_launch(half* x, const half* s, const half* g, const half* b, int num, int size, cudaStream_t st) {
    using namespace et;
    if (num == 0) return ET_OK;
    const int warps_needed = num;
    int blocks = (warps_needed + 7) / 8;
    const int cap = sm_count() * 8;  // 8 blocks of 8 warps per SM: the full 64 resident warps
    if (blocks > cap) blocks = cap;
    const bool vec = size % 8 == 0 && size <= 2048 && aligned16(x) && (!s || aligned16(s)) &&
                     aligned16(g) && aligned16(b);
    if (vec) {
        const int ch = (size / 8 + 31) / 32;
        switch (ch) {
            case 1: launch_pdl(skip_layernorm_vec<1>, dim3(blocks), dim3(256), 0, st, x, s, g, b, num, size); break;
            case 2: launch_pdl(skip_layernorm_vec<2>, dim3(blocks), dim3(256), 0, st, x, s, g, b, num, size); break;
            case 3: launch_pdl(skip_layernorm_vec<3>, dim3(blocks), dim3(256), 0, st, x, s, g, b, num, size); break;
            case 4: launch_pdl(skip_layernorm_vec<4>, dim3(blocks), dim3(256), 0, st, x, s, g, b, num, size); break;
            case 5:
            case 6: launch_pdl(skip_layernorm_vec<6>, dim3(blocks), dim3(256), 0, st, x, s, g, b, num, size); break;
            default: launch_pdl(skip_layernorm_vec<8>, dim3(blocks), dim3(256), 0, st, x, s, g, b, num, size); break;
        }
    } else {
        launch_pdl(skip_layernorm_generic, dim3(blocks), dim3(256), 0, st, x, s, g, b, num, size);
    }
    return cuda_status(cudaGetLastError(), "et_skip_layernorm launch");
}
