// Compact row-pruned activations back to their original feature positions, zeros where a feature was pruned.
//
// The row-pruned linears (encoder/Linear.h:48-72 of the reference) produce only the retained output features, packed
// side by side; the reference's pruned attention kernel (kernels/attention.cu:149-271) gathers each head's retained
// columns 16 at a time and means to scatter its result back to the original columns. A head's window of retained
// columns starts at an arbitrary element offset, which no 16-byte copy and no TMA box can address, and a zero-padded
// 64-wide head is exactly what attention over the retained dimensions needs: a zero column adds nothing to Q K^T,
// and a zero column of V gives a zero column of the result, which is the scatter with zero fill. So the encoder
// expands Q, K and V once (one bandwidth-bound pass, a few microseconds) and runs the tensor-core attention kernel
// on the expanded operands.
#include "attention.h"
#include "common.h"

namespace et {

namespace {

struct ExpandParams {
    const half* src[3];
    half* dst[3];
    const int* inv[3];    // per operand: inv[p] = compact column holding original feature p, or -1
    int src_pitch[3], dst_pitch[3];
    int n, d, T;
};

// One warp per token and operand pass: every lane builds eight consecutive output features from scalar reads of
// the token's compact row (a few hundred bytes, served by L1) and writes them as one 16-byte store.
__global__ void __launch_bounds__(256) expand_rows_kernel(const ExpandParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = (blockDim.x >> 5) * gridDim.x;
    for (int t = blockIdx.x * (blockDim.x >> 5) + warp; t < p.T; t += warps) {
#pragma unroll
        for (int o = 0; o < 3; ++o) {
            if (o >= p.n) break;
            const half* __restrict__ src = p.src[o] + (size_t)t * p.src_pitch[o];
            half* __restrict__ dst = p.dst[o] + (size_t)t * p.dst_pitch[o];
            const int* __restrict__ inv = p.inv[o];
            for (int c = lane * 8; c < p.d; c += 256) {
                const int4 i0 = __ldg(reinterpret_cast<const int4*>(inv + c));
                const int4 i1 = __ldg(reinterpret_cast<const int4*>(inv + c) + 1);
                const int idx[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
                __align__(16) half v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = idx[j] >= 0 ? src[idx[j]] : __float2half(0.f);
                *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(v);
            }
        }
    }
}

}  // namespace

// dst[o][t][p] = inv[o][p] >= 0 ? src[o][t][inv[o][p]] : 0 for up to three operands in one launch. d must be a
// multiple of 8, destinations 16-byte aligned with pitches that are multiples of 8.
int expand_rows_launch(int n, const half* const* src, const int* src_pitch, half* const* dst, const int* dst_pitch,
                       const int* const* inv, int d, int T, cudaStream_t st) {
    if (n < 1 || n > 3 || d <= 0 || (d & 7)) return fail(ET_ERR_INVALID, "expand rows: bad arguments");
    if (T <= 0) return ET_OK;
    ExpandParams p;
    p.n = n; p.d = d; p.T = T;
    for (int o = 0; o < 3; ++o) {
        const int k = o < n ? o : 0;
        if (!src[k] || !dst[k] || !inv[k]) return fail(ET_ERR_INVALID, "expand rows: null pointer");
        if (!aligned16(dst[k]) || (dst_pitch[k] & 7)) return fail(ET_ERR_INVALID, "expand rows: destination must be 16-byte aligned");
        p.src[o] = src[k]; p.dst[o] = dst[k]; p.inv[o] = inv[k];
        p.src_pitch[o] = src_pitch[k]; p.dst_pitch[o] = dst_pitch[k];
    }
    const int blocks = std::min((T + 7) / 8, sm_count() * 8);
    return cuda_status(launch_pdl(expand_rows_kernel, dim3(blocks), dim3(256), 0, st, p), "expand rows launch");
}

}  // namespace et
