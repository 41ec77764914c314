// Softmax over one dimension and its backward: the step between S = Q.K^T and S.V in the
// attention-shaped use of the batched GEMM (ops/norm.rs:52-89, :125-163; kernels/softmax.cu).
// HBM-bound: the forward reads x once and writes out once (8 bytes per element), the backward reads
// dy and out once and writes dx once (12 bytes per element).  A row that fits a warp's registers
// (<= 2048 elements, length a multiple of 4) never leaves them between the max, the sum and the
// division; other shapes take a block-per-row or a block-per-32-columns loop over the same arithmetic.
#include "internal.h"

#include <algorithm>

namespace mni {

namespace {

constexpr int kRowsPerBlock = 8;   // one warp per row
constexpr float kNegInf = -__builtin_huge_valf();

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// Row in registers: lane l holds float4 chunks l, l+32, ... (CH of them; chunk index < len4 is live).
template <int CH>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
softmax_rows_fwd_kernel(const float4 *__restrict__ x, float4 *__restrict__ out, long long rows, int len4) {
    const long long row = blockIdx.x * static_cast<long long>(kRowsPerBlock) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float4 *xr = x + row * len4;
    float4 v[CH];
    float mx = kNegInf;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = c * 32 + lane;
        if (i < len4) {
            v[c] = __ldcs(xr + i);
            mx = fmaxf(fmaxf(fmaxf(mx, v[c].x), fmaxf(v[c].y, v[c].z)), v[c].w);
        }
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        if (c * 32 + lane < len4) {
            v[c].x = expf(v[c].x - mx); v[c].y = expf(v[c].y - mx);
            v[c].z = expf(v[c].z - mx); v[c].w = expf(v[c].w - mx);
            sum += (v[c].x + v[c].y) + (v[c].z + v[c].w);
        }
    }
    sum = warp_sum(sum);
    float4 *orow = out + row * len4;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = c * 32 + lane;
        if (i < len4) orow[i] = make_float4(v[c].x / sum, v[c].y / sum, v[c].z / sum, v[c].w / sum);
    }
}

template <int CH>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
softmax_rows_bwd_kernel(const float4 *__restrict__ dy, const float4 *__restrict__ out, float4 *__restrict__ dx,
                        long long rows, int len4) {
    const long long row = blockIdx.x * static_cast<long long>(kRowsPerBlock) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float4 *gr = dy + row * len4, *sr = out + row * len4;
    float4 g[CH], s[CH];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = c * 32 + lane;
        if (i < len4) {
            g[c] = __ldcs(gr + i);
            s[c] = __ldcs(sr + i);
            dot += (g[c].x * s[c].x + g[c].y * s[c].y) + (g[c].z * s[c].z + g[c].w * s[c].w);
        }
    }
    dot = warp_sum(dot);
    float4 *drow = dx + row * len4;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = c * 32 + lane;
        if (i < len4)
            drow[i] = make_float4(s[c].x * (g[c].x - dot), s[c].y * (g[c].y - dot), s[c].z * (g[c].z - dot),
                                  s[c].w * (g[c].w - dot));
    }
}

// Any length, any alignment, inner == 1: one block per row, three passes over the row (the second
// and third hit L2 or L1).  Block reductions in a fixed order.
constexpr int kBlockThreads = 256;
__device__ __forceinline__ float block_reduce(float x, bool is_max) {
    __shared__ float ws[kBlockThreads / 32];
    __shared__ float result;
    x = is_max ? warp_max(x) : warp_sum(x);
    __syncthreads();                                 // ws / result may still be read from the last call
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = x;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = ws[0];
        for (int w = 1; w < kBlockThreads / 32; ++w) t = is_max ? fmaxf(t, ws[w]) : t + ws[w];
        result = t;
    }
    __syncthreads();
    return result;
}
__global__ void __launch_bounds__(kBlockThreads)
softmax_long_fwd_kernel(const float *__restrict__ x, float *__restrict__ out, long long len) {
    const float *xr = x + blockIdx.x * len;
    float *orow = out + blockIdx.x * len;
    float mx = kNegInf;
    for (long long i = threadIdx.x; i < len; i += kBlockThreads) mx = fmaxf(mx, xr[i]);
    mx = block_reduce(mx, true);
    float sum = 0.f;
    for (long long i = threadIdx.x; i < len; i += kBlockThreads) {
        const float e = expf(xr[i] - mx);
        orow[i] = e;
        sum += e;
    }
    sum = block_reduce(sum, false);
    for (long long i = threadIdx.x; i < len; i += kBlockThreads) orow[i] /= sum;
}
__global__ void __launch_bounds__(kBlockThreads)
softmax_long_bwd_kernel(const float *__restrict__ dy, const float *__restrict__ out, float *__restrict__ dx,
                        long long len) {
    const float *gr = dy + blockIdx.x * len, *sr = out + blockIdx.x * len;
    float *drow = dx + blockIdx.x * len;
    float dot = 0.f;
    for (long long i = threadIdx.x; i < len; i += kBlockThreads) dot += gr[i] * sr[i];
    dot = block_reduce(dot, false);
    for (long long i = threadIdx.x; i < len; i += kBlockThreads) drow[i] = sr[i] * (gr[i] - dot);
}

// inner > 1 (softmax over a dimension that is not the last): a block owns 32 neighbouring (outer, inner)
// columns, so every access is a coalesced 128-byte line, and its 8 warps split the dimension; the
// per-column max and sums meet in shared memory in warp order.
constexpr int kColWarps = 8;
__device__ __forceinline__ float cols_reduce(float x, bool is_max, float (*sh)[32]) {
    const int cx = threadIdx.x & 31, sg = threadIdx.x >> 5;
    __syncthreads();                                  // sh may still be read from the previous reduce
    sh[sg][cx] = x;
    __syncthreads();
    float t = sh[0][cx];
#pragma unroll
    for (int w = 1; w < kColWarps; ++w) t = is_max ? fmaxf(t, sh[w][cx]) : t + sh[w][cx];
    return t;
}
__global__ void __launch_bounds__(32 * kColWarps)
softmax_cols_fwd_kernel(const float *__restrict__ x, float *__restrict__ out, long long columns, long long dim,
                        long long inner) {
    __shared__ float sh[kColWarps][32];
    const int cx = threadIdx.x & 31, sg = threadIdx.x >> 5;
    const long long c = blockIdx.x * 32LL + cx;
    const bool live = c < columns;
    const long long base = live ? (c / inner) * dim * inner + (c % inner) : 0;
    float mx = kNegInf;
    if (live)
        for (long long s = sg; s < dim; s += kColWarps) mx = fmaxf(mx, x[base + s * inner]);
    mx = cols_reduce(mx, true, sh);
    float sum = 0.f;
    if (live)
        for (long long s = sg; s < dim; s += kColWarps) {
            const float e = expf(x[base + s * inner] - mx);
            out[base + s * inner] = e;
            sum += e;
        }
    sum = cols_reduce(sum, false, sh);
    if (live)
        for (long long s = sg; s < dim; s += kColWarps) out[base + s * inner] /= sum;   // own writes only
}
__global__ void __launch_bounds__(32 * kColWarps)
softmax_cols_bwd_kernel(const float *__restrict__ dy, const float *__restrict__ out, float *__restrict__ dx,
                        long long columns, long long dim, long long inner) {
    __shared__ float sh[kColWarps][32];
    const int cx = threadIdx.x & 31, sg = threadIdx.x >> 5;
    const long long c = blockIdx.x * 32LL + cx;
    const bool live = c < columns;
    const long long base = live ? (c / inner) * dim * inner + (c % inner) : 0;
    float dot = 0.f;
    if (live)
        for (long long s = sg; s < dim; s += kColWarps) dot += dy[base + s * inner] * out[base + s * inner];
    dot = cols_reduce(dot, false, sh);
    if (live)
        for (long long s = sg; s < dim; s += kColWarps)
            dx[base + s * inner] = out[base + s * inner] * (dy[base + s * inner] - dot);
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int chunks_for(long long len) {          // float4 chunks per lane, rounded up to a compiled variant
    const long long need = (len / 4 + 31) / 32;
    for (int ch : {1, 2, 4, 8, 16})
        if (need <= ch) return ch;
    return 0;
}

}  // namespace

int launch_softmax_fwd(const float *x, float *out, int64_t outer, int64_t dim, int64_t inner, cudaStream_t stream) {
    if (outer * dim * inner == 0) return MNI_B200_OK;
    if (inner == 1) {
        const int ch = (dim % 4 == 0 && aligned16(x) && aligned16(out)) ? chunks_for(dim) : 0;
        if (ch) {
            const int len4 = static_cast<int>(dim / 4);
            const unsigned blocks = static_cast<unsigned>((outer + kRowsPerBlock - 1) / kRowsPerBlock);
            const float4 *x4 = reinterpret_cast<const float4 *>(x);
            float4 *o4 = reinterpret_cast<float4 *>(out);
            switch (ch) {
                case 1: softmax_rows_fwd_kernel<1><<<blocks, kRowsPerBlock * 32, 0, stream>>>(x4, o4, outer, len4); break;
                case 2: softmax_rows_fwd_kernel<2><<<blocks, kRowsPerBlock * 32, 0, stream>>>(x4, o4, outer, len4); break;
                case 4: softmax_rows_fwd_kernel<4><<<blocks, kRowsPerBlock * 32, 0, stream>>>(x4, o4, outer, len4); break;
                case 8: softmax_rows_fwd_kernel<8><<<blocks, kRowsPerBlock * 32, 0, stream>>>(x4, o4, outer, len4); break;
                default: softmax_rows_fwd_kernel<16><<<blocks, kRowsPerBlock * 32, 0, stream>>>(x4, o4, outer, len4); break;
            }
            MNI_LAUNCH_CHECK("softmax_rows_fwd");
            return MNI_B200_OK;
        }
        softmax_long_fwd_kernel<<<static_cast<unsigned>(outer), kBlockThreads, 0, stream>>>(x, out, dim);
        MNI_LAUNCH_CHECK("softmax_long_fwd");
        return MNI_B200_OK;
    }
    const long long columns = outer * inner;
    softmax_cols_fwd_kernel<<<static_cast<unsigned>((columns + 31) / 32), 32 * kColWarps, 0, stream>>>(x, out, columns,
                                                                                                  dim, inner);
    MNI_LAUNCH_CHECK("softmax_cols_fwd");
    return MNI_B200_OK;
}

int launch_softmax_bwd(const float *dy, const float *out, float *dx, int64_t outer, int64_t dim, int64_t inner,
                       cudaStream_t stream) {
    if (outer * dim * inner == 0) return MNI_B200_OK;
    if (inner == 1) {
        const int ch = (dim % 4 == 0 && aligned16(dy) && aligned16(out) && aligned16(dx)) ? chunks_for(dim) : 0;
        if (ch && ch <= 8) {              // two rows live in registers here: 1024 elements at most
            const int len4 = static_cast<int>(dim / 4);
            const unsigned blocks = static_cast<unsigned>((outer + kRowsPerBlock - 1) / kRowsPerBlock);
            const float4 *g4 = reinterpret_cast<const float4 *>(dy), *s4 = reinterpret_cast<const float4 *>(out);
            float4 *d4 = reinterpret_cast<float4 *>(dx);
            switch (ch) {
                case 1: softmax_rows_bwd_kernel<1><<<blocks, kRowsPerBlock * 32, 0, stream>>>(g4, s4, d4, outer, len4); break;
                case 2: softmax_rows_bwd_kernel<2><<<blocks, kRowsPerBlock * 32, 0, stream>>>(g4, s4, d4, outer, len4); break;
                case 4: softmax_rows_bwd_kernel<4><<<blocks, kRowsPerBlock * 32, 0, stream>>>(g4, s4, d4, outer, len4); break;
                default: softmax_rows_bwd_kernel<8><<<blocks, kRowsPerBlock * 32, 0, stream>>>(g4, s4, d4, outer, len4); break;
            }
            MNI_LAUNCH_CHECK("softmax_rows_bwd");
            return MNI_B200_OK;
        }
        softmax_long_bwd_kernel<<<static_cast<unsigned>(outer), kBlockThreads, 0, stream>>>(dy, out, dx, dim);
        MNI_LAUNCH_CHECK("softmax_long_bwd");
        return MNI_B200_OK;
    }
    const long long columns = outer * inner;
    softmax_cols_bwd_kernel<<<static_cast<unsigned>((columns + 31) / 32), 32 * kColWarps, 0, stream>>>(dy, out, dx,
                                                                                                  columns, dim, inner);
    MNI_LAUNCH_CHECK("softmax_cols_bwd");
    return MNI_B200_OK;
}

}  // namespace mni
