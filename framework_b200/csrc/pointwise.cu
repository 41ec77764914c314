// HBM-bound helpers around the GEMM: bias add, column sums (dbias), device-side
// gather of strided views, device-side unbroadcast, plain copy.
#include "internal.h"

#include <algorithm>

namespace mni {

namespace {

constexpr int kMaxDims = MNI_B200_MAX_DIMS;

int grid_for(long long work_items, int threads) {
    const long long blocks = (work_items + threads - 1) / threads;
    return static_cast<int>(std::max<long long>(1, std::min<long long>(blocks, device_sm_count() * 16LL)));
}

// out[r, j] = y[r, j] + bias[j]; one float4 per thread-iteration when n % 4 == 0.
__global__ void add_bias_vec_kernel(const float4 *__restrict__ y, const float4 *__restrict__ bias,
                                    float4 *__restrict__ out, long long total4, int n4) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total4;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float4 b = __ldg(bias + static_cast<int>(i % n4));
        float4 v = y[i];
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
        out[i] = v;
    }
}
__global__ void add_bias_scalar_kernel(const float *__restrict__ y, const float *__restrict__ bias,
                                       float *__restrict__ out, long long total, long long n) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        out[i] = y[i] + __ldg(bias + i % n);
}

// Column sums, stage 1: block (bx, by) sums rows [by*rows_per, ...) of a 128-column strip
// (32 lanes x float4).  8 warps take interleaved rows and are combined through shared
// memory in a fixed order, so the result does not depend on scheduling.
__global__ void colsum_partial_kernel(const float *__restrict__ dy, long long ld, float *__restrict__ partial,
                                      long long rows, long long n, long long rows_per) {
    __shared__ float4 red[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long col = (static_cast<long long>(blockIdx.x) * 32 + lane) * 4;
    const long long r0 = blockIdx.y * rows_per;
    const long long r1 = min(rows, r0 + rows_per);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const bool vec = ((ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(dy) & 15) == 0) && col + 3 < n;
    if (col < n) {
        long long r = r0 + warp;
        if (vec) {
            // four rows in flight per thread, added in the same ascending order as the one-row loop
            for (; r + 24 < r1; r += 32) {
                float4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = __ldcs(reinterpret_cast<const float4 *>(dy + (r + 8 * u) * ld + col));
#pragma unroll
                for (int u = 0; u < 4; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
            }
        }
        for (; r < r1; r += 8) {
            const float *p = dy + r * ld + col;
            if (vec) {
                const float4 v = __ldg(reinterpret_cast<const float4 *>(p));
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            } else {
                acc.x += __ldg(p);
                if (col + 1 < n) acc.y += __ldg(p + 1);
                if (col + 2 < n) acc.z += __ldg(p + 2);
                if (col + 3 < n) acc.w += __ldg(p + 3);
            }
        }
    }
    red[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && col < n) {
        float4 s = red[0][lane];
        for (int w = 1; w < 8; ++w) {
            s.x += red[w][lane].x; s.y += red[w][lane].y; s.z += red[w][lane].z; s.w += red[w][lane].w;
        }
        float *o = partial + static_cast<long long>(blockIdx.y) * n + col;
        o[0] = s.x;
        if (col + 1 < n) o[1] = s.y;
        if (col + 2 < n) o[2] = s.z;
        if (col + 3 < n) o[3] = s.w;
    }
}
// stage 2: out[j] (+)= sum over slabs, ascending.
__global__ void colsum_final_kernel(const float *__restrict__ partial, float *__restrict__ out, long long n,
                                    int slabs, int accumulate) {
    const long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (j >= n) return;
    float s = partial[j];
    for (int i = 1; i < slabs; ++i) s += partial[static_cast<long long>(i) * n + j];
    out[j] = accumulate ? out[j] + s : s;
}

// ---- bias + GELU (tanh form), the fused pointwise op that follows the MLP up-projection --------
// gelu(v) = 0.5 v (1 + tanh(sqrt(2/pi) (v + 0.044715 v^3))), v = x + bias   (kernels/fused_ops.cu:66-82)
__device__ __forceinline__ float gelu_tanh(float v) {
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(inner));
}
// d gelu / d v                                                             (kernels/fused_ops.cu:96-103)
__device__ __forceinline__ float gelu_tanh_grad(float v) {
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    const float th = tanhf(inner);
    const float sech2 = 1.0f - th * th;
    const float d_inner = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * v * v);
    return 0.5f * (1.0f + th) + 0.5f * v * sech2 * d_inner;
}

__global__ void bias_gelu_vec_kernel(const float4 *__restrict__ x, const float4 *__restrict__ bias,
                                     float4 *__restrict__ out, long long total4, int n4) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total4;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float4 b = __ldg(bias + static_cast<int>(i % n4));
        const float4 v = x[i];
        out[i] = make_float4(gelu_tanh(v.x + b.x), gelu_tanh(v.y + b.y), gelu_tanh(v.z + b.z), gelu_tanh(v.w + b.w));
    }
}
__global__ void bias_gelu_scalar_kernel(const float *__restrict__ x, const float *__restrict__ bias,
                                        float *__restrict__ out, long long total, long long n) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        out[i] = gelu_tanh(x[i] + __ldg(bias + i % n));
}

// Backward, stage 1: dx = grad * gelu'(x + bias) written once, and the column sums of dx over a slab of
// rows (same block shape and fixed summation order as colsum_partial_kernel; no atomics).
__global__ void bias_gelu_bwd_partial_kernel(const float *__restrict__ grad, const float *__restrict__ x,
                                             const float *__restrict__ bias, float *__restrict__ dx,
                                             float *__restrict__ partial, long long rows, long long n,
                                             long long rows_per) {
    __shared__ float4 red[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long col = (static_cast<long long>(blockIdx.x) * 32 + lane) * 4;
    const long long r0 = blockIdx.y * rows_per;
    const long long r1 = min(rows, r0 + rows_per);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const bool vec = ((n & 3) == 0) && col + 3 < n &&
                     (((reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(x) |
                        reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(bias)) & 15) == 0);
    if (col < n) {
        float b[4] = {0.f, 0.f, 0.f, 0.f};
        for (int e = 0; e < 4; ++e)
            if (col + e < n) b[e] = __ldg(bias + col + e);
        for (long long r = r0 + warp; r < r1; r += 8) {
            const long long off = r * n + col;
            if (vec) {
                const float4 g = __ldg(reinterpret_cast<const float4 *>(grad + off));
                const float4 v = __ldg(reinterpret_cast<const float4 *>(x + off));
                float4 d;
                d.x = g.x * gelu_tanh_grad(v.x + b[0]);
                d.y = g.y * gelu_tanh_grad(v.y + b[1]);
                d.z = g.z * gelu_tanh_grad(v.z + b[2]);
                d.w = g.w * gelu_tanh_grad(v.w + b[3]);
                *reinterpret_cast<float4 *>(dx + off) = d;
                acc.x += d.x; acc.y += d.y; acc.z += d.z; acc.w += d.w;
            } else {
                float d[4] = {0.f, 0.f, 0.f, 0.f};
                for (int e = 0; e < 4; ++e) {
                    if (col + e < n) {
                        d[e] = __ldg(grad + off + e) * gelu_tanh_grad(__ldg(x + off + e) + b[e]);
                        dx[off + e] = d[e];
                    }
                }
                acc.x += d[0]; acc.y += d[1]; acc.z += d[2]; acc.w += d[3];
            }
        }
    }
    red[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && col < n) {
        float4 s = red[0][lane];
        for (int w = 1; w < 8; ++w) {
            s.x += red[w][lane].x; s.y += red[w][lane].y; s.z += red[w][lane].z; s.w += red[w][lane].w;
        }
        float *o = partial + static_cast<long long>(blockIdx.y) * n + col;
        o[0] = s.x;
        if (col + 1 < n) o[1] = s.y;
        if (col + 2 < n) o[2] = s.z;
        if (col + 3 < n) o[3] = s.w;
    }
}

// ---- AdamW step: the consumer of the weight gradient (kernels/adamw.cu) -------------------------
// One pass: grad read once, m / v / param read and written once (28 bytes per element).
__device__ __forceinline__ void adamw_one(float &p, float &m, float &v, float g, float lr, float beta1, float beta2,
                                          float eps, float decay, float bc1, float bc2) {
    const float mi = beta1 * m + (1.0f - beta1) * g;
    const float vi = beta2 * v + (1.0f - beta2) * g * g;
    m = mi;
    v = vi;
    p = p * decay - lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
}
// Clip factor of ops/optimizer.rs:232-236: max_norm / norm when the norm (f64 sum of squares, rounded to
// f32, then sqrt) exceeds max_norm, else 1.  The sum of squares is read from device memory, so no
// host round trip sits between the norm and the step.
__device__ __forceinline__ float clip_scale(const double *sumsq, float max_norm) {
    if (sumsq == nullptr || !(max_norm > 0.0f)) return 1.0f;
    const float norm = sqrtf(static_cast<float>(*sumsq));
    return norm > max_norm ? max_norm / norm : 1.0f;
}
__global__ void adamw_vec_kernel(float4 *__restrict__ param, float4 *__restrict__ m, float4 *__restrict__ v,
                                 float4 *__restrict__ grad, long long n4, float lr, float beta1, float beta2,
                                 float eps, float decay, float bc1, float bc2, const double *sumsq, float max_norm,
                                 int write_grad) {
    const float scale = clip_scale(sumsq, max_norm);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float4 p = param[i], mm = m[i], vv = v[i];
        float4 g = __ldcs(grad + i);
        if (scale != 1.0f) {
            g.x *= scale; g.y *= scale; g.z *= scale; g.w *= scale;
            if (write_grad) grad[i] = g;
        }
        adamw_one(p.x, mm.x, vv.x, g.x, lr, beta1, beta2, eps, decay, bc1, bc2);
        adamw_one(p.y, mm.y, vv.y, g.y, lr, beta1, beta2, eps, decay, bc1, bc2);
        adamw_one(p.z, mm.z, vv.z, g.z, lr, beta1, beta2, eps, decay, bc1, bc2);
        adamw_one(p.w, mm.w, vv.w, g.w, lr, beta1, beta2, eps, decay, bc1, bc2);
        param[i] = p; m[i] = mm; v[i] = vv;
    }
}
__global__ void adamw_scalar_kernel(float *__restrict__ param, float *__restrict__ m, float *__restrict__ v,
                                    float *__restrict__ grad, long long n, float lr, float beta1, float beta2,
                                    float eps, float decay, float bc1, float bc2, const double *sumsq, float max_norm,
                                    int write_grad) {
    const float scale = clip_scale(sumsq, max_norm);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float g = grad[i];
        if (scale != 1.0f) {
            g *= scale;
            if (write_grad) grad[i] = g;
        }
        adamw_one(param[i], m[i], v[i], g, lr, beta1, beta2, eps, decay, bc1, bc2);
    }
}

// ---- gradient norm (ops/optimizer.rs:126-138): f64 sum of f32 squares ------------------------------
// Stage 1: a fixed grid, each thread a grid-stride f64 sum, each block a fixed-order tree -> partial[block].
// Stage 2: one block adds the partials in a fixed order.  The grid depends only on n and the SM count,
// so the result is reproducible run to run.
constexpr int kNormThreads = 256;
__device__ __forceinline__ double block_sum_f64(double x) {
    __shared__ double warp_sums[kNormThreads / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_down_sync(0xffffffffu, x, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = x;
    __syncthreads();
    double t = 0.0;
    if (threadIdx.x == 0)
        for (int w = 0; w < kNormThreads / 32; ++w) t += warp_sums[w];
    return t;   // valid in thread 0
}
__global__ void __launch_bounds__(kNormThreads)
sumsq_partial_kernel(const float *__restrict__ g, long long n, double *__restrict__ partial) {
    double acc = 0.0;
    const long long tid = blockIdx.x * static_cast<long long>(kNormThreads) + threadIdx.x;
    const long long nthreads = static_cast<long long>(gridDim.x) * kNormThreads;
    if ((reinterpret_cast<uintptr_t>(g) & 15) == 0) {
        const long long n4 = n / 4;
        const float4 *g4 = reinterpret_cast<const float4 *>(g);
        for (long long i = tid; i < n4; i += nthreads) {
            const float4 t = __ldg(g4 + i);
            acc += static_cast<double>(t.x) * t.x;
            acc += static_cast<double>(t.y) * t.y;
            acc += static_cast<double>(t.z) * t.z;
            acc += static_cast<double>(t.w) * t.w;
        }
        for (long long i = n4 * 4 + tid; i < n; i += nthreads) acc += static_cast<double>(g[i]) * g[i];
    } else {
        for (long long i = tid; i < n; i += nthreads) acc += static_cast<double>(g[i]) * g[i];
    }
    const double t = block_sum_f64(acc);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
}
__global__ void __launch_bounds__(kNormThreads)
sumsq_final_kernel(const double *__restrict__ partial, int count, double *__restrict__ out, int accumulate) {
    double acc = 0.0;
    for (int i = threadIdx.x; i < count; i += kNormThreads) acc += partial[i];
    const double t = block_sum_f64(acc);
    if (threadIdx.x == 0) *out = accumulate ? *out + t : t;
}

struct PackArgs {
    int nd;
    long long shape[kMaxDims];
    long long stride[kMaxDims];
    long long ld_dst;      // destination pitch of the last dim's rows
    long long total;
};
// dst row-major (last dim padded to ld_dst) <- strided view.  Threads run along the
// destination, so writes are coalesced; reads are as coalesced as the view allows.
__global__ void pack_kernel(const float *__restrict__ src, float *__restrict__ dst, const PackArgs a) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < a.total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        long long rem = i, off = 0;
        const long long last = a.shape[a.nd - 1];
        const long long c = rem % last;
        rem /= last;
        off += c * a.stride[a.nd - 1];
        const long long row = rem;
        for (int d = a.nd - 2; d >= 0; --d) {
            const long long q = rem % a.shape[d];
            rem /= a.shape[d];
            off += q * a.stride[d];
        }
        dst[row * a.ld_dst + c] = src[off];
    }
}

struct UnbArgs {
    int nd;                      // dims of the original (small) shape, right-aligned into the grad shape
    long long oshape[kMaxDims];  // original shape
    long long gstride[kMaxDims]; // grad stride of the matching grad dim
    int nred;                    // number of reduced (broadcast) dims incl. leading extra dims
    long long rshape[kMaxDims];  // extents of reduced dims, outermost first
    long long rstride[kMaxDims]; // grad strides of reduced dims
    long long rtotal;
    long long total;
};
// One thread per element of the original shape; it sums the grad elements that
// broadcast onto it in ascending flat order -- the order utils::unbroadcast adds them.
__global__ void unbroadcast_kernel(const float *__restrict__ grad, float *__restrict__ out, const UnbArgs a,
                                   int accumulate) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < a.total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        long long rem = i, base = 0;
        for (int d = a.nd - 1; d >= 0; --d) {
            const long long q = rem % a.oshape[d];
            rem /= a.oshape[d];
            base += q * a.gstride[d];
        }
        float s = 0.f;
        for (long long r = 0; r < a.rtotal; ++r) {
            long long rr = r, off = base;
            for (int d = a.nred - 1; d >= 0; --d) {
                off += (rr % a.rshape[d]) * a.rstride[d];
                rr /= a.rshape[d];
            }
            s += grad[off];
        }
        out[i] = accumulate ? out[i] + s : s;
    }
}

}  // namespace

int launch_add_bias(const float *y, const float *bias, float *out, int64_t rows, int64_t n,
                    cudaStream_t stream) {
    const long long total = static_cast<long long>(rows) * n;
    if (total == 0) return MNI_B200_OK;
    const bool vec = (n % 4 == 0) && ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out) |
                                       reinterpret_cast<uintptr_t>(bias)) & 15) == 0;
    if (vec) {
        add_bias_vec_kernel<<<grid_for(total / 4, 256), 256, 0, stream>>>(
            reinterpret_cast<const float4 *>(y), reinterpret_cast<const float4 *>(bias),
            reinterpret_cast<float4 *>(out), total / 4, static_cast<int>(n / 4));
    } else {
        add_bias_scalar_kernel<<<grid_for(total, 256), 256, 0, stream>>>(y, bias, out, total, n);
    }
    MNI_LAUNCH_CHECK("add_bias");
    return MNI_B200_OK;
}

static int colsum_slabs(int64_t rows, int64_t n, int sm_count) {
    const long long strips = (n + 127) / 128;
    long long slabs = std::max<long long>(1, (sm_count * 4LL) / strips);
    slabs = std::min<long long>(slabs, (rows + 63) / 64);
    return static_cast<int>(std::max<long long>(1, slabs));
}

size_t colsum_partial_bytes(int64_t rows, int64_t n, int sm_count) {
    return static_cast<size_t>(colsum_slabs(rows, n, sm_count)) * n * sizeof(float);
}

int launch_colsum(const float *dy, int64_t ld, float *out, int64_t rows, int64_t n, bool accumulate,
                  float *partial, int sm_count, cudaStream_t stream) {
    if (n == 0) return MNI_B200_OK;
    const int slabs = colsum_slabs(rows, n, sm_count);
    const long long rows_per = (rows + slabs - 1) / slabs;
    dim3 grid(static_cast<unsigned>((n + 127) / 128), static_cast<unsigned>(slabs));
    colsum_partial_kernel<<<grid, 256, 0, stream>>>(dy, ld, partial, rows, n, rows_per);
    MNI_LAUNCH_CHECK("colsum_partial_kernel");
    colsum_final_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(partial, out, n, slabs,
                                                                                  accumulate ? 1 : 0);
    MNI_LAUNCH_CHECK("colsum_final_kernel");
    return MNI_B200_OK;
}

int launch_bias_gelu(const float *x, const float *bias, float *out, int64_t rows, int64_t n,
                     cudaStream_t stream) {
    const long long total = static_cast<long long>(rows) * n;
    if (total == 0) return MNI_B200_OK;
    const bool vec = (n % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) |
                                       reinterpret_cast<uintptr_t>(bias)) & 15) == 0;
    if (vec) {
        bias_gelu_vec_kernel<<<grid_for(total / 4, 256), 256, 0, stream>>>(
            reinterpret_cast<const float4 *>(x), reinterpret_cast<const float4 *>(bias),
            reinterpret_cast<float4 *>(out), total / 4, static_cast<int>(n / 4));
    } else {
        bias_gelu_scalar_kernel<<<grid_for(total, 256), 256, 0, stream>>>(x, bias, out, total, n);
    }
    MNI_LAUNCH_CHECK("bias_gelu");
    return MNI_B200_OK;
}

int launch_bias_gelu_bwd(const float *grad, const float *x, const float *bias, float *dx, float *dbias,
                         int64_t rows, int64_t n, bool accumulate, float *partial, int sm_count,
                         cudaStream_t stream) {
    if (n == 0 || rows == 0) return MNI_B200_OK;
    const int slabs = colsum_slabs(rows, n, sm_count);
    const long long rows_per = (rows + slabs - 1) / slabs;
    dim3 grid(static_cast<unsigned>((n + 127) / 128), static_cast<unsigned>(slabs));
    bias_gelu_bwd_partial_kernel<<<grid, 256, 0, stream>>>(grad, x, bias, dx, partial, rows, n, rows_per);
    MNI_LAUNCH_CHECK("bias_gelu_bwd_partial_kernel");
    colsum_final_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(partial, dbias, n, slabs,
                                                                                  accumulate ? 1 : 0);
    MNI_LAUNCH_CHECK("colsum_final_kernel");
    return MNI_B200_OK;
}

int launch_adamw(float *param, float *m, float *v, float *grad, int64_t n, float lr, float beta1, float beta2,
                 float eps, float weight_decay, float bc1, float bc2, const double *sumsq, float max_norm,
                 bool write_grad, cudaStream_t stream) {
    if (n == 0) return MNI_B200_OK;
    const float decay = 1.0f - lr * weight_decay;
    const bool vec = (n % 4 == 0) && ((reinterpret_cast<uintptr_t>(param) | reinterpret_cast<uintptr_t>(m) |
                                       reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(grad)) & 15) == 0;
    if (vec)
        adamw_vec_kernel<<<grid_for(n / 4, 256), 256, 0, stream>>>(
            reinterpret_cast<float4 *>(param), reinterpret_cast<float4 *>(m), reinterpret_cast<float4 *>(v),
            reinterpret_cast<float4 *>(grad), n / 4, lr, beta1, beta2, eps, decay, bc1, bc2, sumsq, max_norm,
            write_grad ? 1 : 0);
    else
        adamw_scalar_kernel<<<grid_for(n, 256), 256, 0, stream>>>(param, m, v, grad, n, lr, beta1, beta2, eps, decay, bc1,
                                                                 bc2, sumsq, max_norm, write_grad ? 1 : 0);
    MNI_LAUNCH_CHECK("adamw");
    return MNI_B200_OK;
}

int sumsq_blocks(int64_t n, int sm_count) {
    const int64_t want = (n + 4 * kNormThreads - 1) / (4 * kNormThreads);
    return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, 4 * static_cast<int64_t>(sm_count))));
}
size_t sumsq_partial_bytes(int64_t n, int sm_count) { return sizeof(double) * sumsq_blocks(n, sm_count); }
int launch_sumsq(const float *grad, int64_t n, double *out, bool accumulate, void *partial, int sm_count,
                 cudaStream_t stream) {
    const int blocks = sumsq_blocks(n, sm_count);
    double *p = static_cast<double *>(partial);
    sumsq_partial_kernel<<<blocks, kNormThreads, 0, stream>>>(grad, n, p);
    MNI_LAUNCH_CHECK("sumsq_partial");
    sumsq_final_kernel<<<1, kNormThreads, 0, stream>>>(p, blocks, out, accumulate ? 1 : 0);
    MNI_LAUNCH_CHECK("sumsq_final");
    return MNI_B200_OK;
}

int launch_copy(const float *src, float *dst, int64_t n, cudaStream_t stream) {
    if (n == 0 || src == dst) return MNI_B200_OK;
    MNI_CUDA(cudaMemcpyAsync(dst, src, static_cast<size_t>(n) * sizeof(float), cudaMemcpyDeviceToDevice, stream));
    return MNI_B200_OK;
}

int launch_pack(const mni_b200_view &src, float *dst, int64_t ld_dst, cudaStream_t stream) {
    PackArgs a{};
    a.nd = src.ndim;
    a.total = 1;
    for (int d = 0; d < src.ndim; ++d) {
        a.shape[d] = src.shape[d];
        a.stride[d] = src.stride[d];
        a.total *= src.shape[d];
    }
    a.ld_dst = ld_dst;
    if (a.total == 0) return MNI_B200_OK;
    pack_kernel<<<grid_for(a.total, 256), 256, 0, stream>>>(src.ptr, dst, a);
    MNI_LAUNCH_CHECK("pack_kernel");
    return MNI_B200_OK;
}

int launch_unbroadcast(const float *grad, const int64_t *gshape, int gnd, const int64_t *oshape, int ond,
                       float *out, bool accumulate, cudaStream_t stream) {
    long long gstr[kMaxDims];
    long long acc = 1;
    for (int d = gnd - 1; d >= 0; --d) { gstr[d] = acc; acc *= gshape[d]; }
    UnbArgs a{};
    a.nd = ond;
    a.total = 1;
    a.rtotal = 1;
    a.nred = 0;
    const int off = gnd - ond;
    for (int d = 0; d < off; ++d) {           // leading dims the original does not have
        a.rshape[a.nred] = gshape[d];
        a.rstride[a.nred] = gstr[d];
        a.rtotal *= gshape[d];
        ++a.nred;
    }
    for (int d = 0; d < ond; ++d) {
        a.oshape[d] = oshape[d];
        a.total *= oshape[d];
        if (oshape[d] == 1 && gshape[d + off] != 1) {
            a.gstride[d] = 0;
            a.rshape[a.nred] = gshape[d + off];
            a.rstride[a.nred] = gstr[d + off];
            a.rtotal *= gshape[d + off];
            ++a.nred;
        } else {
            a.gstride[d] = gstr[d + off];
        }
    }
    if (a.total == 0) return MNI_B200_OK;
    unbroadcast_kernel<<<grid_for(a.total, 256), 256, 0, stream>>>(grad, out, a, accumulate ? 1 : 0);
    MNI_LAUNCH_CHECK("unbroadcast_kernel");
    return MNI_B200_OK;
}

}  // namespace mni
