// Skinny path: at most 16 output rows (decode-like M).  These shapes move the whole
// weight matrix through the SMs for a handful of flops per byte, so they are bound by
// HBM, not by the tensor pipe; they run as CUDA-core fp32 FMA kernels with 16-byte
// loads and a split of the contraction over the grid.
//
//   fwd : y[M,N]  = x[M,K] . W[K,N] (+bias)        W streamed once, split-K partials, fused finish
//   dW  : dW[K,N] = x[M,K]^T . dy[M,N]             dW written once
//   dx  : dx[M,K] = dy[M,N] . W[K,N]^T             W streamed once, one warp per two rows of W
#include "internal.h"

#include <algorithm>

namespace mni {

namespace {

constexpr int kSkinnyThreads = 128;   // each thread owns 4 consecutive output columns

// Tickets of the fused split-K finish: one counter per 128-column strip.  The block that takes the
// last ticket of a strip sums that strip's partials; it puts the counter back to zero, so the array
// is clean again when the kernel ends.
constexpr int kMaxStrips = 4096;
constexpr int kFwdCols = 32;                               // column-threads per block: a 128-column strip
constexpr int kFwdGroups = 16;                             // k-groups per block
constexpr int kFwdThreads = kFwdCols * kFwdGroups;         // 512
__device__ unsigned int g_skinny_tickets[kMaxStrips];

// grid = (n strips of 128 columns, k splits), 512 threads = 32 column-threads x 16 k-groups: a warp
// reads 512 contiguous bytes of a W row, and narrow strips keep the number of K splits (and with it
// the serial tail of the finish) small.
// x[M, k-slice] is staged in shared memory; each k-group streams its sixteenth of the block's W rows
// with 16-byte loads, a batch of U rows in flight per thread while the previous batch is multiplied.
// The groups are added through shared memory in group order, the block's sum goes to scratch,
// and the last block to finish a strip adds the strip's partials in ascending split order, applies
// bias / accumulate and writes y.  Every sum has a fixed order: results do not depend on scheduling.
template <int MT>
__global__ void __launch_bounds__(kFwdThreads)
skinny_fwd_kernel(const float *__restrict__ x, long long ldx, const float *__restrict__ W, long long ldw,
                  float *__restrict__ partial, float *__restrict__ y, long long ldy,
                  const float *__restrict__ bias, int accumulate, int M, long long N, long long K,
                  long long k_per) {
    constexpr int U = MT <= 2 ? 8 : 4;
    extern __shared__ float smem_f[];
    float *xs = smem_f;                                                  // [MT][k_per]
    float4 *red = reinterpret_cast<float4 *>(smem_f + MT * k_per);       // [groups-1][MT][128]
    __shared__ unsigned int s_ticket;
    const int kg = threadIdx.x / kFwdCols, ct = threadIdx.x % kFwdCols;
    const long long k0 = blockIdx.y * k_per;
    const long long k1 = min(K, k0 + k_per);
    const int kc = static_cast<int>(k1 - k0);
    const int g0 = (kc * kg / kFwdGroups) & ~3;
    const int g1 = kg == kFwdGroups - 1 ? kc : ((kc * (kg + 1) / kFwdGroups) & ~3);
    const long long col = (static_cast<long long>(blockIdx.x) * kFwdCols + ct) * 4;
    const bool live = col < N;
    const bool vec = col + 3 < N;
    const float *wp = W + k0 * ldw + col;
    float4 w[U];
    if (vec && g0 + U <= g1) {
#pragma unroll
        for (int u = 0; u < U; ++u) w[u] = __ldcs(reinterpret_cast<const float4 *>(wp + (g0 + u) * ldw));
    }
    for (int i = threadIdx.x; i < MT * static_cast<int>(k_per); i += kFwdThreads) {
        const int m = i / static_cast<int>(k_per), kk = i - m * static_cast<int>(k_per);
        xs[i] = (m < M && kk < kc) ? __ldg(x + m * ldx + k0 + kk) : 0.f;
    }
    __syncthreads();
    float4 acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = make_float4(0.f, 0.f, 0.f, 0.f);
    int kk = g0;
    if (vec) {
        for (; kk + U <= g1; kk += U) {
            float4 wn[U];
            const bool more = kk + 2 * U <= g1;
            if (more) {
#pragma unroll
                for (int u = 0; u < U; ++u) wn[u] = __ldcs(reinterpret_cast<const float4 *>(wp + (kk + U + u) * ldw));
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
#pragma unroll
                for (int u4 = 0; u4 < U; u4 += 4) {
                    const float4 xv = *reinterpret_cast<const float4 *>(xs + m * k_per + kk + u4);
                    const float xa[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        acc[m].x = fmaf(xa[u], w[u4 + u].x, acc[m].x);
                        acc[m].y = fmaf(xa[u], w[u4 + u].y, acc[m].y);
                        acc[m].z = fmaf(xa[u], w[u4 + u].z, acc[m].z);
                        acc[m].w = fmaf(xa[u], w[u4 + u].w, acc[m].w);
                    }
                }
            }
            if (more) {
#pragma unroll
                for (int u = 0; u < U; ++u) w[u] = wn[u];
            }
        }
    }
    if (live) {
        for (; kk < g1; ++kk) {
            float wr[4] = {0.f, 0.f, 0.f, 0.f};
            if (vec) {
                const float4 t = __ldcs(reinterpret_cast<const float4 *>(wp + kk * ldw));
                wr[0] = t.x; wr[1] = t.y; wr[2] = t.z; wr[3] = t.w;
            } else {
                for (int e = 0; e < 4; ++e)
                    if (col + e < N) wr[e] = __ldg(wp + kk * ldw + e);
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const float xv = xs[m * k_per + kk];
                acc[m].x = fmaf(xv, wr[0], acc[m].x);
                acc[m].y = fmaf(xv, wr[1], acc[m].y);
                acc[m].z = fmaf(xv, wr[2], acc[m].z);
                acc[m].w = fmaf(xv, wr[3], acc[m].w);
            }
        }
    }
    // k-groups 1..3 hand their sums to group 0 through shared memory.
    if (kg > 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) red[((kg - 1) * MT + m) * kFwdCols + ct] = acc[m];
    }
    __syncthreads();
    if (kg == 0 && live) {
        float *out = partial + static_cast<long long>(blockIdx.y) * M * N;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m >= M) break;
            float4 a = acc[m];
#pragma unroll
            for (int g = 0; g < kFwdGroups - 1; ++g) {
                const float4 t = red[(g * MT + m) * kFwdCols + ct];
                a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
            }
            float *o = out + m * N + col;
            const float av[4] = {a.x, a.y, a.z, a.w};
            for (int e = 0; e < 4; ++e)
                if (col + e < N) __stcg(o + e, av[e]);
        }
    }
    // Fused finish: the block holding the strip's last ticket reduces it; k-group g takes rows g, g+4, ...
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_ticket = atomicAdd(&g_skinny_tickets[blockIdx.x], 1u);
    __syncthreads();
    if (s_ticket != gridDim.y - 1) return;
    __threadfence();
    if (live) {
        const int splits = static_cast<int>(gridDim.y);
        const long long slab = static_cast<long long>(M) * N;
        const bool vec4 = vec && (N & 3) == 0;
        for (int m = kg; m < M; m += kFwdGroups) {
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            const float *src = partial + m * N + col;
            if (vec4) {
                int sp = 0;
                for (; sp + 8 <= splits; sp += 8) {      // 8 independent loads in flight, added in order
                    float4 t[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) t[u] = __ldcg(reinterpret_cast<const float4 *>(src + (sp + u) * slab));
#pragma unroll
                    for (int u = 0; u < 8; ++u) { sum[0] += t[u].x; sum[1] += t[u].y; sum[2] += t[u].z; sum[3] += t[u].w; }
                }
                for (; sp < splits; ++sp) {
                    const float4 t = __ldcg(reinterpret_cast<const float4 *>(src + sp * slab));
                    sum[0] += t.x; sum[1] += t.y; sum[2] += t.z; sum[3] += t.w;
                }
            } else {
                for (int sp = 0; sp < splits; ++sp)
                    for (int e = 0; e < 4; ++e)
                        if (col + e < N) sum[e] += __ldcg(src + sp * slab + e);
            }
            for (int e = 0; e < 4; ++e) {
                if (col + e >= N) break;
                float v = sum[e];
                if (bias) v += __ldg(bias + col + e);
                float *dst = y + m * ldy + col + e;
                *dst = accumulate ? *dst + v : v;
            }
        }
    }
    if (threadIdx.x == 0) g_skinny_tickets[blockIdx.x] = 0u;
}

// grid = (n strips of 512 columns, k slabs).  dy[M, 4 cols] lives in registers; each
// k row of dW is one float4 store per thread.
template <int MT>
__global__ void __launch_bounds__(kSkinnyThreads)
skinny_dw_kernel(const float *__restrict__ x, long long ldx, const float *__restrict__ dy, long long lddy,
                 float *__restrict__ dW, long long lddw, int accumulate, int M, long long N, long long K,
                 long long k_per) {
    extern __shared__ float xs[];   // [k_per][MT]
    const long long k0 = blockIdx.y * k_per;
    const long long k1 = min(K, k0 + k_per);
    const int kc = static_cast<int>(k1 - k0);
    for (int i = threadIdx.x; i < MT * kc; i += kSkinnyThreads) {
        const int kk = i % kc, m = i / kc;
        xs[kk * MT + m] = m < M ? __ldg(x + m * ldx + k0 + kk) : 0.f;
    }
    __syncthreads();
    const long long col = (static_cast<long long>(blockIdx.x) * kSkinnyThreads + threadIdx.x) * 4;
    if (col >= N) return;
    float g[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
        for (int e = 0; e < 4; ++e) g[m][e] = (m < M && col + e < N) ? __ldg(dy + m * lddy + col + e) : 0.f;
    const bool vec = (col + 3 < N) && ((lddw & 3) == 0) && ((reinterpret_cast<uintptr_t>(dW) & 15) == 0);
    for (int kk = 0; kk < kc; ++kk) {
        float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float xv = xs[kk * MT + m];
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = fmaf(xv, g[m][e], o[e]);
        }
        float *dst = dW + (k0 + kk) * lddw + col;
        if (vec) {
            float4 v = make_float4(o[0], o[1], o[2], o[3]);
            if (accumulate) {
                const float4 old = *reinterpret_cast<const float4 *>(dst);
                v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
            }
            __stcs(reinterpret_cast<float4 *>(dst), v);
        } else {
            for (int e = 0; e < 4; ++e)
                if (col + e < N) dst[e] = accumulate ? dst[e] + o[e] : o[e];
        }
    }
}

// dx[M,K] = dy[M,N] . W[K,N]^T.  A warp owns kDxRows rows of W; its lanes walk the row 128 floats at
// a time with 16-byte streaming loads, multiply with the matching dy slices (a few KB, served from
// L1/L2) and a shuffle tree folds the 32 lane sums.  W is read exactly once.
constexpr int kDxThreads = 256;
constexpr int kDxRows = 2;
// FULL: M == MT and N a multiple of 512, so the loop carries no bounds tests and the compiler can issue
// all 8 weight loads and all 4 * MT dy loads of a step before the first multiply.
template <int MT, bool FULL>
__global__ void __launch_bounds__(kDxThreads)
skinny_dx_kernel(const float *__restrict__ dy, long long lddy, const float *__restrict__ W, long long ldw,
                 float *__restrict__ dx, long long lddx, int accumulate, int M, long long N, long long K) {
    const int lane = threadIdx.x & 31;
    const long long gw = static_cast<long long>(blockIdx.x) * (kDxThreads / 32) + (threadIdx.x >> 5);
    const long long k0 = gw * kDxRows;
    if (k0 >= K) return;
    float acc[kDxRows][MT];
#pragma unroll
    for (int r = 0; r < kDxRows; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
    const float *w0 = W + k0 * ldw;
    const bool row1 = k0 + 1 < K;
    const float *w1 = row1 ? w0 + ldw : w0;
    // 512 floats of both rows per step: eight 16-byte weight loads in flight per lane (4 KB per warp),
    // enough outstanding bytes per SM to keep HBM busy with 16 resident warps.
    constexpr int P = 4;                                   // 128-float positions per step
    for (long long n = lane * 4; n < N; n += 128 * P) {
        float4 wa[P], wb[P];
#pragma unroll
        for (int q = 0; q < P; ++q) {
            const long long nq = n + 128 * q;
            if (FULL || nq < N) {
                wa[q] = __ldcs(reinterpret_cast<const float4 *>(w0 + nq));
                wb[q] = __ldcs(reinterpret_cast<const float4 *>(w1 + nq));
            } else {
                wa[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                wb[q] = wa[q];
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (FULL || m < M) {
#pragma unroll
                for (int q = 0; q < P; ++q) {
                    const long long nq = n + 128 * q;
                    if (FULL || nq < N) {
                        const float4 g = __ldg(reinterpret_cast<const float4 *>(dy + m * lddy + nq));
                        acc[0][m] = fmaf(g.x, wa[q].x, fmaf(g.y, wa[q].y, fmaf(g.z, wa[q].z, fmaf(g.w, wa[q].w, acc[0][m]))));
                        acc[1][m] = fmaf(g.x, wb[q].x, fmaf(g.y, wb[q].y, fmaf(g.z, wb[q].z, fmaf(g.w, wb[q].w, acc[1][m]))));
                    }
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kDxRows; ++r) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[r][m];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0 && m < M && k0 + r < K) {
                float *dst = dx + m * lddx + k0 + r;
                *dst = accumulate ? *dst + v : v;
            }
        }
    }
}

int pick_mt(int64_t M) { return M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16; }

struct FwdPlan { int splits; long long k_per; int strips; };

FwdPlan fwd_plan(int64_t M, int64_t N, int64_t K, int sm_count) {
    FwdPlan pl;
    pl.strips = static_cast<int>((N + 4 * kFwdCols - 1) / (4 * kFwdCols));
    // Two 512-thread blocks per SM in total, but keep the partial traffic (splits * M * N * 8 bytes)
    // well under the weight traffic (K * N * 4 bytes) and every k-group at least 8 rows deep.
    long long want = std::max<long long>(1, (sm_count * 2LL) / pl.strips);
    long long cap = std::max<long long>(1, K / (16 * std::max<int64_t>(M, 1)));
    long long splits = std::min(want, cap);
    splits = std::min<long long>(splits, std::max<long long>(1, K / (8 * kFwdGroups)));
    splits = std::max<long long>(splits, (K + 2047) / 2048);   // shared-memory bound on a k slice
    // Every k-group then gets a multiple of 8 rows: whole batches of loads in flight, no serial remainder
    // (a 4-row remainder cost four dependent DRAM round trips, 3 us of a 17 us kernel).
    const long long unit = 8LL * kFwdGroups;
    pl.k_per = ((K + splits - 1) / splits + unit - 1) / unit * unit;
    pl.splits = static_cast<int>((K + pl.k_per - 1) / pl.k_per);
    return pl;
}

}  // namespace

bool skinny_fwd_supported(int64_t M, int64_t N, int64_t K) {
    return M >= 1 && M <= 16 && N >= 1 && K >= 1;
}

size_t skinny_fwd_partial_bytes(int64_t M, int64_t N, int64_t K, int sm_count) {
    const FwdPlan pl = fwd_plan(M, N, K, sm_count);
    return static_cast<size_t>(pl.splits) * M * N * sizeof(float);
}

int launch_skinny_fwd(const float *x, int64_t ldx, const float *W, int64_t ldw, float *y, int64_t ldy,
                      const float *bias, bool accumulate, int64_t M, int64_t N, int64_t K, float *partial,
                      int sm_count, cudaStream_t stream) {
    const FwdPlan pl = fwd_plan(M, N, K, sm_count);
    const int mt = pick_mt(M);
    dim3 grid(pl.strips, pl.splits);
    const size_t smem = static_cast<size_t>(mt) * pl.k_per * sizeof(float) +
                        static_cast<size_t>(kFwdGroups - 1) * mt * kFwdCols * sizeof(float4);
    const bool vec_w = (ldw % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);
    if (!vec_w) return fail(MNI_B200_ERR_ARG, "skinny path needs a 16-byte aligned weight with ld %% 4 == 0");
    if (pl.strips > kMaxStrips) return fail(MNI_B200_ERR_ARG, "skinny path: N too large");
#define MNI_SKINNY_FWD(MT)                                                                             \
    case MT:                                                                                           \
        cudaFuncSetAttribute(skinny_fwd_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); \
        skinny_fwd_kernel<MT><<<grid, kFwdThreads, smem, stream>>>(x, ldx, W, ldw, partial, y, ldy, bias,    \
                                                                      accumulate ? 1 : 0, (int)M, N, K, pl.k_per); \
        break;
    switch (mt) {
        MNI_SKINNY_FWD(1) MNI_SKINNY_FWD(2) MNI_SKINNY_FWD(4) MNI_SKINNY_FWD(8) MNI_SKINNY_FWD(16)
    }
#undef MNI_SKINNY_FWD
    MNI_LAUNCH_CHECK("skinny_fwd_kernel");
    return MNI_B200_OK;
}

bool skinny_dx_supported(const float *dy, int64_t lddy, const float *W, int64_t ldw, int64_t M, int64_t N) {
    return M >= 1 && M <= 8 && N % 4 == 0 && ldw % 4 == 0 && lddy % 4 == 0 &&
           ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(dy)) & 15) == 0;
}

int launch_skinny_dx(const float *dy, int64_t lddy, const float *W, int64_t ldw, float *dx, int64_t lddx,
                     bool accumulate, int64_t M, int64_t N, int64_t K, cudaStream_t stream) {
    const int mt = pick_mt(M);
    const long long rows_per_block = (kDxThreads / 32) * kDxRows;
    const unsigned blocks = static_cast<unsigned>((K + rows_per_block - 1) / rows_per_block);
    const bool full = M == mt && mt >= 4 && N % 512 == 0;   // measured: slower than the guarded loop for 1-2 rows
#define MNI_SKINNY_DX(MT)                                                                              \
    case MT:                                                                                           \
        if (full)                                                                                      \
            skinny_dx_kernel<MT, true><<<blocks, kDxThreads, 0, stream>>>(dy, lddy, W, ldw, dx, lddx,    \
                                                                           accumulate ? 1 : 0, (int)M, N, K); \
        else                                                                                           \
            skinny_dx_kernel<MT, false><<<blocks, kDxThreads, 0, stream>>>(dy, lddy, W, ldw, dx, lddx,   \
                                                                            accumulate ? 1 : 0, (int)M, N, K); \
        break;
    switch (mt) {
        MNI_SKINNY_DX(1) MNI_SKINNY_DX(2) MNI_SKINNY_DX(4) MNI_SKINNY_DX(8)
        default: return fail(MNI_B200_ERR_ARG, "skinny dx handles at most 8 rows");
    }
#undef MNI_SKINNY_DX
    MNI_LAUNCH_CHECK("skinny_dx_kernel");
    return MNI_B200_OK;
}

int launch_skinny_dw(const float *x, int64_t ldx, const float *dy, int64_t lddy, float *dW, int64_t lddw,
                     bool accumulate, int64_t M, int64_t N, int64_t K, cudaStream_t stream) {
    const int mt = pick_mt(M);
    const int strips = static_cast<int>((N + 4 * kSkinnyThreads - 1) / (4 * kSkinnyThreads));
    long long slabs = std::max<long long>(1, (148 * 8LL) / strips);
    long long k_per = std::max<long long>(8, (K + slabs - 1) / slabs);
    k_per = std::min<long long>(k_per, 1024);
    slabs = (K + k_per - 1) / k_per;
    dim3 grid(strips, static_cast<unsigned>(slabs));
    const size_t smem = static_cast<size_t>(mt) * k_per * sizeof(float);
#define MNI_SKINNY_DW(MT)                                                                              \
    case MT:                                                                                           \
        cudaFuncSetAttribute(skinny_dw_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
        skinny_dw_kernel<MT><<<grid, kSkinnyThreads, smem, stream>>>(x, ldx, dy, lddy, dW, lddw,       \
                                                                     accumulate ? 1 : 0, (int)M, N, K, k_per); \
        break;
    switch (mt) {
        MNI_SKINNY_DW(1) MNI_SKINNY_DW(2) MNI_SKINNY_DW(4) MNI_SKINNY_DW(8) MNI_SKINNY_DW(16)
    }
#undef MNI_SKINNY_DW
    MNI_LAUNCH_CHECK("skinny_dw_kernel");
    return MNI_B200_OK;
}

}  // namespace mni
