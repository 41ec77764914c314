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
#include <cstdlib>

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

// ---- forward through a per-thread cp.async ring ----------------------------------------------------
// Same decomposition as skinny_fwd_kernel (128-column strips x K splits, k-groups inside a block, fused
// ticket finish), but the weight no longer travels through registers: every thread copies its own
// 16-byte pieces of W into a private ring in shared memory with cp.async, kRingAhead batches of four
// rows ahead of the batch it multiplies.  The bytes in flight are then set by the ring, not by the
// register file, so a thread can keep 16 accumulator vectors (16 rows of x) and still have 192 bytes
// on their way; and a k-group's chain of dependent DRAM round trips shrinks from one per batch to the
// ring's fill.  No thread reads another thread's ring slots, so the loop needs no block barrier.
constexpr int kRingThreads = 256;                           // COLS column-threads x GROUPS k-groups
constexpr int kRingBatch = 4;                               // rows of W per cp.async group
// Measured at K = N = 4096 (1 / 8 rows): 8 groups x 4 batches 15.4 / 18.7 us; 4 groups 17.0 / 20.1; 2 groups
// 17.3 / 25.4; a ring of 6 batches 15.5 / 19.8 (and one block per SM from 8 rows on).
constexpr int kRingGroups = 8;                              // k-groups per block: 32 column-threads, a 128-column strip
constexpr int kRingDepth = 4;                               // batches held by the ring, all but one in flight
constexpr size_t kRingXBytes = 40 * 1024;                   // cap on the staged x slice: two blocks per SM

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem, bool valid) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    const int bytes = valid ? 16 : 0;                       // 0: nothing is read, the slot is zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Thread-block-cluster helpers for the ring kernel's finish: the K splits of a strip form one cluster, every
// CTA leaves its block sums in its own shared memory and the sums are added straight from there.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_cluster_f4(const void *own_smem, unsigned rank) {
    const unsigned local = static_cast<unsigned>(__cvta_generic_to_shared(own_smem));
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}

// Requires N % 4 == 0, W 16-byte aligned with ldw % 4 == 0, k_per a multiple of kRingUnit.
// cluster != 0: launched as clusters of gridDim.y CTAs along y (at most 8); the finish then goes through
// distributed shared memory instead of scratch, fence and ticket, in the same ascending split order.
template <int MT, int GROUPS, int DEPTH>
__global__ void __launch_bounds__(kRingThreads, 2)
skinny_fwd_ring_kernel(const float *__restrict__ x, long long ldx, const float *__restrict__ W, long long ldw,
                       float *__restrict__ partial, float *__restrict__ y, long long ldy,
                       const float *__restrict__ bias, int accumulate, int M, long long N, long long K, int k_per,
                       int x_vec, int cluster) {
    extern __shared__ __align__(16) float smem_f[];
    float *xs = smem_f;                                                  // [MT][k_per], zero beyond M / K
    float4 *ring = reinterpret_cast<float4 *>(smem_f + MT * k_per);      // [depth * batch][threads]; later the group sums
    __shared__ unsigned int s_ticket;
    constexpr int COLS = kRingThreads / GROUPS, AHEAD = DEPTH - 1;
    const int kg = threadIdx.x / COLS, ct = threadIdx.x % COLS;
    const long long k0 = static_cast<long long>(blockIdx.y) * k_per;
    const int kc = static_cast<int>(min(K, k0 + k_per) - k0);
    const int rpg = k_per / GROUPS;                                 // rows per k-group, a multiple of 4
    const int g0 = kg * rpg;
    const int nb = rpg / kRingBatch;
    const long long col = (static_cast<long long>(blockIdx.x) * COLS + ct) * 4;
    const bool live = col < N;
    const float *wp = W + k0 * ldw + (live ? col : 0);
    float4 *mine = ring + threadIdx.x;
    auto issue = [&](int b) {
        if (b < nb) {
#pragma unroll
            for (int u = 0; u < kRingBatch; ++u) {
                const int r = g0 + b * kRingBatch + u;
                const bool ok = live && r < kc;
                cp_async16(mine + ((b % DEPTH) * kRingBatch + u) * kRingThreads,
                           wp + static_cast<long long>(ok ? r : 0) * ldw, ok);
            }
        }
        cp_async_commit();                                               // empty groups keep the count uniform
    };
    // The x slice goes first and asynchronously as well (16-byte pieces, zero-filled beyond M rows / kc
    // columns): staged with ordinary loads its 4 * MT * k_per bytes cost one L2 round trip per few elements
    // of every thread, which at 16 rows was a third of the kernel's time.
    if (x_vec) {
        const int quads = k_per / 4;
        for (int i = threadIdx.x; i < MT * quads; i += kRingThreads) {
            const int m = i / quads, kk = (i - m * quads) * 4;
            const int valid = m < M ? max(0, min(4, kc - kk)) : 0;
            const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(xs + m * k_per + kk));
            const float *src = valid > 0 ? x + m * ldx + k0 + kk : x;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid * 4) : "memory");
        }
    } else {
        for (int i = threadIdx.x; i < MT * k_per; i += kRingThreads) {
            const int m = i / k_per, kk = i - m * k_per;
            xs[i] = (m < M && kk < kc) ? __ldg(x + m * ldx + k0 + kk) : 0.f;
        }
    }
    cp_async_commit();
#pragma unroll
    for (int b = 0; b < AHEAD; ++b) issue(b);
    cp_async_wait<AHEAD>();                                         // the x slice (oldest group) has landed
    __syncthreads();
    float4 acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int b = 0; b < nb; ++b) {
        issue(b + AHEAD);
        cp_async_wait<AHEAD>();                                     // batch b has landed
        float4 w[kRingBatch];
#pragma unroll
        for (int u = 0; u < kRingBatch; ++u) w[u] = mine[((b % DEPTH) * kRingBatch + u) * kRingThreads];
        const float *xr = xs + g0 + b * kRingBatch;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float4 xv = *reinterpret_cast<const float4 *>(xr + m * k_per);
            const float xa[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int u = 0; u < kRingBatch; ++u) {
                acc[m].x = fmaf(xa[u], w[u].x, acc[m].x);
                acc[m].y = fmaf(xa[u], w[u].y, acc[m].y);
                acc[m].z = fmaf(xa[u], w[u].z, acc[m].z);
                acc[m].w = fmaf(xa[u], w[u].w, acc[m].w);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();                                                     // every thread is done with its ring slots
    float4 *red = ring;                                                  // [groups - 1][MT][cols]
    float4 *mine_sums = ring + (GROUPS - 1) * MT * COLS;                 // [MT][cols]: this block's sums (cluster finish)
    if (kg > 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) red[((kg - 1) * MT + m) * COLS + ct] = acc[m];
    }
    __syncthreads();
    if (kg == 0) {
        float *out = partial + static_cast<long long>(blockIdx.y) * M * N;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m >= M) break;
            float4 a = acc[m];
#pragma unroll
            for (int g = 0; g < GROUPS - 1; ++g) {
                const float4 t = red[(g * MT + m) * COLS + ct];
                a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
            }
            if (cluster) mine_sums[m * COLS + ct] = a;
            else if (live) __stcg(reinterpret_cast<float4 *>(out + m * N + col), a);
        }
    }
    if (cluster) {
        // Rows are dealt out over (CTA rank, k-group); a row's splits are added in ascending rank = split order.
        cluster_sync_all();
        const int ranks = static_cast<int>(gridDim.y);
        if (live) {
            for (int m = static_cast<int>(blockIdx.y) * GROUPS + kg; m < M; m += ranks * GROUPS) {
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int r = 0; r < ranks; ++r) {
                    const float4 t = ld_cluster_f4(mine_sums + m * COLS + ct, static_cast<unsigned>(r));
                    sum.x += t.x; sum.y += t.y; sum.z += t.z; sum.w += t.w;
                }
                const float sv[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = sv[e];
                    if (bias) v += __ldg(bias + col + e);
                    float *dst = y + m * ldy + col + e;
                    *dst = accumulate ? *dst + v : v;
                }
            }
        }
        cluster_sync_all();                                              // no CTA leaves while its sums may still be read
        return;
    }
    // Fused finish, as in skinny_fwd_kernel: the block that takes a strip's last ticket adds the strip's
    // partials in ascending split order; k-group g takes rows g, g + 8, ...
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_ticket = atomicAdd(&g_skinny_tickets[blockIdx.x], 1u);
    __syncthreads();
    if (s_ticket != gridDim.y - 1) return;
    __threadfence();
    if (live) {
        const int splits = static_cast<int>(gridDim.y);
        const long long slab = static_cast<long long>(M) * N;
        for (int m = kg; m < M; m += GROUPS) {
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            const float *src = partial + m * N + col;
            int sp = 0;
            for (; sp + 4 <= splits; sp += 4) {                          // 4 independent loads in flight, added in order
                float4 t[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) t[u] = __ldcg(reinterpret_cast<const float4 *>(src + (sp + u) * slab));
#pragma unroll
                for (int u = 0; u < 4; ++u) { sum.x += t[u].x; sum.y += t[u].y; sum.z += t[u].z; sum.w += t[u].w; }
            }
            for (; sp < splits; ++sp) {
                const float4 t = __ldcg(reinterpret_cast<const float4 *>(src + sp * slab));
                sum.x += t.x; sum.y += t.y; sum.z += t.z; sum.w += t.w;
            }
            const float sv[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = sv[e];
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

// Second form of dx = dy . W^T, used from 3 rows up.  In the kernel above a warp walks its two weight rows
// through all of N: eight sequential steps, each a full DRAM round trip, and 4 * MT loads of dy (from L1) per
// step.  Here a block of 8 warps owns 16 weight rows and each warp owns a 128 * P-float slice of N for all 16
// rows: its dy slice is loaded ONCE into registers (MT * P 16-byte vectors) and stays there while the warp
// streams the 16 rows' slice in row pairs, the next pair's weight loads issued before the current pair is
// multiplied, so two pairs (4 * P 16-byte loads per lane) are always in flight.  Lane sums are folded with
// shuffles, a warp adds its slices into its own line of shared memory, and after one block barrier the
// block's first threads add the 8 warps' lines in warp order (fixed order: bit-reproducible) and write dx.
constexpr int kDxsWarps = 8;
constexpr int kDxsRows = 16;
template <int MT, int P, int MINB>
__global__ void __launch_bounds__(32 * kDxsWarps, MINB)
skinny_dx_sliced_kernel(const float *__restrict__ dy, long long lddy, const float *__restrict__ W, long long ldw,
                        float *__restrict__ dx, long long lddx, int accumulate, int M, long long N, long long K) {
    __shared__ float part[kDxsWarps][kDxsRows][MT];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long k0 = static_cast<long long>(blockIdx.x) * kDxsRows;
    for (int i = lane; i < kDxsRows * MT; i += 32) (&part[warp][0][0])[i] = 0.f;
    __syncwarp();
    const long long slice_w = 128LL * P;
    const long long nslices = (N + slice_w - 1) / slice_w;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long slice = warp; slice < nslices; slice += kDxsWarps) {
        const long long n0 = slice * slice_w + lane * 4;
        float4 g[MT][P];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int q = 0; q < P; ++q) {
                const long long nq = n0 + 128 * q;
                g[m][q] = (m < M && nq < N) ? __ldg(reinterpret_cast<const float4 *>(dy + m * lddy + nq)) : zero4;
            }
        auto load_pair = [&](int pr, float4 (&wa)[P], float4 (&wb)[P]) {
            // rows past K repeat the last row: loaded, never stored
            const long long ra = min(k0 + 2 * pr, K - 1), rb = min(k0 + 2 * pr + 1, K - 1);
            const float *pa = W + ra * ldw, *pb = W + rb * ldw;
#pragma unroll
            for (int q = 0; q < P; ++q) {
                const long long nq = n0 + 128 * q;
                if (nq < N) {
                    wa[q] = __ldcs(reinterpret_cast<const float4 *>(pa + nq));
                    wb[q] = __ldcs(reinterpret_cast<const float4 *>(pb + nq));
                } else {
                    wa[q] = zero4;
                    wb[q] = zero4;
                }
            }
        };
        float4 wa[P], wb[P], na[P], nb[P];
        load_pair(0, wa, wb);
#pragma unroll
        for (int pr = 0; pr < kDxsRows / 2; ++pr) {
            if (pr + 1 < kDxsRows / 2) load_pair(pr + 1, na, nb);
            float acc[2][MT];
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                acc[0][m] = 0.f;
                acc[1][m] = 0.f;
#pragma unroll
                for (int q = 0; q < P; ++q) {
                    const float4 gv = g[m][q];
                    acc[0][m] = fmaf(gv.x, wa[q].x, fmaf(gv.y, wa[q].y, fmaf(gv.z, wa[q].z, fmaf(gv.w, wa[q].w, acc[0][m]))));
                    acc[1][m] = fmaf(gv.x, wb[q].x, fmaf(gv.y, wb[q].y, fmaf(gv.z, wb[q].z, fmaf(gv.w, wb[q].w, acc[1][m]))));
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float v = acc[r][m];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                    if (lane == 0) part[warp][2 * pr + r][m] += v;
                }
            if (pr + 1 < kDxsRows / 2) {
#pragma unroll
                for (int q = 0; q < P; ++q) { wa[q] = na[q]; wb[q] = nb[q]; }
            }
        }
        __syncwarp();
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kDxsRows * MT; i += 32 * kDxsWarps) {
        const int row = i / MT, m = i - row * MT;
        if (m >= M || k0 + row >= K) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kDxsWarps; ++w) v += part[w][row][m];
        float *dst = dx + m * lddx + k0 + row;
        *dst = accumulate ? *dst + v : v;
    }
}

// Which dx kernel runs.  The sliced kernel is opt-in (MNI_B200_SKINNY_DX_SLICED=1): measured inside the
// benchmark step at 4 rows, K = N = 4096, it needs ~28 us against ~18 us for the row-pair kernel.
int dx_sliced_mode() {
    const char *v = getenv("MNI_B200_SKINNY_DX_SLICED");
    return v && *v ? atoi(v) : -1;
}

int pick_mt(int64_t M) { return M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16; }

struct FwdPlan { int splits; long long k_per; int strips; bool ring; bool cluster = false; };

// The cp.async-ring kernel takes every aligned problem (K = N = 4096, weight not in L2, cluster finish:
// 14.2 / 14.6 / 15.8 / 17.7 us at 1 / 2 / 4 / 8 rows against 17.4 / 19.0 / 16.4 / 27.3 us for the
// register-staged kernel).  MNI_B200_SKINNY_RING=0 keeps the register-staged kernel everywhere.
int ring_mode() {
    static const int mode = [] {
        const char *v = getenv("MNI_B200_SKINNY_RING");
        return v && *v ? atoi(v) : 1;
    }();
    return mode;
}

bool ring_wanted(int64_t M, int64_t N) {
    (void)M;
    return ring_mode() != 0 && N % 4 == 0;
}

FwdPlan ring_plan(int64_t M, int64_t N, int64_t K, int sm_count) {
    FwdPlan pl;
    pl.ring = true;
    const int cols = kRingThreads / kRingGroups, unit = kRingGroups * kRingBatch;
    pl.strips = static_cast<int>((N + 4 * cols - 1) / (4 * cols));
    // Two 256-thread blocks per SM in one wave; partial traffic (splits * M * N * 8 bytes) at most a quarter
    // of the weight traffic (K * N * 4 bytes); every k-group at least one batch deep.
    const long long want = std::max<long long>(1, (sm_count * 2LL) / pl.strips);
    const long long cap = std::max<long long>(1, K / (8 * std::max<int64_t>(M, 1)));
    long long splits = std::min(want, cap);
    splits = std::min<long long>(splits, std::max<long long>(1, K / unit));
    long long k_per = ((K + splits - 1) / splits + unit - 1) / unit * unit;
    const long long k_max = static_cast<long long>(kRingXBytes / sizeof(float) / pick_mt(M)) / unit * unit;
    k_per = std::min(k_per, std::min<long long>(k_max, 2048));
    // Up to 8 splits can finish as one thread-block cluster through distributed shared memory; a plan of 9-12
    // splits is rounded down to 8 when the longer k slice still fits (MNI_B200_RING_CLUSTER=0: ticket finish only).
    static const bool cluster_on = [] {
        const char *v = getenv("MNI_B200_RING_CLUSTER");
        return !(v && *v) || atoi(v) != 0;
    }();
    if (cluster_on) {
        const long long k8 = ((K + 7) / 8 + unit - 1) / unit * unit;
        const long long n_now = (K + k_per - 1) / k_per;
        if (n_now > 8 && n_now <= 12 && k8 <= std::min<long long>(k_max, 2048)) k_per = k8;
    }
    pl.k_per = k_per;
    pl.splits = static_cast<int>((K + k_per - 1) / k_per);
    pl.cluster = cluster_on && pl.splits >= 2 && pl.splits <= 8;
    return pl;
}

FwdPlan fwd_plan(int64_t M, int64_t N, int64_t K, int sm_count) {
    if (ring_wanted(M, N)) return ring_plan(M, N, K, sm_count);
    FwdPlan pl;
    pl.ring = false;
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

// Rows up to which the streaming forward beats the tensor path (measured at K = N = 4096, weight not in L2:
// ring kernel 17.7 us at 8 rows, register-staged kernel 26.7 us at 5, tensor path 20-23.5 us at either).
int64_t skinny_fwd_row_limit(int64_t N) { return ring_mode() != 0 && N % 4 == 0 ? 8 : 4; }

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
    if (pl.ring) {
        const size_t ring_smem = static_cast<size_t>(mt) * pl.k_per * sizeof(float) +
                                 static_cast<size_t>(kRingDepth) * kRingBatch * kRingThreads * sizeof(float4);
        const bool x_vec = (ldx % 4 == 0 || M == 1) && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kRingThreads);
        cfg.dynamicSmemBytes = ring_smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = static_cast<unsigned>(pl.splits);
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pl.cluster ? 1 : 0;
        const int acc_i = accumulate ? 1 : 0, m_i = static_cast<int>(M), kper_i = static_cast<int>(pl.k_per);
        const int xvec_i = x_vec ? 1 : 0, cluster_i = pl.cluster ? 1 : 0;
        const long long ldx_l = ldx, ldw_l = ldw, ldy_l = ldy, n_l = N, k_l = K;
#define MNI_SKINNY_RING(MT)                                                                            \
    case MT:                                                                                           \
        cudaFuncSetAttribute(skinny_fwd_ring_kernel<MT, kRingGroups, kRingDepth>,                      \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);                 \
        cudaLaunchKernelEx(&cfg, skinny_fwd_ring_kernel<MT, kRingGroups, kRingDepth>, x, ldx_l, W, ldw_l, partial, \
                           y, ldy_l, bias, acc_i, m_i, n_l, k_l, kper_i, xvec_i, cluster_i);           \
        break;
        switch (mt) {
            MNI_SKINNY_RING(1) MNI_SKINNY_RING(2) MNI_SKINNY_RING(4) MNI_SKINNY_RING(8) MNI_SKINNY_RING(16)
        }
#undef MNI_SKINNY_RING
        MNI_LAUNCH_CHECK("skinny_fwd_ring_kernel");
        return MNI_B200_OK;
    }
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
    const int sliced = dx_sliced_mode();
    if (sliced > 0) {
        const unsigned sblocks = static_cast<unsigned>((K + kDxsRows - 1) / kDxsRows);
#define MNI_SKINNY_DXS(MT, P_, B_)                                                                              \
    skinny_dx_sliced_kernel<MT, P_, B_><<<sblocks, 32 * kDxsWarps, 0, stream>>>(dy, lddy, W, ldw, dx, lddx,       \
                                                                               accumulate ? 1 : 0, (int)M, N, K)
        const char *vv = getenv("MNI_B200_DXS_VARIANT");      // register / slice-width variants of the 4- and 8-row forms
        const int variant = vv && *vv ? atoi(vv) : 0;
        switch (mt) {
            case 1: MNI_SKINNY_DXS(1, 4, 2); break;
            case 2: MNI_SKINNY_DXS(2, 4, 2); break;
            case 4:
                if (variant == 1) MNI_SKINNY_DXS(4, 4, 1);
                else if (variant == 2) MNI_SKINNY_DXS(4, 4, 2);
                else MNI_SKINNY_DXS(4, 2, 2);
                break;
            case 8:
                if (variant == 1) MNI_SKINNY_DXS(8, 2, 1);
                else if (variant == 2) MNI_SKINNY_DXS(8, 2, 2);
                else MNI_SKINNY_DXS(8, 1, 2);
                break;
            default: return fail(MNI_B200_ERR_ARG, "skinny dx handles at most 8 rows");
        }
#undef MNI_SKINNY_DXS
        MNI_LAUNCH_CHECK("skinny_dx_sliced_kernel");
        return MNI_B200_OK;
    }
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
    long long slabs = std::max<long long>(1, (device_sm_count() * 8LL) / strips);
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
