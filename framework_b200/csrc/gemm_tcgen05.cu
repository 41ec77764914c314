// Tensor-core GEMM for sm_100a: C[M,N] = sum_k A[m,k] * B[n,k] on f32 storage.
//
// Data path of one CTA (persistent over output tiles, one CTA per SM):
//
//   warp 0      TMA producer: cp.async.bulk.tensor (5-D maps: 2 matrix dims + up to 3
//               batch dims) brings a 128 x BK tile of A and a BN x BK tile of B into a
//               128B/64B-swizzled shared-memory stage.  K-major and MN-major operands
//               differ only in the tensor map and the box list, so transposed / permuted
//               operands are read in place -- no transposed copy is ever written.
//   warps 2-5   split: for every f32 x of the landed stage, lo = x - trunc_tf32(x) (exact in
//               f32) is written to a sibling buffer of identical layout (the split is position
//               independent, so it needs no knowledge of the swizzle).  The landed tile itself
//               serves as hi: the tensor core ignores the low 13 mantissa bits of a TF32
//               operand (tests/test_matmul_gpu.py pins that behaviour).
//   warp 1      one thread issues tcgen05.mma.kind::tf32 per 8-deep k-step:
//               lo*hi, hi*lo, hi*hi into one f32 accumulator in TMEM ("3xTF32").  In the
//               optional fast mode the split warps idle and one MMA per k-step is issued
//               on the raw tile.
//   warps 6-9   epilogue: tcgen05.ld of the 128 x BN accumulator (double buffered in
//               TMEM, so it overlaps the next tile's main loop), transposed through a
//               padded smem patch so that global stores are row-contiguous 16-byte
//               vectors; bias add / accumulate / split-K partial output are fused here.
//
// Every wait on an mbarrier is bounded: after ~2 s worth of clock cycles the waiter
// records a code in a global error word, raises a CTA-wide abort flag and all roles
// drain to the common exit, where TMEM is released.  Nothing traps.
#include "internal.h"

#include <algorithm>
#include <mutex>

namespace mni {

namespace {

constexpr int BM = 128;
constexpr int kThreads = 320;
constexpr int kMaxStages = 8;
constexpr int kEpiPitch = 36;                        // floats per staged row (32 + 4 pad)
constexpr int kEpiBytes = 4 * 32 * kEpiPitch * 4;    // 4 epilogue warps
constexpr long long kWaitCycles = 4000000000LL;      // ~2 s at 2 GHz

struct KParams {
    int M, N;
    int tiles_m, tiles_n, group_m;
    int batch;                 // output batches
    int kiters;                // k-blocks per folded batch
    int fold;
    int splits;
    int a_batch, a_d1, a_d2;   // operand flat batch count and inner dim sizes
    int b_batch, b_d1, b_d2;
    int a_kmajor, b_kmajor;
    int bn, bk;
    int stages;
    int fast;
    uint32_t idesc;
    uint32_t a_bytes, b_bytes; // raw bytes of one stage's A / B tile
    uint32_t stage_bytes;      // whole stage incl. lo copies
    // smem descriptor constants (without start address)
    uint64_t a_desc_hi, b_desc_hi;   // upper 32 bits pre-shifted | version | layout
    uint32_t a_desc_lbo, b_desc_lbo; // (lbo >> 4) << 16, lives in the low word
    uint32_t a_kstep, b_kstep;       // descriptor address advance (16-byte units) per k-step
    float *C;
    long long ldc, c_bstride;
    float *partial;            // split-K: [split][batch][M][N]
    const float *bias;
    int accumulate;
    unsigned int *err;
};

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait.  Returns false if the CTA is aborting (this waiter or another gave up).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          unsigned int *err, uint32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitCycles) {
                *abort_flag = 1u;
                atomicCAS(err, 0u, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0,
                                            int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
        "r"(c4)
        : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
          "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
          "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
          "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct TileCoord {
    int bt, tm, tn, split, it0, it1;
};

__device__ __forceinline__ TileCoord decode_unit(const KParams &p, int unit) {
    TileCoord t;
    const int tile = unit / p.splits;
    t.split = unit - tile * p.splits;
    const int per_batch = p.tiles_m * p.tiles_n;
    t.bt = tile / per_batch;
    const int r = tile - t.bt * per_batch;
    const int group_sz = p.group_m * p.tiles_n;
    const int g = r / group_sz;
    const int first_m = g * p.group_m;
    const int gm = min(p.group_m, p.tiles_m - first_m);
    const int rin = r - g * group_sz;
    t.tn = rin / gm;
    t.tm = first_m + (rin - t.tn * gm);
    const long long total = static_cast<long long>(p.fold) * p.kiters;
    t.it0 = static_cast<int>(total * t.split / p.splits);
    t.it1 = static_cast<int>(total * (t.split + 1) / p.splits);
    return t;
}

__device__ __forceinline__ void batch_coords(int q, int cnt, int d1, int d2, int &c0, int &c1, int &c2) {
    q = cnt == 1 ? 0 : q % cnt;
    c2 = q % d2;
    const int r = q / d2;
    c1 = r % d1;
    c0 = r / d1;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const KParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint8_t *stage_base = smem;
    float *epi_stage = reinterpret_cast<float *>(smem + static_cast<size_t>(p.stages) * p.stage_bytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(epi_stage) + kEpiBytes);
    // bars: full[S] | xform[S] | empty[S] | acc_full[2] | acc_empty[2]
    const uint32_t bar_full = smem_u32(bars);
    const uint32_t bar_xform = bar_full + 8u * kMaxStages;
    const uint32_t bar_empty = bar_xform + 8u * kMaxStages;
    const uint32_t bar_acc_full = bar_empty + 8u * kMaxStages;
    const uint32_t bar_acc_empty = bar_acc_full + 16u;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * kMaxStages + 4);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t tmem_cols = static_cast<uint32_t>(2 * p.bn);   // 128 / 256 / 512

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(bar_full + 8u * s, 1);
            mbar_init(bar_xform + 8u * s, 128);
            mbar_init(bar_empty + 8u * s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_acc_full + 8u * i, 1);
            mbar_init(bar_acc_empty + 8u * i, 128);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_units = p.batch * p.tiles_m * p.tiles_n * p.splits;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int armed = 0;
            bool ok = true;
            const uint32_t tx = p.a_bytes + p.b_bytes;
            const uint32_t a_chunk = 128u * p.bk;   // bytes of one 32-wide MN chunk
            for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
                const TileCoord t = decode_unit(p, unit);
                for (int it = t.it0; it < t.it1; ++it) {
                    ok = mbar_wait(bar_empty + 8u * stage, phase ^ 1u, abort_flag, p.err, 0x100u | stage);
                    if (!ok) break;
                    const uint32_t full = bar_full + 8u * stage;
                    mbar_arrive_expect_tx(full, tx);
                    ++armed;
                    const int f = it / p.kiters;
                    const int k0 = (it - f * p.kiters) * p.bk;
                    const int q = t.bt * p.fold + f;
                    const uint32_t dstA = smem_u32(stage_base + static_cast<size_t>(stage) * p.stage_bytes);
                    const uint32_t dstB = dstA + p.a_bytes;
                    int c0, c1, c2;
                    batch_coords(q, p.a_batch, p.a_d1, p.a_d2, c0, c1, c2);
                    if (p.a_kmajor) {
                        tma_load_5d(dstA, &tmA, full, k0, t.tm * BM, c2, c1, c0);
                    } else {
                        for (int c = 0; c < BM / 32; ++c)
                            tma_load_5d(dstA + c * a_chunk, &tmA, full, t.tm * BM + c * 32, k0, c2, c1, c0);
                    }
                    batch_coords(q, p.b_batch, p.b_d1, p.b_d2, c0, c1, c2);
                    if (p.b_kmajor) {
                        tma_load_5d(dstB, &tmB, full, k0, t.tn * p.bn, c2, c1, c0);
                    } else {
                        for (int c = 0; c < p.bn / 32; ++c)
                            tma_load_5d(dstB + c * a_chunk, &tmB, full, t.tn * p.bn + c * 32, k0, c2, c1, c0);
                    }
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // Aborting: let the copies already issued land before the CTA exits.
                const int pending = min(armed, p.stages);
                for (int i = 0; i < pending; ++i) {
                    if (--stage < 0) { stage = p.stages - 1; phase ^= 1u; }
                    const long long t0 = clock64();
                    while (!mbar_try_wait(bar_full + 8u * stage, phase) && clock64() - t0 < kWaitCycles / 8) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc_it = 0;
            bool ok = true;
            const int ksteps = p.bk / 8;
            const uint32_t lo_off = (p.a_bytes + p.b_bytes) >> 4;   // lo copy of the stage, 16-byte units
            for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
                const TileCoord t = decode_unit(p, unit);
                const int buf = acc_it & 1;
                const uint32_t acc_phase = (acc_it >> 1) & 1;
                ok = mbar_wait(bar_acc_empty + 8u * buf, acc_phase ^ 1u, abort_flag, p.err, 0x200u | buf);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * p.bn);
                uint32_t accumulate = 0;
                for (int it = t.it0; it < t.it1; ++it) {
                    const uint32_t ready = (p.fast ? bar_full : bar_xform) + 8u * stage;
                    ok = mbar_wait(ready, phase, abort_flag, p.err, 0x300u | stage);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(stage_base + static_cast<size_t>(stage) * p.stage_bytes);
                    const uint32_t a_lo32 = ((sa >> 4) & 0x3FFFu) | p.a_desc_lbo;
                    const uint32_t b_lo32 = (((sa + p.a_bytes) >> 4) & 0x3FFFu) | p.b_desc_lbo;
                    for (int ks = 0; ks < ksteps; ++ks) {
                        const uint64_t a_hi = p.a_desc_hi | (a_lo32 + ks * p.a_kstep);
                        const uint64_t b_hi = p.b_desc_hi | (b_lo32 + ks * p.b_kstep);
                        if (p.fast) {
                            umma_tf32(d_tmem, a_hi, b_hi, p.idesc, accumulate);
                        } else {
                            const uint64_t a_lo = a_hi + lo_off;
                            const uint64_t b_lo = b_hi + lo_off;
                            umma_tf32(d_tmem, a_lo, b_hi, p.idesc, accumulate);
                            umma_tf32(d_tmem, a_hi, b_lo, p.idesc, 1u);
                            umma_tf32(d_tmem, a_hi, b_hi, p.idesc, 1u);
                        }
                        accumulate = 1u;
                    }
                    umma_commit(bar_empty + 8u * stage);
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(bar_acc_full + 8u * buf);
                ++acc_it;
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ hi/lo split
        if (!p.fast) {
            const int tid = threadIdx.x - 64;
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const int n4 = static_cast<int>((p.a_bytes + p.b_bytes) >> 4);
            for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
                const TileCoord t = decode_unit(p, unit);
                for (int it = t.it0; it < t.it1; ++it) {
                    ok = mbar_wait(bar_full + 8u * stage, phase, abort_flag, p.err, 0x400u | stage);
                    if (!ok) break;
                    float4 *raw = reinterpret_cast<float4 *>(stage_base + static_cast<size_t>(stage) * p.stage_bytes);
                    float4 *lo = raw + n4;
#pragma unroll 4
                    for (int i = tid; i < n4; i += 128) {
                        // The tensor core reads only the TF32 bits of a 32-bit operand (the low 13
                        // mantissa bits are ignored), so the landed tile already is "hi"; only the
                        // residual lo = x - trunc(x), exact in f32, has to be written.
                        const float4 v = raw[i];
                        float4 l;
                        l.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
                        l.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
                        l.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
                        l.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
                        lo[i] = l;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    mbar_arrive(bar_xform + 8u * stage);
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;                       // TMEM lane quarter this warp may read
        float *stg = epi_stage + (warp - 6) * 32 * kEpiPitch;
        int acc_it = 0;
        bool ok = true;
        const bool vec_ok = ((p.ldc & 3) == 0) && ((p.c_bstride & 3) == 0) &&
                            ((reinterpret_cast<uintptr_t>(p.splits > 1 ? p.partial : p.C) & 15) == 0) &&
                            (p.splits == 1 || (p.N & 3) == 0);
        for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
            const TileCoord t = decode_unit(p, unit);
            const int buf = acc_it & 1;
            const uint32_t acc_phase = (acc_it >> 1) & 1;
            ok = mbar_wait(bar_acc_full + 8u * buf, acc_phase, abort_flag, p.err, 0x500u | buf);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            float *out;
            long long ld;
            if (p.splits > 1) {
                ld = p.N;
                out = p.partial + (static_cast<long long>(t.split) * p.batch + t.bt) * p.M * ld;
            } else {
                ld = p.ldc;
                out = p.C + static_cast<long long>(t.bt) * p.c_bstride;
            }
            const bool fuse = p.splits == 1;
            const int row_base = t.tm * BM + q * 32;
            const int rsub = lane >> 3;               // 0..3
            const int c4 = (lane & 7) * 4;            // 0,4,..,28
            for (int chunk = 0; chunk < p.bn / 32; ++chunk) {
                const int col0 = t.tn * p.bn + chunk * 32;
                if (col0 >= p.N) break;               // warp-uniform
                uint32_t v[32];
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                       static_cast<uint32_t>(buf * p.bn + chunk * 32);
                tmem_ld32(taddr, v);
                float4 *srow = reinterpret_cast<float4 *>(stg + lane * kEpiPitch);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    srow[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                          __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                __syncwarp();
                const int col = col0 + c4;
                float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (fuse && p.bias != nullptr) {
                    if (col + 0 < p.N) bv.x = __ldg(p.bias + col + 0);
                    if (col + 1 < p.N) bv.y = __ldg(p.bias + col + 1);
                    if (col + 2 < p.N) bv.z = __ldg(p.bias + col + 2);
                    if (col + 3 < p.N) bv.w = __ldg(p.bias + col + 3);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = i * 4 + rsub;
                    const int row = row_base + r;
                    if (row >= p.M || col >= p.N) continue;
                    float4 x = *reinterpret_cast<const float4 *>(stg + r * kEpiPitch + c4);
                    x.x += bv.x; x.y += bv.y; x.z += bv.z; x.w += bv.w;
                    float *dst = out + static_cast<long long>(row) * ld + col;
                    if (vec_ok && col + 3 < p.N) {
                        if (fuse && p.accumulate) {
                            const float4 o = *reinterpret_cast<const float4 *>(dst);
                            x.x += o.x; x.y += o.y; x.z += o.z; x.w += o.w;
                        }
                        *reinterpret_cast<float4 *>(dst) = x;
                    } else {
                        const float xs[4] = {x.x, x.y, x.z, x.w};
                        for (int e = 0; e < 4; ++e) {
                            if (col + e < p.N) {
                                float y = xs[e];
                                if (fuse && p.accumulate) y += dst[e];
                                dst[e] = y;
                            }
                        }
                    }
                }
                __syncwarp();
            }
            tc_fence_before();
            mbar_arrive(bar_acc_empty + 8u * buf);
            ++acc_it;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols)
                     : "memory");
    }
}

// Deterministic split-K finish: C = sum_s partial[s] (+ bias) (+ C).
__global__ void splitk_reduce_kernel(const float *__restrict__ partial, float *__restrict__ C, long long ldc,
                                     long long c_bstride, const float *__restrict__ bias, int accumulate,
                                     int splits, long long batch, int M, int N) {
    const long long total = batch * M * N;
    const long long slab = total;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int col = static_cast<int>(i % N);
        const long long r = i / N;
        const int row = static_cast<int>(r % M);
        const long long bt = r / M;
        float acc = partial[i];
        for (int s = 1; s < splits; ++s) acc += partial[s * slab + i];
        if (bias) acc += __ldg(bias + col);
        float *dst = C + bt * c_bstride + static_cast<long long>(row) * ldc + col;
        if (accumulate) acc += *dst;
        *dst = acc;
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

int make_map(CUtensorMap *map, const Operand &op, int box_rows, int bk) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(MNI_B200_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
    cuuint64_t dims[5];
    cuuint64_t strides[4];   // bytes, dims 1..4
    cuuint32_t box[5] = {1, 1, 1, 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUtensorMapSwizzle swz;
    if (op.k_major) {
        dims[0] = static_cast<cuuint64_t>(op.kdim);
        dims[1] = static_cast<cuuint64_t>(op.rows);
        box[0] = static_cast<cuuint32_t>(bk);
        box[1] = static_cast<cuuint32_t>(box_rows);
        swz = bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    } else {
        dims[0] = static_cast<cuuint64_t>(op.rows);
        dims[1] = static_cast<cuuint64_t>(op.kdim);
        box[0] = 32;
        box[1] = static_cast<cuuint32_t>(bk);
        // 32-bit elements read MN-major by the tensor core use the 128-byte swizzle whose unit
        // is a 32-byte chunk (8 k-steps' worth of one row pair), not the usual 16-byte chunk.
        swz = static_cast<CUtensorMapSwizzle>(env_int("MNI_B200_DEBUG_MN_TMA_SWIZZLE",
                                                      static_cast<int>(CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)));
    }
    // A size-1 dim never advances, but its stride must still be a positive multiple of 16 bytes.
    uint64_t span = 16;
    auto stride_or = [&](int64_t extent, int64_t stride_elems) -> cuuint64_t {
        uint64_t s = (extent > 1 && stride_elems > 0) ? static_cast<uint64_t>(stride_elems) * 4u : span;
        return static_cast<cuuint64_t>(s);
    };
    span = std::max<uint64_t>(16, (static_cast<uint64_t>(dims[0]) * 4u + 15u) & ~15ull);
    strides[0] = stride_or(static_cast<int64_t>(dims[1]), op.ld);
    span = std::max<uint64_t>(span, strides[0] * dims[1]);
    for (int i = 0; i < 3; ++i) {   // map dim 2 = innermost batch dim
        const int bi = 2 - i;
        dims[2 + i] = static_cast<cuuint64_t>(op.bshape[bi]);
        strides[1 + i] = stride_or(op.bshape[bi], op.bstride[bi]);
        span = std::max<uint64_t>(span, strides[1 + i] * dims[2 + i]);
    }
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float *>(op.ptr), dims, strides, box,
                     estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(MNI_B200_ERR_CUDA,
                    "cuTensorMapEncodeTiled failed (%d): dims %llu x %llu, ld %lld, k_major %d", static_cast<int>(r),
                    static_cast<unsigned long long>(dims[0]), static_cast<unsigned long long>(dims[1]),
                    static_cast<long long>(op.ld), static_cast<int>(op.k_major));
    return MNI_B200_OK;
}

struct Plan {
    int bn, bk, stages, splits, tiles_m, tiles_n, grid;
    size_t smem;
};

Plan make_plan(const GemmProblem &p, int sm_count) {
    Plan pl;
    pl.bn = p.N <= 64 ? 64 : (p.N <= 128 ? 128 : 256);
    const int bn_env = env_int("MNI_B200_BN", 0);
    if (bn_env == 64 || bn_env == 128 || bn_env == 256) pl.bn = bn_env;
    pl.bk = (pl.bn == 256 && !p.fast_tf32) ? 16 : 32;
    const int bk_env = env_int("MNI_B200_BK", 0);
    if (bk_env == 16 || bk_env == 32) pl.bk = bk_env;
    const size_t raw = static_cast<size_t>(BM + pl.bn) * pl.bk * 4;
    const size_t stage = p.fast_tf32 ? raw : 2 * raw;
    const size_t fixed = 1024 + kEpiBytes + (3 * kMaxStages + 4) * 8 + 16;
    const size_t budget = 227 * 1024;
    pl.stages = static_cast<int>(std::min<size_t>(kMaxStages, (budget - fixed) / stage));
    const int st_env = env_int("MNI_B200_STAGES", 0);
    if (st_env >= 1 && st_env <= pl.stages) pl.stages = st_env;
    pl.smem = fixed + static_cast<size_t>(pl.stages) * stage;
    pl.tiles_m = static_cast<int>((p.M + BM - 1) / BM);
    pl.tiles_n = static_cast<int>((p.N + pl.bn - 1) / pl.bn);
    const long long tiles = static_cast<long long>(p.batch) * pl.tiles_m * pl.tiles_n;
    const long long iters = p.fold * ((p.K + pl.bk - 1) / pl.bk);
    int splits = 1;
    if (p.force_splits > 0) {
        splits = p.force_splits;
    } else if (tiles * 2 <= sm_count && iters >= 8) {
        // Few output tiles and a long contraction: split K so that the whole GPU works.
        splits = static_cast<int>(std::min<long long>(sm_count / tiles, iters / 4));
    }
    splits = static_cast<int>(std::max<long long>(1, std::min<long long>(std::min<long long>(splits, iters), 64)));
    pl.splits = splits;
    const long long units = tiles * splits;
    pl.grid = static_cast<int>(std::min<long long>(units, sm_count));
    return pl;
}

uint64_t desc_hi_bits(uint32_t sbo_bytes, uint32_t layout_type) {
    return (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) |
           (static_cast<uint64_t>(layout_type) << 61);
}

}  // namespace

size_t gemm_tc_partial_bytes(const GemmProblem &p, int sm_count) {
    const Plan pl = make_plan(p, sm_count);
    if (pl.splits <= 1) return 0;
    return static_cast<size_t>(pl.splits) * p.batch * p.M * p.N * sizeof(float);
}

int launch_gemm_tc(const GemmProblem &p, float *partial, uint32_t *err_word, int sm_count,
                   cudaStream_t stream) {
    if (p.M <= 0 || p.N <= 0 || p.batch <= 0) return MNI_B200_OK;
    const Plan pl = make_plan(p, sm_count);
    if (p.K <= 0) {
        // Empty contraction: the product is all zeros (ops/matmul.rs:48 starts from a zeroed output).
        return fail(MNI_B200_ERR_ARG, "empty contraction reached the tensor-core launcher");
    }
    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, [] {
        attr_err = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    });
    if (attr_err != cudaSuccess)
        return fail(MNI_B200_ERR_CUDA, "cudaFuncSetAttribute(smem) failed: %s", cudaGetErrorString(attr_err));

    CUtensorMap tmA, tmB;
    int rc = make_map(&tmA, p.A, BM, pl.bk);
    if (rc) return rc;
    rc = make_map(&tmB, p.B, pl.bn, pl.bk);
    if (rc) return rc;

    KParams k{};
    k.M = static_cast<int>(p.M);
    k.N = static_cast<int>(p.N);
    k.tiles_m = pl.tiles_m;
    k.tiles_n = pl.tiles_n;
    k.group_m = std::max(1, std::min(pl.tiles_m, env_int("MNI_B200_GROUP_M", 16)));
    k.batch = static_cast<int>(p.batch);
    k.kiters = static_cast<int>((p.K + pl.bk - 1) / pl.bk);
    k.fold = static_cast<int>(p.fold);
    k.splits = pl.splits;
    k.a_batch = static_cast<int>(p.A.batch);
    k.a_d1 = static_cast<int>(p.A.bshape[1]);
    k.a_d2 = static_cast<int>(p.A.bshape[2]);
    k.b_batch = static_cast<int>(p.B.batch);
    k.b_d1 = static_cast<int>(p.B.bshape[1]);
    k.b_d2 = static_cast<int>(p.B.bshape[2]);
    k.a_kmajor = p.A.k_major;
    k.b_kmajor = p.B.k_major;
    k.bn = pl.bn;
    k.bk = pl.bk;
    k.stages = pl.stages;
    k.fast = p.fast_tf32;
    k.idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((p.A.k_major ? 0u : 1u) << 15) |
              ((p.B.k_major ? 0u : 1u) << 16) | (static_cast<uint32_t>(pl.bn >> 3) << 17) |
              (static_cast<uint32_t>(BM >> 4) << 24);
    k.a_bytes = static_cast<uint32_t>(BM * pl.bk * 4);
    k.b_bytes = static_cast<uint32_t>(pl.bn * pl.bk * 4);
    k.stage_bytes = (k.a_bytes + k.b_bytes) * (p.fast_tf32 ? 1u : 2u);
    // K-major tile: rows of BK floats, 8-row groups SBO apart, swizzle span = one row.
    // MN-major tile: 32-float chunks of BK k-rows (LBO apart); the 32-byte-unit swizzle repeats every
    // 4 k-rows (SBO = 512), and one 8-deep k-step spans two such groups (1024 bytes).
    const uint32_t k_layout = pl.bk == 32 ? 2u : 4u;   // SWIZZLE_128B : SWIZZLE_64B
    const uint32_t k_sbo = static_cast<uint32_t>(8 * pl.bk * 4);
    const uint32_t mn_lbo = static_cast<uint32_t>(env_int("MNI_B200_DEBUG_MN_LBO", pl.bk * 128));
    const uint32_t mn_sbo = static_cast<uint32_t>(env_int("MNI_B200_DEBUG_MN_SBO", 512));
    const uint32_t mn_layout = static_cast<uint32_t>(env_int("MNI_B200_DEBUG_MN_LAYOUT", 1));   // SWIZZLE_128B_BASE32B
    if (p.A.k_major) { k.a_desc_hi = desc_hi_bits(k_sbo, k_layout); k.a_desc_lbo = 0; k.a_kstep = 2; }
    else { k.a_desc_hi = desc_hi_bits(mn_sbo, mn_layout); k.a_desc_lbo = ((mn_lbo >> 4) & 0x3FFFu) << 16; k.a_kstep = 64; }
    if (p.B.k_major) { k.b_desc_hi = desc_hi_bits(k_sbo, k_layout); k.b_desc_lbo = 0; k.b_kstep = 2; }
    else { k.b_desc_hi = desc_hi_bits(mn_sbo, mn_layout); k.b_desc_lbo = ((mn_lbo >> 4) & 0x3FFFu) << 16; k.b_kstep = 64; }
    k.C = p.C;
    k.ldc = p.ldc;
    k.c_bstride = p.c_bstride;
    k.partial = partial;
    k.bias = p.bias;
    k.accumulate = p.accumulate;
    k.err = err_word;
    if (pl.splits > 1 && partial == nullptr)
        return fail(MNI_B200_ERR_WORKSPACE, "split-K launch without partial storage");

    gemm_tc_kernel<<<pl.grid, kThreads, pl.smem, stream>>>(tmA, tmB, k);
    MNI_LAUNCH_CHECK("gemm_tc_kernel");
    if (pl.splits > 1) {
        const long long total = static_cast<long long>(p.batch) * p.M * p.N;
        const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 148 * 8));
        splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(partial, p.C, p.ldc, p.c_bstride, p.bias, p.accumulate,
                                                         pl.splits, p.batch, k.M, k.N);
        MNI_LAUNCH_CHECK("splitk_reduce_kernel");
    }
    return MNI_B200_OK;
}

}  // namespace mni
