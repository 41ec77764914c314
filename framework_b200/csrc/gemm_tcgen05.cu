// Tensor-core GEMM for sm_100a: C[M,N] = sum_k A[m,k] * B[n,k] on f32 storage.
//
// Data path of one CTA (persistent over output tiles, one CTA per SM; 2 + NS + 8 warps):
//
//   warp 0      TMA producer: cp.async.bulk.tensor (5-D maps: matrix dims + batch dims) brings
//               a 128 x BK tile of A and a BN x BK tile of B into a swizzled shared-memory
//               stage.  K-major and MN-major operands differ only in the tensor map and the
//               box list, so transposed / permuted operands are read in place -- no transposed
//               copy is ever written.
//   warps 2..   split (NS = 8 warps; 4 idle relays in single-pass mode): for every f32 x of the
//               landed stage, lo = x - trunc_tf32(x) (exact in f32) is written to a sibling buffer
//               of identical layout (the split is position independent, so it needs no knowledge
//               of the swizzle).  The landed tile itself serves as hi: the tensor core ignores the
//               low 13 mantissa bits of a TF32 operand (tests/test_matmul_gpu.py pins that).
//               Narrow tiles (BN <= 128, lone CTA) instead move A into tensor memory: each thread
//               reads 16 k-values of its row and stores hi and lo with tcgen05.st; only B keeps a
//               lo copy in shared memory.  For long contractions the eight warps take alternate
//               k-blocks as two groups of four (SG = 2), so two k-blocks are in flight.  When the
//               tile is wider than the output, MMAs, B box and lo copy cover only the live columns.
//   warp 1      issues tcgen05.mma.kind::tf32 per 8-deep k-step: lo*hi, hi*lo, hi*hi into one f32
//               accumulator in TMEM ("3xTF32"); one MMA on the raw tile in single-pass mode.  The
//               warp runs its loop uniformly and predicates the issue with elect.sync, and it reads
//               the next stage's barrier before queueing this stage's MMAs.
//   last 8      epilogue, two warps per TMEM lane quarter, half of the tile's columns each:
//               tcgen05.ld of the accumulator (double buffered in TMEM, so it overlaps the next
//               tile's main loop), bias add in registers, 128B-swizzled staging patch, TMA store
//               (or TMA reduce-add for C += ...) of 32 x 32 boxes; the tensor map clips the M / N
//               tails.  Split-K partials go through the same path into scratch.  Outputs whose row
//               pitch is not a multiple of 16 bytes take a plain-store fallback.
//
// CG = 2: two CTAs of a cluster share a 256 x BN tile (cta_group::2 MMAs issued by the leader).
// Work is dealt out as whole tiles, round-robin over the CTAs (pairs); a badly ragged last wave is cut
// into equal ranges of k-blocks instead, and a tile shared by several CTAs is summed in slot order
// by whichever of them finishes last (tickets and flags in global memory, bounded waits).
//
// The tensor core's f32 accumulate rounds toward zero (measured: 2.35e-9 * K relative per chain, three
// chains' worth in 3xTF32), so a long contraction is not summed in one accumulator: a unit is handed
// out in pieces of at most KParams::chunk_iters k-blocks, each piece gets a fresh accumulator, and the
// epilogue adds the later pieces to the output with ordered TMA reduce-adds (fixed order: reproducible).
//
// Every wait on an mbarrier or flag is bounded: after KParams::wait_cycles clock cycles (~2 s unless a
// test shortens it) the waiter records a code in a global error word, raises a CTA-wide abort flag and
// all roles drain to the common exit, where TMEM is released.  Nothing traps.
#include "internal.h"

#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <unordered_map>

namespace mni {

namespace {

constexpr int BM = 128;
constexpr int kMaxStages = 8;
constexpr int kSkMaxShare = 6;                             // balanced tail: most units that may share one tile
constexpr int kEpiWarps = 8;                                // two per TMEM lane quarter, half of the columns each
constexpr int kEpiBufBytes = 32 * 128;                     // one 32 x 32 f32 patch
constexpr int kBarBytes = (3 * kMaxStages + 4) * 8 + 16;
constexpr long long kWaitCycles = 4000000000LL;            // default limit of every device-side wait: ~2 s at 2 GHz

enum OperandMode { kKMajor = 0, kMnMultiBox = 1, kMnSingleBox = 2 };
enum EpilogueMode { kEpiPlainStores = 0, kEpiTmaStore = 1, kEpiTmaReduce = 2, kEpiVectorStores = 3 };

// Division by a launch-time constant as a multiply-high and a shift (exact for 0 <= n < 2^31): every role
// decodes every tile it visits, and with short contractions a handful of hardware divisions per tile showed
// up as 1 250 cycles of a 3 000-cycle main loop.  mul = ceil(2^(31 + ceil(log2 d)) / d), shr = ceil(log2 d) - 1.
struct FastDiv {
    uint32_t mul, shr, d;
};
__host__ inline FastDiv make_fastdiv(long long d_in) {
    FastDiv f;
    const uint32_t d = static_cast<uint32_t>(d_in < 1 ? 1 : d_in);
    f.d = d;
    if (d == 1) { f.mul = 0; f.shr = 0; return f; }
    uint32_t l = 0;
    while ((1ull << l) < d) ++l;
    const uint32_t p = 31 + l;
    f.mul = static_cast<uint32_t>(((1ull << p) + d - 1) / d);
    f.shr = p - 32;
    return f;
}
__device__ __forceinline__ int fd_div(int n, const FastDiv &f) {
    return f.d == 1 ? n : static_cast<int>(__umulhi(static_cast<uint32_t>(n), f.mul) >> f.shr);
}

struct KParams {
    int M, N;
    int tiles_m, tiles_n, group_m;
    int batch;                 // output batches
    int kiters;                // k-blocks per folded batch
    int fold;
    int splits;
    int dep_mode;              // 0: depends on everything before it; 1 / 2: first / second of two independent products (see GemmProblem)
    int chunk_iters;           // longest run of k-blocks summed in one tensor-memory accumulator (0 = no limit)
    int a_batch, a_d1, a_d2;   // operand flat batch count and inner dim sizes
    int b_batch, b_d1, b_d2;
    int a_mode, b_mode;        // OperandMode
    int stages;
    int epi_mode;              // EpilogueMode
    int epi_patches;           // staging patches per epilogue warp: TMA stores in flight per warp
    uint32_t idesc;
    // A tile wider than the output (lone CTA, K-major B): the B box, the lo copy and the MMAs cover only the rows
    // that exist.  b_rows_live = rows of the B tile that are loaded and split (the tile's width otherwise).
    int b_rows_live;
    uint32_t a_desc_hi, b_desc_hi;   // upper 32 bits of the smem descriptors (SBO | version | layout)
    uint32_t a_desc_lbo, b_desc_lbo; // LBO field, already shifted into the low word
    uint32_t a_kstep, b_kstep;       // descriptor address advance (16-byte units) per 8-deep k-step
    float *C;
    long long ldc, c_bstride;
    float *partial;            // split-K: [split][batch][M][N]
    const float *bias;
    int accumulate;
    int transpose_out;         // the kernel computes C^T (operands exchanged): patches are stored transposed, bias is per row
    int act;                   // 1: also emit gelu(acc + bias) through the second output map
    int store_pre;             // act mode: write the raw product through the first map as well
    FastDiv fd_splits, fd_per_batch, fd_group_sz, fd_group_m, fd_last_gm;   // decode_unit
    FastDiv fd_a_cnt, fd_a_d1, fd_a_d2, fd_b_cnt, fd_b_d1, fd_b_d2;         // batch_coords
    unsigned int *err;
    long long wait_cycles;     // limit of every bounded wait in clock cycles (kWaitCycles unless a test shortens it)
    int withhold_at;           // test hook: the producer arms its n-th k-block (1-based) but issues no copy for it; 0 = off
    unsigned long long *prof;  // optional role wait counters (null = off)
    // Balanced tail ("stream-K"): tiles [sk_first_tile, tiles) are not dealt out whole; their k-blocks are
    // cut into one contiguous range per CTA (pair), so a ragged last wave costs its share, not a full wave.
    int sk;                    // 0 = off
    int sk_first_tile;         // tiles below this index are dealt out whole, round-robin
    float *sk_partial;         // two parked accumulator tiles per CTA: [cta][2][epilogue warp][chunk][8][lane] float4
    unsigned int *sk_flags;    // ready flags [cta][2][epilogue warp] (1 = parked), then tickets [tile][rank][epilogue warp]
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
// With `timed`, `waited` accumulates the cycles spent blocked (role-level wait accounting, including
// the time the first try_wait is suspended by the hardware); without it the satisfied case costs one
// try_wait and no clock reads.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          unsigned int *err, uint32_t code, long long &waited, bool timed,
                                          long long limit) {
    long long t0 = 0;
    if (timed) t0 = clock64();
    if (mbar_try_wait(bar, parity)) {
        if (timed) waited += clock64() - t0;
        return true;
    }
    if (!timed) t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) {
            if (timed) waited += clock64() - t0;
            return true;
        }
        if ((++spins & 63u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit) {
                *abort_flag = 1u;
                atomicCAS(err, 0u, code);
                return false;
            }
        }
    }
}
// Warp-collective form: every lane polls, the verdict is made uniform.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                               unsigned int *err, uint32_t code, long long &waited, bool timed,
                                               long long limit) {
    const bool ok = mbar_wait(bar, parity, abort_flag, err, code, waited, timed, limit);
    return __all_sync(0xffffffffu, ok);
}
// Non-blocking look at a barrier phase (try_wait may suspend the thread; this never does).
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// True in exactly one lane of a converged warp.  The TMA and MMA issuing warps run their loops
// warp-uniformly and predicate only the issuing instruction with this: descriptors and
// coordinates then stay in uniform registers, which makes an MMA issue ~3x cheaper than from a
// single-lane branch (measured: 40 vs 120 cycles).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
        "elect.sync rx|px, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, px;\n\t}"
        : "=r"(pred));
    return pred != 0;
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
__device__ __forceinline__ void tma_store_5d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(0), "r"(0)
                 : "memory");
}
__device__ __forceinline__ void tma_reduce_add_5d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.5d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(0), "r"(0)
        : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                          uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// A operand from tensor memory (lanes = rows, one 32-bit column per k element), B from shared memory.
__device__ __forceinline__ void umma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                             uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
// ---- CTA-pair (cta_group::2) forms: one MMA spans two SMs; the leader CTA issues it.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `cta` of the cluster.
__device__ __forceinline__ void mbar_arrive_cta(uint32_t bar, uint32_t cta) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(bar), "r"(cta)
        : "memory");
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Commit that arrives on the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(static_cast<uint16_t>(3))
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&v)[32]) {
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
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// gelu(v) = 0.5 v (1 + tanh(sqrt(2/pi) (v + 0.044715 v^3)))   (kernels/fused_ops.cu:66-82)
__device__ __forceinline__ float gelu_tanh_f(float v) {
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(inner));
}

struct TileCoord {
    int bt, tm, tn, split, it0, it1;
    int shared;      // balanced tail: this unit is only a range of the tile's k-blocks
    int park;        // shared: which of the CTA's two parking places it uses (0 = first unit of its range)
    int tile;        // flat tile index
    int chunk;       // > 0: a later piece of a unit whose contraction is summed in several accumulators (added to the output)
};

__device__ __forceinline__ TileCoord decode_unit(const KParams &p, int unit) {
    TileCoord t;
    const int tile = fd_div(unit, p.fd_splits);
    t.split = unit - tile * p.splits;
    t.shared = 0;
    t.park = 0;
    t.chunk = 0;
    t.tile = tile;
    const int per_batch = p.tiles_m * p.tiles_n;
    t.bt = fd_div(tile, p.fd_per_batch);
    const int r = tile - t.bt * per_batch;
    const int group_sz = p.group_m * p.tiles_n;
    const int g = fd_div(r, p.fd_group_sz);
    const int first_m = g * p.group_m;
    const int gm = min(p.group_m, p.tiles_m - first_m);       // the last group may be shorter
    const int rin = r - g * group_sz;
    t.tn = gm == p.group_m ? fd_div(rin, p.fd_group_m) : fd_div(rin, p.fd_last_gm);
    t.tm = first_m + (rin - t.tn * gm);
    const int total = p.fold * p.kiters;
    if (p.splits == 1) {
        t.it0 = 0;
        t.it1 = total;
    } else {
        t.it0 = static_cast<int>(static_cast<long long>(total) * t.split / p.splits);
        t.it1 = static_cast<int>(static_cast<long long>(total) * (t.split + 1) / p.splits);
    }
    return t;
}

// The work of one CTA (pair), in the order every role walks it: whole tiles slot, slot + P, ... and then,
// with the balanced tail on, this slot's contiguous range of the tail's k-blocks, which touches at most the
// end of one tile, whole tiles, and the beginning of one tile.
struct WorkIter {
    int unit, unit_step, unit_end;     // whole units
    long long w0, w, w1;               // tail range in k-blocks, relative to the tail's first tile
    // A unit with a long contraction is handed out as consecutive pieces of at most p.chunk_iters k-blocks:
    // the tensor core's f32 accumulate truncates, so one long chain loses ~7e-9 * K of relative accuracy;
    // every piece gets a fresh accumulator and the epilogue adds it to the output (round-to-nearest adds).
    TileCoord cur;                     // the unit being handed out in pieces
    int piece_it, piece_end, piece_len, piece_no;
};
__device__ __forceinline__ long long sk_range_begin(const KParams &p, int slot, int nslots) {
    const long long total = static_cast<long long>(p.batch * p.tiles_m * p.tiles_n - p.sk_first_tile) * (p.fold * p.kiters);
    return total * slot / nslots;
}
__device__ __forceinline__ WorkIter work_begin(const KParams &p, int slot, int nslots) {
    WorkIter wi;
    wi.unit = slot;
    wi.unit_step = nslots;
    wi.unit_end = p.sk ? p.sk_first_tile : p.batch * p.tiles_m * p.tiles_n * p.splits;
    wi.w0 = wi.w = wi.w1 = 0;
    wi.piece_it = wi.piece_end = wi.piece_len = wi.piece_no = 0;
    if (p.sk) {
        wi.w0 = wi.w = sk_range_begin(p, slot, nslots);
        wi.w1 = sk_range_begin(p, slot + 1, nslots);
    }
    return wi;
}
__device__ __forceinline__ TileCoord decode_unit(const KParams &p, int unit);
// Cuts a long unit into equal pieces of at most p.chunk_iters k-blocks: `t` becomes the first piece, the iterator
// remembers the rest.
__device__ __forceinline__ void first_piece(const KParams &p, WorkIter &wi, TileCoord &t) {
    const int len = t.it1 - t.it0;
    if (p.chunk_iters > 0 && len > p.chunk_iters + (p.chunk_iters >> 1)) {
        const int pieces = (len + p.chunk_iters - 1) / p.chunk_iters;
        wi.cur = t;
        wi.piece_len = (len + pieces - 1) / pieces;
        wi.piece_end = t.it1;
        wi.piece_no = 0;
        t.it1 = t.it0 + wi.piece_len;
        wi.piece_it = t.it1;
    }
}
__device__ __forceinline__ bool work_next(const KParams &p, WorkIter &wi, TileCoord &t) {
    if (wi.piece_it < wi.piece_end) {          // next piece of the current unit
        t = wi.cur;
        t.it0 = wi.piece_it;
        t.it1 = min(wi.piece_end, wi.piece_it + wi.piece_len);
        t.chunk = ++wi.piece_no;
        wi.piece_it = t.it1;
        return true;
    }
    if (wi.unit < wi.unit_end) {
        t = decode_unit(p, wi.unit);
        wi.unit += wi.unit_step;
        first_piece(p, wi, t);
        return true;
    }
    if (wi.w < wi.w1) {
        const int per_tile = p.fold * p.kiters;
        const int rel = static_cast<int>(wi.w / per_tile);
        const int it0 = static_cast<int>(wi.w - static_cast<long long>(rel) * per_tile);
        const int it1 = static_cast<int>(min(static_cast<long long>(per_tile), it0 + (wi.w1 - wi.w)));
        t = decode_unit(p, p.sk_first_tile + rel);          // splits == 1 here: unit == tile
        t.it0 = it0;
        t.it1 = it1;
        t.shared = (it0 != 0 || it1 != per_tile) ? 1 : 0;
        t.park = wi.w == wi.w0 ? 0 : 1;
        wi.w += it1 - it0;
        // A whole tile inside a tail range is summed in pieces like any other unit; a cut tile is not (its one
        // accumulator is what gets parked or reduced), so its chain is as long as its share of the contraction.
        if (!t.shared) first_piece(p, wi, t);
        return true;
    }
    return false;
}

__device__ __forceinline__ void batch_coords(int q, int cnt, int d1, int d2, const FastDiv &fcnt, const FastDiv &fd1,
                                             const FastDiv &fd2, int &c0, int &c1, int &c2) {
    q = cnt == 1 ? 0 : q - fd_div(q, fcnt) * cnt;
    const int r = fd_div(q, fd2);
    c2 = q - r * d2;
    c0 = fd_div(r, fd1);
    c1 = r - c0 * d1;
}

// Issues the TMA copies of one operand tile.  row0 = first row of the tile, nchunk = tile rows / 32.
__device__ __forceinline__ void load_operand(int mode, uint32_t dst, const CUtensorMap *map, uint32_t bar, int k0,
                                             int row0, int nchunk, uint32_t chunk_bytes, int c0, int c1, int c2) {
    if (mode == kKMajor) {
        tma_load_5d(dst, map, bar, k0, row0, c2, c1, c0);
    } else if (mode == kMnSingleBox) {
        tma_load_5d(dst, map, bar, 0, k0, row0 >> 5, c2, c1);
    } else {
        for (int c = 0; c < nchunk; ++c) tma_load_5d(dst + c * chunk_bytes, map, bar, row0 + c * 32, k0, c2, c1, c0);
    }
}

// CG = 1: one CTA computes a 128 x BN tile.  CG = 2: a pair of CTAs (a 2-CTA cluster) computes a
// 256 x BN tile with cta_group::2 MMAs issued by the pair's leader; each CTA stages its own 128 rows
// of A and half (BN/2 rows) of B, so shared-memory and L2 traffic per flop drop by a third.
// TA = true (3xTF32, lone CTA, BK = 32, BN <= 128): the A operand of the MMAs comes from tensor memory.
// The split warps read each landed A row once, and store hi and lo with tcgen05.st into a TMEM slot
// of the stage (columns 2*BN + stage*64: 32 of hi, 32 of lo); no lo copy of A is written to shared
// memory and no MMA re-reads A from it, which is what bounds narrow tiles otherwise.
// SK = true compiles the balanced-tail epilogue (parking / reducing shared tiles) in; the other
// instantiations carry none of its code or registers.
// SG = 2 (TA only): the split warps work as two groups on alternate k-blocks (see the split role).
template <int BN, int BK, bool FAST, int NS, int CG, bool TA = false, bool SK = false, int SG = 1>
__global__ void __launch_bounds__(32 * (2 + NS + kEpiWarps), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmD,
               const KParams p) {
    constexpr int BNL = BN / CG;                           // B rows staged by this CTA
    constexpr uint32_t A_BYTES = BM * BK * 4;
    constexpr uint32_t B_BYTES = BNL * BK * 4;
    constexpr uint32_t RAW_BYTES = A_BYTES + B_BYTES;
    static_assert(!TA || (!FAST && CG == 1 && BK == 32 && NS == 8 && BN <= 128), "unsupported A-from-TMEM variant");
    constexpr uint32_t STAGE_BYTES = FAST ? RAW_BYTES : (TA ? A_BYTES + 2 * B_BYTES : 2 * RAW_BYTES);
    constexpr uint32_t STAGE16 = STAGE_BYTES >> 4;
    constexpr uint32_t LO16 = (TA ? B_BYTES : RAW_BYTES) >> 4;   // lo copy relative to its raw tile, 16-byte units
    constexpr int KSTEPS = BK / 8;
    constexpr uint32_t TMEM_COLS = TA ? 512 : 2 * BN;      // double-buffered accumulator (+ the A slots)
    constexpr uint32_t TA_COL0 = 2 * BN;                   // first column of the A slots
    constexpr uint32_t TA_SLOT = 2 * BK;                   // hi | lo

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint8_t *stage_base = smem;
    uint8_t *epi_base = smem + static_cast<size_t>(p.stages) * STAGE_BYTES;      // 1024-aligned
    uint64_t *bars = reinterpret_cast<uint64_t *>(epi_base + kEpiWarps * p.epi_patches * kEpiBufBytes);
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
    const bool timed = p.prof != nullptr;
    const long long t_kernel0 = clock64();
    const uint32_t cta_rank = CG == 2 ? cluster_ctarank() : 0u;   // 0 = the pair's leader
    const int unit0 = static_cast<int>(blockIdx.x) / CG;           // this CTA (pair) starts at this unit ...
    const int unit_step = static_cast<int>(gridDim.x) / CG;        // ... and strides by the number of CTAs (pairs)

    // The next grid in the stream may be scheduled already -- unless it is the independent second product of
    // a pair, which skips its own wait: then it may only start once this grid's predecessors are known complete.
    if (threadIdx.x == 0 && p.dep_mode != 1) grid_dependency_trigger();
    if (warp == 0 && lane == 1) {
        // descriptor fetches overlap the barrier and TMEM set-up
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmA)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmB)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmC)) : "memory");
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(bar_full + 8u * s, 1);
            mbar_init(bar_xform + 8u * s, CG * NS / SG);   // one arrival per split warp (of the k-block's group; of both CTAs for a pair)
            mbar_init(bar_empty + 8u * s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_acc_full + 8u * i, 1);
            mbar_init(bar_acc_empty + 8u * i, CG * kEpiWarps);   // one arrival per epilogue warp, of both CTAs for a pair
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (CG == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(tmem_slot)),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(tmem_slot)),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (CG == 2) cluster_sync_all();   // the peer's barriers exist before anyone arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above overlapped the previous grid; its results are needed from here on.  The second product of
    // an independent pair needs nothing from the first: it runs beside it and waits for it only before it ends.
    if (p.dep_mode != 2) grid_dependency_wait();
    if (p.dep_mode == 1 && threadIdx.x == 0) grid_dependency_trigger();


    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // The whole warp runs the loop; one elected lane issues the copies.
        {
            int stage = 0;
            uint32_t phase = 0;
            int armed = 0;
            bool ok = true;
            long long waited = 0;
            constexpr uint32_t CHUNK_BYTES = 128u * BK;   // one 32-wide MN chunk: BK k-rows of 128 bytes
            const uint32_t dstA0 = smem_u32(stage_base);
            uint32_t dstA = dstA0;
            WorkIter wi = work_begin(p, unit0, unit_step);
            TileCoord t;
            while (ok && work_next(p, wi, t)) {
                int f = 0, kk = t.it0;
                if (t.it0 >= p.kiters) {
                    f = t.it0 / p.kiters;
                    kk = t.it0 - f * p.kiters;
                }
                int a0, a1, a2, b0, b1, b2;
                batch_coords(t.bt * p.fold + f, p.a_batch, p.a_d1, p.a_d2, p.fd_a_cnt, p.fd_a_d1, p.fd_a_d2, a0, a1, a2);
                batch_coords(t.bt * p.fold + f, p.b_batch, p.b_d1, p.b_d2, p.fd_b_cnt, p.fd_b_d1, p.fd_b_d2, b0, b1, b2);
                const int rowA = t.tm * (BM * CG) + static_cast<int>(cta_rank) * BM;
                const int rowB = t.tn * BN + static_cast<int>(cta_rank) * BNL;
                for (int it = t.it0; it < t.it1; ++it) {
                    ok = mbar_wait_warp(bar_empty + 8u * stage, phase ^ 1u, abort_flag, p.err, 0x100u | stage, waited, timed, p.wait_cycles);
                    if (!ok) break;
                    const uint32_t full = bar_full + 8u * stage;
                    const int k0 = kk * BK;
                    ++armed;
                    if (elect_one()) {
                        mbar_arrive_expect_tx(full, A_BYTES + static_cast<uint32_t>(p.b_rows_live) * BK * 4u);
                        if (armed != p.withhold_at) {        // test hook: a stage that is armed and never filled
                            load_operand(p.a_mode, dstA, &tmA, full, k0, rowA, BM / 32, CHUNK_BYTES, a0, a1, a2);
                            load_operand(p.b_mode, dstA + A_BYTES, &tmB, full, k0, rowB, BNL / 32, CHUNK_BYTES, b0, b1, b2);
                        }
                    }
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; dstA = dstA0; } else { dstA += STAGE_BYTES; }
                    if (++kk == p.kiters) {
                        kk = 0;
                        ++f;
                        if (p.fold > 1) {
                            batch_coords(t.bt * p.fold + f, p.a_batch, p.a_d1, p.a_d2, p.fd_a_cnt, p.fd_a_d1, p.fd_a_d2, a0, a1, a2);
                            batch_coords(t.bt * p.fold + f, p.b_batch, p.b_d1, p.b_d2, p.fd_b_cnt, p.fd_b_d1, p.fd_b_d2, b0, b1, b2);
                        }
                    }
                }
            }
            if (!ok) {
                // Aborting: let the copies already issued land before the CTA exits.
                const int pending = min(armed, p.stages);
                for (int i = 0; i < pending; ++i) {
                    if (--stage < 0) { stage = p.stages - 1; phase ^= 1u; }
                    const long long t0 = clock64();
                    while (!mbar_try_wait(bar_full + 8u * stage, phase) && clock64() - t0 < p.wait_cycles / 8) {}
                }
            }
            if (p.prof && lane == 0) atomicAdd(p.prof + 0, static_cast<unsigned long long>(waited));
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp runs the loop; one elected lane issues each MMA and commit.  In a CTA pair
        // only the leader's warp issues (its MMAs drive both SMs); the peer's warp just holds TMEM.
        if (CG == 1 || cta_rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc_it = 0;
            bool ok = true;
            long long waited = 0, waited_acc = 0;
            bool next_ready = false;                   // the stage about to be consumed was already seen complete
            const uint32_t sa0 = smem_u32(stage_base);
            const uint32_t a_lo0 = ((sa0 >> 4) & 0x3FFFu) | p.a_desc_lbo;
            const uint32_t b_lo0 = (((sa0 + A_BYTES) >> 4) & 0x3FFFu) | p.b_desc_lbo;
            uint32_t a_lo = a_lo0, b_lo = b_lo0;
            const uint32_t a_hi = p.a_desc_hi, b_hi = p.b_desc_hi;
            const uint32_t a_ks = p.a_kstep, b_ks = p.b_kstep;
            const uint32_t idesc = p.idesc;
            // A lone CTA in single-pass mode consumes the TMA barrier directly; otherwise the split warps
            // (of both CTAs, for a pair) announce the stage on the leader's barrier.
            const uint32_t ready0 = (FAST && CG == 1) ? bar_full : bar_xform;
            WorkIter wi = work_begin(p, unit0, unit_step);
            TileCoord wt;
            while (ok && work_next(p, wi, wt)) {
                const int iters = wt.it1 - wt.it0;
                const int buf = acc_it & 1;
                const uint32_t acc_phase = (acc_it >> 1) & 1;
                ok = mbar_wait_warp(bar_acc_empty + 8u * buf, acc_phase ^ 1u, abort_flag, p.err, 0x200u | buf, waited_acc, timed, p.wait_cycles);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
                uint32_t accumulate = 0;
                for (int it = 0; it < iters; ++it) {
                    if (!next_ready) {
                        ok = mbar_wait_warp(ready0 + 8u * stage, phase, abort_flag, p.err, 0x300u | stage, waited, timed, p.wait_cycles);
                        if (!ok) break;
                    }
                    tc_fence_after();
                    // Look at the following stage now; the answer is used after this stage's MMAs are
                    // queued, so the barrier read overlaps them (narrow tiles retire an MMA every 32
                    // cycles and would otherwise drain the queue during the wait).
                    const int nstage = stage + 1 == p.stages ? 0 : stage + 1;
                    const uint32_t peek = mbar_test_wait(ready0 + 8u * nstage, stage + 1 == p.stages ? phase ^ 1u : phase);
                    // This warp's own instruction count sets the pace of narrow tiles (an MMA retires every
                    // 32 cycles there): one election guards the whole k-block's MMAs and its stage commit
                    // (one election per MMA measured 12 % slower on the attention-shaped products; wide
                    // tiles measured the same either way).
                    if (elect_one()) {
#pragma unroll
                        for (int ks = 0; ks < KSTEPS; ++ks) {
                            const uint32_t ak = a_lo + ks * a_ks, bk = b_lo + ks * b_ks;
                            const uint32_t acc_first = ks == 0 ? accumulate : 1u;
                            if constexpr (TA) {
                                const uint32_t at = tmem_base + TA_COL0 + static_cast<uint32_t>(stage) * TA_SLOT + ks * 8;
                                umma_tf32_ts(d_tmem, at + BK, bk, b_hi, idesc, acc_first);
                                umma_tf32_ts(d_tmem, at, bk + LO16, b_hi, idesc, 1u);
                                umma_tf32_ts(d_tmem, at, bk, b_hi, idesc, 1u);
                            } else if constexpr (CG == 2 && FAST) {
                                umma_tf32_pair(d_tmem, ak, a_hi, bk, b_hi, idesc, acc_first);
                            } else if constexpr (CG == 2) {
                                umma_tf32_pair(d_tmem, ak + LO16, a_hi, bk, b_hi, idesc, acc_first);
                                umma_tf32_pair(d_tmem, ak, a_hi, bk + LO16, b_hi, idesc, 1u);
                                umma_tf32_pair(d_tmem, ak, a_hi, bk, b_hi, idesc, 1u);
                            } else if constexpr (FAST) {
                                umma_tf32(d_tmem, ak, a_hi, bk, b_hi, idesc, acc_first);
                            } else {
                                umma_tf32(d_tmem, ak + LO16, a_hi, bk, b_hi, idesc, acc_first);
                                umma_tf32(d_tmem, ak, a_hi, bk + LO16, b_hi, idesc, 1u);
                                umma_tf32(d_tmem, ak, a_hi, bk, b_hi, idesc, 1u);
                            }
                        }
                        if constexpr (CG == 2) umma_commit_pair(bar_empty + 8u * stage);
                        else umma_commit(bar_empty + 8u * stage);
                    }
                    accumulate = 1u;
                    next_ready = __all_sync(0xffffffffu, peek != 0u);
                    if (++stage == p.stages) {
                        stage = 0; phase ^= 1u; a_lo = a_lo0; b_lo = b_lo0;
                    } else {
                        a_lo += STAGE16; b_lo += STAGE16;
                    }
                }
                if (!ok) break;
                if constexpr (CG == 2) { if (elect_one()) umma_commit_pair(bar_acc_full + 8u * buf); }
                else { if (elect_one()) umma_commit(bar_acc_full + 8u * buf); }
                ++acc_it;
            }
            if (p.prof && lane == 0) {
                atomicAdd(p.prof + 1, static_cast<unsigned long long>(waited_acc));
                atomicAdd(p.prof + 2, static_cast<unsigned long long>(waited));
            }
        }
    } else if (warp < 2 + NS) {
        // ------------------------------------------------------------ hi/lo split
        // In single-pass mode there is nothing to split; for a CTA pair these warps still relay "my
        // CTA's tile has landed" to the leader's barrier.
        if (!FAST || CG == 2) {
            // With A in tensor memory one k-block is a serial chain per warp (barrier wake-up, loads, split, tensor-
            // memory stores and their completion, fence, arrival: ~600 cycles, measured) that the eight warps walk in
            // lockstep, each on one k-half of its lane quarter's rows (SG = 1).  With SG = 2 they work as two groups
            // of four (one warp per lane quarter) on alternate k-blocks instead: twice the work per warp and k-block,
            // two k-blocks in flight.  The host picks SG = 2 for long contractions.
            static_assert(SG == 1 || (SG == 2 && TA), "two split groups exist for the tensor-memory A variants only");
            constexpr int GROUPS = SG;
            const int group = TA ? (warp - 2) >> 2 : 0;   // SG = 1: the k-half this warp splits; SG = 2: its group
            const int tid = (threadIdx.x - 64) & (32 * NS / GROUPS - 1);   // index within the group
            int stage = 0;
            int kb = 0;                                   // k-blocks this CTA has seen: the group takes those of its parity
            uint32_t phase = 0;
            bool ok = true;
            long long waited = 0;
            constexpr int N4 = (TA ? B_BYTES : RAW_BYTES) >> 4;   // float4 count of what gets a lo copy
            constexpr int NT = 32 * NS / GROUPS;          // split threads that share one k-block
            constexpr int PER = (N4 + NT - 1) / NT;       // float4s per thread (the last round may be partial)
            constexpr bool EXACT = N4 % NT == 0;
            constexpr int U = !EXACT ? 1 : (PER % 4 == 0) ? 4 : (PER % 2 == 0 ? 2 : 1);
            WorkIter wi = work_begin(p, unit0, unit_step);
            TileCoord wt;
            while (ok && work_next(p, wi, wt)) {
                const int iters = wt.it1 - wt.it0;
                for (int it = 0; it < iters; ++it) {
                    if (SG == 2 && ((kb++ & 1) != group)) {    // the other group's k-block
                        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                        continue;
                    }
                    ok = mbar_wait(bar_full + 8u * stage, phase, abort_flag, p.err, 0x400u | stage, waited, timed, p.wait_cycles);
                    if (!ok) break;
                    if constexpr (TA) {
                      // A: this thread owns a row (lane quarter of its warp), 16 of the 32 k columns at a time.
                      const uint8_t *sa = stage_base + static_cast<size_t>(stage) * STAGE_BYTES;
                      const int row = (warp & 3) * 32 + lane;
#pragma unroll
                      for (int h = 0; h < SG; ++h) {
                        const int half = SG == 2 ? h : group;
                        uint32_t hi[16], lo16[16];
                        if (p.a_mode == kKMajor) {
                            // 128-byte rows, 16-byte chunk c of row r sits at chunk c ^ (r % 8)
                            const uint8_t *rp = sa + row * 128;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float4 x = *reinterpret_cast<const float4 *>(rp + (((half * 4 + j) ^ (row & 7)) << 4));
                                hi[4 * j + 0] = __float_as_uint(x.x); hi[4 * j + 1] = __float_as_uint(x.y);
                                hi[4 * j + 2] = __float_as_uint(x.z); hi[4 * j + 3] = __float_as_uint(x.w);
                            }
                        } else {
                            // 32-row chunks of BK k-lines of 128 bytes; 32-byte atom a of k-line k sits at a ^ (k % 4)
                            const uint8_t *cp = sa + (row >> 5) * (128 * BK) + ((row & 7) << 2);
                            const int atom = (row & 31) >> 3;
#pragma unroll
                            for (int kk = 0; kk < 16; ++kk) {
                                const int k = half * 16 + kk;
                                hi[kk] = *reinterpret_cast<const uint32_t *>(cp + k * 128 + ((atom ^ (k & 3)) << 5));
                            }
                        }
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const float x = __uint_as_float(hi[e]);
                            hi[e] &= 0xFFFFE000u;
                            lo16[e] = __float_as_uint(x - __uint_as_float(hi[e]));
                        }
                        const uint32_t ta = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + TA_COL0 +
                                            static_cast<uint32_t>(stage) * TA_SLOT + half * 16;
                        __syncwarp();                      // tcgen05.st is warp-collective
                        tmem_st16(ta, hi);
                        tmem_st16(ta + BK, lo16);
                      }
                    }
                    // TA: only the B tile gets a lo copy in shared memory (it sits right behind the raw B tile).
                    const float4 *raw = reinterpret_cast<const float4 *>(stage_base + static_cast<size_t>(stage) * STAGE_BYTES +
                                                                         (TA ? A_BYTES : 0));
                    float4 *lo = const_cast<float4 *>(raw) + N4;
                    // float4s that hold data: all of them, or A and the live rows of B
                    const int live4 = N4 - ((BNL - p.b_rows_live) * BK * 4 >> 4);
#pragma unroll
                    for (int g = 0; g < (FAST ? 0 : PER); g += U) {
                        float4 v[U];
#pragma unroll
                        for (int u = 0; u < U; ++u)
                            if (tid + (g + u) * NT < live4) v[u] = raw[tid + (g + u) * NT];
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            if (tid + (g + u) * NT >= live4) continue;
                            float4 l;
                            l.x = v[u].x - __uint_as_float(__float_as_uint(v[u].x) & 0xFFFFE000u);
                            l.y = v[u].y - __uint_as_float(__float_as_uint(v[u].y) & 0xFFFFE000u);
                            l.z = v[u].z - __uint_as_float(__float_as_uint(v[u].z) & 0xFFFFE000u);
                            l.w = v[u].w - __uint_as_float(__float_as_uint(v[u].w) & 0xFFFFE000u);
                            lo[tid + (g + u) * NT] = l;
                        }
                    }
                    if constexpr (TA) {                       // the stores above complete while the B tile was split
                        tmem_st_wait();
                        tc_fence_before();
                    }
                    // Every thread publishes its writes to the async proxy; one lane per warp then arrives
                    // (a remote arrival crosses SMs, so they are kept to one per warp).
                    if (!FAST) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        if (CG == 2 && cta_rank != 0) mbar_arrive_cta(bar_xform + 8u * stage, 0u);
                        else mbar_arrive(bar_xform + 8u * stage);
                    }
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
            if (p.prof && tid == 0) atomicAdd(p.prof + 3, static_cast<unsigned long long>(waited));
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;                       // TMEM lane quarter this warp may read
        const int ew = warp - (2 + NS);               // 0..7: warps ew and ew+4 share a lane quarter ...
        constexpr int CHUNKS = BN / 32 / (kEpiWarps / 4);   // ... and take half of the tile's 32-column chunks each
        const int chunk_lo = (ew >> 2) * CHUNKS;
        uint8_t *my_stage = epi_base + ew * p.epi_patches * kEpiBufBytes;
        int acc_it = 0;
        int patch = 0;                                // staging buffer to use next
        int in_flight = 0;                            // bulk groups committed by lane 0 and not yet waited for
        bool ok = true;
        long long waited = 0, t_ld = 0, t_wg = 0;
        const bool use_tma = p.epi_mode == kEpiTmaStore || p.epi_mode == kEpiTmaReduce;
        const bool bias_vec = (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0;
        WorkIter wi = work_begin(p, unit0, unit_step);
        TileCoord t;
        const int my_cta = static_cast<int>(blockIdx.x);                 // slot * CG + rank in the pair
        while (ok && work_next(p, wi, t)) {
            const int buf = acc_it & 1;
            const uint32_t acc_phase = (acc_it >> 1) & 1;
            ok = mbar_wait(bar_acc_full + 8u * buf, acc_phase, abort_flag, p.err, 0x500u | buf, waited, timed, p.wait_cycles);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const bool fuse = p.splits == 1;
            const bool add_piece = t.chunk > 0;       // a later piece of this unit's contraction: added to what the earlier ones wrote
            if (add_piece && use_tma) {
                // this warp's earlier stores to the same patches must have completed, not just been read
                if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                in_flight = 0;
                __syncwarp();
            }
            const int row0 = t.tm * (BM * CG) + static_cast<int>(cta_rank) * BM + q * 32;
            const int cbatch = fuse ? t.bt : t.split * p.batch + t.bt;
            const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * BN);
            // Shared tile of the balanced tail.  Each (tile, CTA rank, epilogue warp) region has a ticket; the
            // units of the tile arrive in any order, all but the last park their accumulator (and raise a
            // ready flag), the last one adds the parked ones to its own in slot order -- the sum does not
            // depend on who came last -- and runs the usual epilogue.
            int seg_first = 0, seg_count = 1;          // slots sharing the tile: seg_first .. seg_first + seg_count - 1
            bool reducer = false;
            const int nslots = static_cast<int>(gridDim.x) / CG;
            if (SK && t.shared) {
                const long long per_tile = p.fold * p.kiters;
                const long long tile_begin = static_cast<long long>(t.tile - p.sk_first_tile) * per_tile;
                const long long tile_end = tile_begin + per_tile;
                seg_first = unit0;
                while (seg_first > 0 && sk_range_begin(p, seg_first, nslots) > tile_begin) --seg_first;
                int last = unit0;
                while (last + 1 < nslots && sk_range_begin(p, last + 1, nslots) < tile_end) ++last;
                seg_count = last - seg_first + 1;
            }
            bool waited_contrib = false, parked = false;
            unsigned int *ticket = nullptr;
            if (SK && t.shared && seg_count > 1 && row0 < p.M && t.tn * BN + chunk_lo * 32 < p.N) {
                const size_t region = (static_cast<size_t>(t.tile - p.sk_first_tile) * CG + cta_rank) * kEpiWarps + ew;
                ticket = p.sk_flags + static_cast<size_t>(gridDim.x) * 2 * kEpiWarps + region;
                unsigned int old = 0;
                if (lane == 0) old = atomicAdd(ticket, 1u);
                old = __shfl_sync(0xffffffffu, old, 0);
                reducer = old == static_cast<unsigned int>(seg_count - 1);
            }
            const bool park_it = SK && t.shared && seg_count > 1 && !reducer;
            // The reducer's list of the tile's other units, in slot order: index of their parking place
            // ((cta * 2 + place) * warps + warp, also the index of its ready flag).
            size_t others[kSkMaxShare - 1];
            int n_others = 0, n_before = 0;
            if (SK && reducer) {
                const long long tile_begin = static_cast<long long>(t.tile - p.sk_first_tile) * (p.fold * p.kiters);
                for (int j = seg_first; j < seg_first + seg_count; ++j) {
                    if (j == unit0) continue;
                    const int idx = (j == seg_first && sk_range_begin(p, j, nslots) < tile_begin) ? 1 : 0;
                    others[n_others++] = (static_cast<size_t>(j * CG + static_cast<int>(cta_rank)) * 2 + idx) * kEpiWarps + ew;
                    if (j < unit0) ++n_before;
                }
            }
            if (row0 < p.M) {
                for (int chunk = chunk_lo; chunk < chunk_lo + CHUNKS; ++chunk) {
                    const int col0 = t.tn * BN + chunk * 32;
                    if (col0 >= p.N) break;           // warp-uniform
                    uint32_t v[32];
                    __syncwarp();                      // tcgen05.ld is warp-collective
                    const long long t_ld0 = p.prof ? clock64() : 0;
                    tmem_ld32_issue(tbase + chunk * 32, v);
                    tmem_ld_wait();
                    if (p.prof) t_ld += clock64() - t_ld0;
                    if (park_it) {
                        // [j][lane] order: one instruction of the warp writes 512 contiguous bytes
                        float4 *dst = reinterpret_cast<float4 *>(
                            p.sk_partial + (((static_cast<size_t>(my_cta) * 2 + t.park) * kEpiWarps + ew) * CHUNKS + (chunk - chunk_lo)) * 1024) + lane;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            __stcg(dst + j * 32, make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                        __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])));
                        parked = true;
                        continue;
                    }
                    if (SK && reducer) {
                        if (!waited_contrib) {
                            // Bounded wait for the ready flag of every other unit of the tile (they took their
                            // tickets earlier, so they are at most one parking pass behind).
                            for (int o = 0; ok && o < n_others; ++o) {
                                const unsigned int *flag = p.sk_flags + others[o];
                                const long long tw0 = clock64();
                                unsigned int seen = 0;
                                while (true) {
                                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
                                    if (seen != 0u) break;
                                    if (*abort_flag || clock64() - tw0 > p.wait_cycles) {
                                        *abort_flag = 1u;
                                        atomicCAS(p.err, 0u, 0x600u);
                                        ok = false;
                                        break;
                                    }
                                }
                            }
                            ok = __all_sync(0xffffffffu, ok);
                            waited_contrib = true;
                            if (!ok) break;
                        }
                        // Sum in slot (= ascending k) order; this warp's own accumulator takes its place in it.
                        // Each parked tile is fetched with independent 16-byte loads, half a chunk at a time.
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            float4 pre[4];
                            for (int o = 0; o < n_before; ++o) {
                                const float4 *src = reinterpret_cast<const float4 *>(
                                                        p.sk_partial + (others[o] * CHUNKS + (chunk - chunk_lo)) * 1024) + h * 128 + lane;
                                float4 x[4];
#pragma unroll
                                for (int u = 0; u < 4; ++u) x[u] = __ldcg(src + u * 32);
#pragma unroll
                                for (int u = 0; u < 4; ++u) {
                                    if (o == 0) pre[u] = x[u];
                                    else { pre[u].x += x[u].x; pre[u].y += x[u].y; pre[u].z += x[u].z; pre[u].w += x[u].w; }
                                }
                            }
                            if (n_before > 0) {
#pragma unroll
                                for (int u = 0; u < 4; ++u) {
                                    const int b = 16 * h + 4 * u;
                                    v[b + 0] = __float_as_uint(pre[u].x + __uint_as_float(v[b + 0]));
                                    v[b + 1] = __float_as_uint(pre[u].y + __uint_as_float(v[b + 1]));
                                    v[b + 2] = __float_as_uint(pre[u].z + __uint_as_float(v[b + 2]));
                                    v[b + 3] = __float_as_uint(pre[u].w + __uint_as_float(v[b + 3]));
                                }
                            }
                            for (int o = n_before; o < n_others; ++o) {
                                const float4 *src = reinterpret_cast<const float4 *>(
                                                        p.sk_partial + (others[o] * CHUNKS + (chunk - chunk_lo)) * 1024) + h * 128 + lane;
                                float4 x[4];
#pragma unroll
                                for (int u = 0; u < 4; ++u) x[u] = __ldcg(src + u * 32);
#pragma unroll
                                for (int u = 0; u < 4; ++u) {
                                    const int b = 16 * h + 4 * u;
                                    v[b + 0] = __float_as_uint(__uint_as_float(v[b + 0]) + x[u].x);
                                    v[b + 1] = __float_as_uint(__uint_as_float(v[b + 1]) + x[u].y);
                                    v[b + 2] = __float_as_uint(__uint_as_float(v[b + 2]) + x[u].z);
                                    v[b + 3] = __float_as_uint(__uint_as_float(v[b + 3]) + x[u].w);
                                }
                            }
                        }
                    }
                    // Stages the 32 values of this lane's row into the warp's next patch and hands the
                    // patch to the TMA unit (store, or reduce-add for C += ...).
                    auto emit = [&](const CUtensorMap *map, bool reduce) {
                        const long long t_wg0 = p.prof ? clock64() : 0;
                        if (lane == 0 && in_flight == p.epi_patches) {   // the patch must have been read by its store
                            if (p.epi_patches == 1) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                            else if (p.epi_patches == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                            else if (p.epi_patches == 4) asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
                            else asm volatile("cp.async.bulk.wait_group.read 7;" ::: "memory");
                            --in_flight;
                        }
                        __syncwarp();
                        if (p.prof) t_wg += clock64() - t_wg0;
                        if (p.transpose_out) {
                            // patch row j = this chunk's column j, float `lane` of it = this lane's row:
                            // the 32 lanes fill one 128-byte line per store, conflict-free
                            uint8_t *dst = my_stage + patch * kEpiBufBytes + ((lane & 3) << 2);
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                *reinterpret_cast<uint32_t *>(dst + j * 128 + (((lane >> 2) ^ (j & 7)) << 4)) = v[j];
                        } else {
                            uint8_t *dst = my_stage + patch * kEpiBufBytes + lane * 128;
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                *reinterpret_cast<float4 *>(dst + ((j ^ (lane & 7)) << 4)) =
                                    make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) {
                            const uint32_t src = smem_u32(my_stage + patch * kEpiBufBytes);
                            const int c0 = p.transpose_out ? row0 : col0, c1 = p.transpose_out ? col0 : row0;
                            if (reduce) tma_reduce_add_5d(map, src, c0, c1, cbatch);
                            else tma_store_5d(map, src, c0, c1, cbatch);
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                            ++in_flight;
                        }
                        if (++patch == p.epi_patches) patch = 0;
                    };
                    const bool do_act = fuse && p.act != 0;          // host guarantees use_tma in this mode
                    if (do_act && p.store_pre) emit(&tmC, false);    // the raw product, what the tape saves
                    if (fuse && p.bias != nullptr && add_piece) {
                        // the bias went in with the first piece
                    } else if (fuse && p.bias != nullptr && p.transpose_out) {
                        const float b = row0 + lane < p.M ? __ldg(p.bias + row0 + lane) : 0.f;   // one bias value per row here
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + b);
                    } else if (fuse && p.bias != nullptr) {
                        if (bias_vec && col0 + 32 <= p.N) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float4 b = __ldg(reinterpret_cast<const float4 *>(p.bias + col0) + j);
                                v[4 * j + 0] = __float_as_uint(__uint_as_float(v[4 * j + 0]) + b.x);
                                v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + b.y);
                                v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + b.z);
                                v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + b.w);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < p.N) v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldg(p.bias + col0 + j));
                        }
                    }
                    if (do_act) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(gelu_tanh_f(__uint_as_float(v[j])));
                        emit(&tmD, false);
                    } else if (use_tma) {
                        emit(&tmC, (p.epi_mode == kEpiTmaReduce && fuse) || add_piece);
                    } else {
                        const int row = row0 + lane;
                        if (row < p.M) {
                            float *out = fuse ? p.C + static_cast<long long>(t.bt) * p.c_bstride + static_cast<long long>(row) * p.ldc
                                              : p.partial + (static_cast<long long>(cbatch) * p.M + row) * p.N;
                            if (p.epi_mode == kEpiVectorStores && col0 + 32 <= p.N) {
                                // Each lane owns one row: four 32-byte stores write whole sectors, no staging.
                                float *dst = out + col0;
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    float y[8];
#pragma unroll
                                    for (int e = 0; e < 8; ++e) y[e] = __uint_as_float(v[8 * j + e]);
                                    if ((fuse && p.accumulate) || add_piece) {
                                        float o[8];
                                        asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                                     : "=f"(o[0]), "=f"(o[1]), "=f"(o[2]), "=f"(o[3]), "=f"(o[4]), "=f"(o[5]),
                                                       "=f"(o[6]), "=f"(o[7])
                                                     : "l"(dst + 8 * j));
#pragma unroll
                                        for (int e = 0; e < 8; ++e) y[e] += o[e];
                                    }
                                    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + 8 * j),
                                                 "f"(y[0]), "f"(y[1]), "f"(y[2]), "f"(y[3]), "f"(y[4]), "f"(y[5]), "f"(y[6]),
                                                 "f"(y[7])
                                                 : "memory");
                                }
                                continue;
                            }
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (col0 + j < p.N) {
                                    float y = __uint_as_float(v[j]);
                                    if ((fuse && p.accumulate) || add_piece) y += out[col0 + j];
                                    out[col0 + j] = y;
                                }
                            }
                        }
                    }
                }
            }
            if (!ok) break;
            if (parked) {
                // publish: every lane's stores are fenced, then one release store of the ready flag
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    unsigned int *flag = p.sk_flags + ((static_cast<size_t>(my_cta) * 2 + t.park) * kEpiWarps + ew);
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(1u) : "memory");
                }
            } else if (SK && reducer) {
                // every lane has read the parked tiles: ticket and ready flags go back to zero for the next launch
                __syncwarp();
                if (lane == 0) {
                    *ticket = 0u;
                    if (waited_contrib)
                        for (int o = 0; o < n_others; ++o) p.sk_flags[others[o]] = 0u;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (CG == 2 && cta_rank != 0) mbar_arrive_cta(bar_acc_empty + 8u * buf, 0u);
                else mbar_arrive(bar_acc_empty + 8u * buf);
            }
            ++acc_it;
        }
        // The staging patches must have been read before the CTA gives up its shared memory; the global
        // writes themselves complete with the grid like any other store.
        if (use_tma && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        if (p.prof && warp == 2 + NS && lane == 0) {
            atomicAdd(p.prof + 4, static_cast<unsigned long long>(waited));
            atomicAdd(p.prof + 7, static_cast<unsigned long long>(t_wg));
            atomicAdd(p.prof + 1, static_cast<unsigned long long>(t_ld));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (p.prof && threadIdx.x == 0) {
        atomicAdd(p.prof + 5, static_cast<unsigned long long>(clock64() - t_kernel0));
        atomicAdd(p.prof + 6, 1ull);
    }
    if constexpr (CG == 2) cluster_sync_all();   // both CTAs are done with the pair's TMEM and barriers
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        if constexpr (CG == 2)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                         : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                         : "memory");
    }
    // Stream order for whatever follows: this grid may not complete before the grid it ran beside has.
    if (p.dep_mode == 2 && threadIdx.x == 0) grid_dependency_wait();
}

// Deterministic split-K finish: C = sum_s partial[s] (+ bias) (+ C), splits added in ascending order.
// One thread per vector of the output (two divisions per thread, none per element); the partials of
// four splits are in flight at a time.
template <typename V, typename I>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float *__restrict__ partial, float *__restrict__ C, long long ldc, long long c_bstride,
                     const float *__restrict__ bias, int accumulate, int splits, long long rows, int M, int N) {
    constexpr int W = sizeof(V) / sizeof(float);
    grid_dependency_trigger();
    grid_dependency_wait();                      // the partials come from the grid before this one
    const I per_row = static_cast<I>(N / W);
    const I item = static_cast<I>(blockIdx.x) * 256 + threadIdx.x;
    if (item >= static_cast<I>(rows) * per_row) return;
    const I row = item / per_row;
    const int col = static_cast<int>(item - row * per_row) * W;
    const I bt = row / static_cast<I>(M);
    const int m = static_cast<int>(row - bt * static_cast<I>(M));
    const long long slab = rows * N;
    const float *src = partial + static_cast<long long>(row) * N + col;
    float acc[W];
#pragma unroll
    for (int e = 0; e < W; ++e) acc[e] = 0.f;
    int sp = 0;
    for (; sp + 4 <= splits; sp += 4) {
        V t[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) t[u] = __ldcg(reinterpret_cast<const V *>(src + (sp + u) * slab));
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float *tv = reinterpret_cast<const float *>(&t[u]);
#pragma unroll
            for (int e = 0; e < W; ++e) acc[e] += tv[e];
        }
    }
    for (; sp < splits; ++sp) {
        const V t = __ldcg(reinterpret_cast<const V *>(src + sp * slab));
        const float *tv = reinterpret_cast<const float *>(&t);
#pragma unroll
        for (int e = 0; e < W; ++e) acc[e] += tv[e];
    }
    if (bias) {
        const V b = __ldg(reinterpret_cast<const V *>(bias + col));
        const float *bv = reinterpret_cast<const float *>(&b);
#pragma unroll
        for (int e = 0; e < W; ++e) acc[e] += bv[e];
    }
    V *out = reinterpret_cast<V *>(C + static_cast<long long>(bt) * c_bstride + static_cast<long long>(m) * ldc + col);
    if (accumulate) {
        const V c0 = *out;
        const float *cv = reinterpret_cast<const float *>(&c0);
#pragma unroll
        for (int e = 0; e < W; ++e) acc[e] += cv[e];
    }
    *out = *reinterpret_cast<const V *>(acc);
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

// Encoded tensor maps are a pure function of (pointer, extents, strides, box, swizzle): a training loop calls with
// the same handful of buffers every step, so each host thread keeps the maps it has built (bounded; dropped
// wholesale when full) and an eager call pays a hash lookup instead of three or four driver encodes.
struct MapKey {
    const void *ptr;
    cuuint64_t dims[5];
    cuuint64_t strides[4];
    cuuint32_t box[5];
    int swz;
    bool operator==(const MapKey &o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
    size_t operator()(const MapKey &k) const {
        const unsigned char *b = reinterpret_cast<const unsigned char *>(&k);
        uint64_t h = 1469598103934665603ull;            // FNV-1a over the key's bytes
        for (size_t i = 0; i < sizeof(MapKey); ++i) { h ^= b[i]; h *= 1099511628211ull; }
        return static_cast<size_t>(h);
    }
};
constexpr size_t kMapCacheEntries = 512;

CUresult encode(CUtensorMap *map, const float *ptr, const cuuint64_t *dims, const cuuint64_t *strides,
                const cuuint32_t *box, CUtensorMapSwizzle swz) {
    static thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static const bool use_cache = env_int("MNI_B200_MAP_CACHE", 1) != 0;
    MapKey key;
    memset(&key, 0, sizeof(key));                       // padding bytes take part in the comparison
    key.ptr = ptr;
    for (int i = 0; i < 5; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
    for (int i = 0; i < 4; ++i) key.strides[i] = strides[i];
    key.swz = static_cast<int>(swz);
    if (use_cache) {
        auto it = cache.find(key);
        if (it != cache.end()) { *map = it->second; return CUDA_SUCCESS; }
    }
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float *>(ptr), dims, strides, box,
                                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS && use_cache) {
        if (cache.size() >= kMapCacheEntries) cache.clear();
        cache.emplace(key, *map);
    }
    return r;
}

// Builds the tensor map of one operand and reports the OperandMode the kernel must use for it.
int make_operand_map(CUtensorMap *map, const Operand &op, int box_rows, int bk, int *mode) {
    if (!encode_fn()) return fail(MNI_B200_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
    cuuint64_t dims[5];
    cuuint64_t strides[4];   // bytes, dims 1..4
    cuuint32_t box[5] = {1, 1, 1, 1, 1};
    // A size-1 dim never advances, but its stride must still be a positive multiple of 16 bytes.
    uint64_t span = 16;
    auto stride_or = [&](int64_t extent, int64_t stride_elems) -> cuuint64_t {
        return static_cast<cuuint64_t>((extent > 1 && stride_elems > 0) ? static_cast<uint64_t>(stride_elems) * 4u : span);
    };
    // 32-bit elements read MN-major by the tensor core use the 128-byte swizzle whose unit is a
    // 32-byte chunk, not the usual 16-byte chunk.
    const CUtensorMapSwizzle mn_swz = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
    if (!op.k_major && op.rows % 32 == 0 && op.bshape[0] == 1 && env_int("MNI_B200_NO_SINGLE_BOX", 0) == 0) {
        // One box per tile: the MN dim is split into (32 contiguous floats, rows/32 chunks), giving the
        // smem order [chunk][k][32 floats] the MMA descriptor expects.
        dims[0] = 32;
        dims[1] = static_cast<cuuint64_t>(op.kdim);
        dims[2] = static_cast<cuuint64_t>(op.rows / 32);
        dims[3] = static_cast<cuuint64_t>(op.bshape[2]);
        dims[4] = static_cast<cuuint64_t>(op.bshape[1]);
        span = 128;
        strides[0] = stride_or(op.kdim, op.ld);
        span = std::max<uint64_t>(span, strides[0] * dims[1]);
        strides[1] = 128;
        strides[2] = stride_or(op.bshape[2], op.bstride[2]);
        span = std::max<uint64_t>(span, strides[2] * dims[3]);
        strides[3] = stride_or(op.bshape[1], op.bstride[1]);
        box[0] = 32;
        box[1] = static_cast<cuuint32_t>(bk);
        box[2] = static_cast<cuuint32_t>(box_rows / 32);
        if (encode(map, op.ptr, dims, strides, box, mn_swz) == CUDA_SUCCESS) {
            *mode = kMnSingleBox;
            return MNI_B200_OK;
        }
        box[2] = 1;   // fall through to the multi-box form
    }
    CUtensorMapSwizzle swz;
    if (op.k_major) {
        dims[0] = static_cast<cuuint64_t>(op.kdim);
        dims[1] = static_cast<cuuint64_t>(op.rows);
        box[0] = static_cast<cuuint32_t>(bk);
        box[1] = static_cast<cuuint32_t>(box_rows);
        swz = bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
        *mode = kKMajor;
    } else {
        dims[0] = static_cast<cuuint64_t>(op.rows);
        dims[1] = static_cast<cuuint64_t>(op.kdim);
        box[0] = 32;
        box[1] = static_cast<cuuint32_t>(bk);
        swz = mn_swz;
        *mode = kMnMultiBox;
    }
    span = std::max<uint64_t>(16, (static_cast<uint64_t>(dims[0]) * 4u + 15u) & ~15ull);
    strides[0] = stride_or(static_cast<int64_t>(dims[1]), op.ld);
    span = std::max<uint64_t>(span, strides[0] * dims[1]);
    for (int i = 0; i < 3; ++i) {   // map dim 2 = innermost batch dim
        const int bi = 2 - i;
        dims[2 + i] = static_cast<cuuint64_t>(op.bshape[bi]);
        strides[1 + i] = stride_or(op.bshape[bi], op.bstride[bi]);
        span = std::max<uint64_t>(span, strides[1 + i] * dims[2 + i]);
    }
    const CUresult r = encode(map, op.ptr, dims, strides, box, swz);
    if (r != CUDA_SUCCESS)
        return fail(MNI_B200_ERR_CUDA,
                    "cuTensorMapEncodeTiled failed (%d): dims %llu x %llu, ld %lld, k_major %d", static_cast<int>(r),
                    static_cast<unsigned long long>(dims[0]), static_cast<unsigned long long>(dims[1]),
                    static_cast<long long>(op.ld), static_cast<int>(op.k_major));
    return MNI_B200_OK;
}

// Tensor map of the output (or of the split-K partial buffer): dims (N, M, batches), 32 x 32 boxes.
int make_output_map(CUtensorMap *map, float *ptr, int64_t N, int64_t M, int64_t batches, int64_t ld, int64_t bstride) {
    cuuint64_t dims[5] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(batches), 1, 1};
    cuuint64_t strides[4];
    strides[0] = static_cast<cuuint64_t>(M > 1 ? ld * 4 : ((N * 4 + 15) & ~15LL));
    strides[1] = static_cast<cuuint64_t>(batches > 1 ? bstride * 4 : std::max<int64_t>(strides[0] * M, 16));
    strides[2] = strides[1] * static_cast<cuuint64_t>(batches);
    strides[3] = strides[2];
    const cuuint32_t box[5] = {32, 32, 1, 1, 1};
    const CUresult r = encode(map, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != CUDA_SUCCESS) return fail(MNI_B200_ERR_CUDA, "cuTensorMapEncodeTiled(output) failed (%d)", static_cast<int>(r));
    return MNI_B200_OK;
}

struct Plan {
    int bn, bk, cg, stages, splits, tiles_m, tiles_n, grid;   // cg = CTAs per tile (1, or 2 = CTA pair)
    int patches;                                              // epilogue staging patches per warp
    bool ta;                                                  // A operand of the MMAs from tensor memory
    bool sk;                                                  // balanced tail: the last, ragged wave is cut by k-blocks
    int sk_first_tile;
    size_t smem;
};

constexpr size_t kFixedSmemNoEpi = 1024 + kBarBytes;

Plan make_plan(const GemmProblem &p, int sm_count) {
    Plan pl;
    pl.bn = p.N <= 64 ? 64 : (p.N <= 128 ? 128 : 256);
    const int bn_env = env_int("MNI_B200_BN", 0);
    if (bn_env == 64 || bn_env == 128 || bn_env == 256) pl.bn = bn_env;
    // CTA pairs: 256-wide tiles and at least two 128-row blocks of output.
    const int pair_env = env_int("MNI_B200_CTA_PAIR", 1);     // 0 never, 1 for 256-wide tiles, 2 for every width
    auto pair_for = [&](int bn) { return (p.M > BM && (pair_env >= 2 || (pair_env == 1 && bn == 256))) ? 2 : 1; };
    // Problems with fewer 128 x 256 tiles than SMs are latency-bound: one tile's k-loop is a serial
    // TMA -> split -> MMA chain, so narrower tiles and a K split put more SMs on it.  The tile width and the
    // split are chosen by a small cost model fitted to measured times of 256^3 .. 1024^3 products:
    // nanoseconds per k element of one tile (30 / 33 for a 256-wide pair / lone CTA, 15.4 for 128, 13.5
    // for 64), 1.5 us for the reduce launch and its traffic at 3 TB/s.
    int model_splits = 0;
    const long long tiles256 = static_cast<long long>(p.batch) * ((p.M + BM - 1) / BM) * ((p.N + 255) / 256);
    if (bn_env == 0 && p.force_splits <= 0 && tiles256 < sm_count && env_int("MNI_B200_PLAN_MODEL", 1) != 0) {
        const double k_eff = static_cast<double>(p.K) * static_cast<double>(p.fold);
        const double out_bytes = 4.0 * static_cast<double>(p.batch) * static_cast<double>(p.M) * static_cast<double>(p.N);
        double best = 1e300;
        for (int bn : {256, 128, 64}) {
            if (bn > 64 && p.N <= bn / 2) continue;               // no tile wider than the output needs
            const int cg = pair_for(bn);
            const long long tiles = static_cast<long long>(p.batch) * ((p.M + BM * cg - 1) / (BM * cg)) * ((p.N + bn - 1) / bn);
            const long long slots = std::max(1, sm_count / cg);
            for (int sp : {1, 2, 3, 4, 6, 8, 12, 16}) {
                if (sp > 1 && (tiles * sp > slots || k_eff / sp < 64.0)) continue;
                // A 128-wide tile with a long contraction runs at its steady state, which shared-memory bandwidth
                // sets (128 KB per 32-deep k-block = 1000 cycles): measured 20.5 ns per k element at K = 8192,
                // against 32 for a 256-wide pair doing twice the work.
                const double c_ns = bn == 256 ? (cg == 2 ? 30.0 : 33.0) : (bn == 128 ? (k_eff / sp >= 1024.0 ? 20.5 : 15.4) : 13.5);
                const double rounds = static_cast<double>((tiles * sp + slots - 1) / slots);
                const double t = rounds * (k_eff / sp) * c_ns + (sp > 1 ? 1500.0 + (sp + 1) * out_bytes / 3000.0 : 0.0);
                if (t < best) { best = t; pl.bn = bn; model_splits = sp; }
            }
        }
    }
    pl.cg = pair_for(pl.bn);
    pl.bk = (pl.bn == 256 && !p.fast_tf32) ? 16 : 32;
    const int bk_env = env_int("MNI_B200_BK", 0);
    if ((bk_env == 16 || bk_env == 32) && pl.bn == 256) pl.bk = bk_env;   // narrower tiles are built for BK = 32 only
    // Narrow tiles of a lone CTA are bound by shared-memory bandwidth; taking A from tensor memory removes
    // most of A's share of it.
    pl.ta = !p.fast_tf32 && pl.cg == 1 && pl.bk == 32 && pl.bn <= 128 && env_int("MNI_B200_TMEM_A", 1) != 0;
    const size_t raw = static_cast<size_t>(BM + pl.bn / pl.cg) * pl.bk * 4;
    const size_t stage = p.fast_tf32 ? raw : (pl.ta ? raw + static_cast<size_t>(pl.bn) * pl.bk * 4 : 2 * raw);
    const size_t budget = 227 * 1024;
    // Tiles with a short contraction spend their time in the epilogue: give it more TMA stores in
    // flight (staging patches) and the main loop fewer stages.  Long contractions get the deepest pipeline.
    const long long iters_per_tile = p.fold * ((p.K + pl.bk - 1) / pl.bk);
    pl.patches = 1;   // staging patches per epilogue warp
    (void)iters_per_tile;
    const int pt_env = env_int("MNI_B200_EPI_PATCHES", 0);
    if (pt_env == 1 || pt_env == 2 || pt_env == 4) pl.patches = pt_env;
    size_t fixed = kFixedSmemNoEpi + static_cast<size_t>(kEpiWarps * pl.patches) * kEpiBufBytes;
    while (pl.patches > 2 && (budget - fixed) / stage < 2) {
        pl.patches /= 2;
        fixed = kFixedSmemNoEpi + static_cast<size_t>(kEpiWarps * pl.patches) * kEpiBufBytes;
    }
    pl.stages = static_cast<int>(std::min<size_t>(kMaxStages, (budget - fixed) / stage));
    if (pl.ta) pl.stages = std::min(pl.stages, (512 - 2 * pl.bn) / (2 * pl.bk));   // one TMEM slot per stage
    const int st_env = env_int("MNI_B200_STAGES", 0);
    if (st_env >= 1 && st_env <= pl.stages) pl.stages = st_env;
    pl.smem = fixed + static_cast<size_t>(pl.stages) * stage;
    const int tile_m = BM * pl.cg;
    const int slots = std::max(1, sm_count / pl.cg);          // CTAs (or CTA pairs) that run at once
    pl.tiles_m = static_cast<int>((p.M + tile_m - 1) / tile_m);
    pl.tiles_n = static_cast<int>((p.N + pl.bn - 1) / pl.bn);
    const long long tiles = static_cast<long long>(p.batch) * pl.tiles_m * pl.tiles_n;
    const long long iters = p.fold * ((p.K + pl.bk - 1) / pl.bk);
    int splits = 1;
    if (p.force_splits > 0) {
        splits = p.force_splits;
    } else if (model_splits > 0) {
        splits = model_splits;
    } else if (tiles * 2 <= slots && iters >= 8) {
        // Few output tiles and a long contraction: split K so that the whole GPU works.
        splits = static_cast<int>(std::min<long long>(slots / tiles, iters / 4));
    }
    splits = static_cast<int>(std::max<long long>(1, std::min<long long>(std::min<long long>(splits, iters), 64)));
    pl.splits = splits;
    const long long units = tiles * splits;
    pl.grid = static_cast<int>(std::min<long long>(units, slots)) * pl.cg;
    // Balanced tail: when the last wave of whole tiles would leave more than 8 % of the slots idle, its
    // k-blocks are dealt out evenly instead (every slot gets one contiguous range; tiles cut by a range
    // boundary are summed in the owner's epilogue, in slot order).
    pl.sk = false;
    pl.sk_first_tile = 0;
    // MNI_B200_STREAMK: unset = on when the whole-tile schedule would idle more than a fifth of the slot-rounds
    // (measured: below that the idle SMs of a ragged wave are power headroom for the busy ones at the 1 kW cap
    // and the balanced tail does not pay); 1 = on from 8 % idle; 0 = never.
    const int sk_env = env_int("MNI_B200_STREAMK", -1);
    if (splits == 1 && p.D == nullptr && sk_env != 0) {
        const long long full_rounds = tiles / slots, rem = tiles - full_rounds * slots;
        const double eff = static_cast<double>(tiles) / static_cast<double>((full_rounds + 1) * slots);
        const double eff_limit = sk_env > 0 ? 0.92 : 0.80;
        if (rem > 0 && eff < eff_limit && iters >= 8 && tiles * 2 > slots) {
            // the tail takes one whole round along when there is one, so that a range is at least a tile long
            const long long whole = full_rounds > 0 ? full_rounds - 1 : 0;
            const long long range = (tiles - whole * slots) * iters / slots;
            // a tile is shared by at most iters / range + 2 units
            // compiled for the variants that meet ragged waves in practice: 256-wide pairs and narrow tensor-memory tiles
            const bool built = (pl.cg == 2 && pl.bn == 256) || pl.ta;
            if (built && range >= 8 && iters / range + 2 <= kSkMaxShare) {
                pl.sk = true;
                pl.sk_first_tile = static_cast<int>(whole * slots);
                pl.grid = static_cast<int>(slots) * pl.cg;
            }
        }
    }
    return pl;
}

// N extent of the MMAs.  A lone CTA's tile that is wider than the output multiplies only the columns that exist
// (units of 16 for a 128-row MMA; whole 32-float chunks when B is read MN-major): an MMA's time is proportional
// to its N, and a 64-wide tile over a 16-column output would spend three quarters of the tensor pipe on zeros.
// The rest of the accumulator is never written, and never stored: the epilogue clips at N.
// MNI_B200_MMA_NARROW=0 keeps full-width MMAs.
int mma_n_for(const GemmProblem &p, const Plan &pl) {
    if (pl.cg != 1 || p.N >= pl.bn || env_int("MNI_B200_MMA_NARROW", 1) == 0) return pl.bn;
    const int64_t unit = p.B.k_major ? 16 : 32;
    return static_cast<int>(std::min<int64_t>(pl.bn, std::max<int64_t>(unit, (p.N + unit - 1) / unit * unit)));
}

uint32_t desc_hi_bits(uint32_t sbo_bytes, uint32_t layout_type) {
    // upper word of the shared-memory descriptor: SBO [32,46) | version 1 [46,48) | layout [61,64)
    return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (layout_type << 29);
}

template <int BN, int BK, bool FAST, int NS, int CG, bool TA = false, bool SK = false, int SG = 1>
cudaError_t launch_variant(const Plan &pl, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmC,
                           const CUtensorMap &tmD, const KParams &k, cudaStream_t stream) {
    // The shared-memory opt-in is an attribute of the function on ONE device: set once per device of the process
    // (a bit per device ordinal; setting it twice from two threads is harmless).
    static std::atomic<uint64_t> opted_in{0};
    int dev = 0;
    cudaError_t attr = cudaGetDevice(&dev);
    if (attr != cudaSuccess) return attr;
    const uint64_t bit = 1ull << (dev & 63);
    if ((opted_in.load(std::memory_order_acquire) & bit) == 0) {
        attr = cudaFuncSetAttribute(gemm_tc_kernel<BN, BK, FAST, NS, CG, TA, SK, SG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    227 * 1024);
        if (attr != cudaSuccess) return attr;
        opted_in.fetch_or(bit, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(pl.grid));
    cfg.blockDim = dim3(32 * (2 + NS + kEpiWarps));
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = CG;
    attrs[1].val.clusterDim.y = 1;
    attrs[1].val.clusterDim.z = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = CG == 2 ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, BK, FAST, NS, CG, TA, SK, SG>, tmA, tmB, tmC, tmD, k);
}

}  // namespace

// Flags of the balanced tail: per (CTA, parking place, epilogue warp) a ready flag, raised after an accumulator
// is parked, and per region of a tail tile a ticket; the unit that reduces a tile clears what it used, so the
// array is all zero between launches.
constexpr int kSkFlagCount = 3 * 256 * kEpiWarps;
constexpr int kSkFlagBanks = 2;            // bank 1 serves the launches a backward call puts on the library's side stream
__device__ unsigned int g_sk_flags[kSkFlagBanks * kSkFlagCount];

unsigned int *sk_flags_ptr() {
    static thread_local int cached_dev = -1;
    static thread_local unsigned int *ptr = nullptr;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    if (dev != cached_dev) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_sk_flags) != cudaSuccess) return nullptr;
        ptr = static_cast<unsigned int *>(p);
        cached_dev = dev;
    }
    return ptr;
}

// Role wait counters (diagnostics): cycles summed over CTAs that each role spent blocked.
__device__ unsigned long long g_role_waits[8];

unsigned long long *role_wait_ptr() {
    static thread_local int cached_dev = -1;
    static thread_local unsigned long long *ptr = nullptr;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    if (dev != cached_dev) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_role_waits) != cudaSuccess) return nullptr;
        ptr = static_cast<unsigned long long *>(p);
        cached_dev = dev;
    }
    return ptr;
}

int read_role_waits(uint64_t out[8], int reset) {
    unsigned long long *ptr = role_wait_ptr();
    if (!ptr) return fail(MNI_B200_ERR_CUDA, "role wait counters unavailable");
    MNI_CUDA(cudaDeviceSynchronize());
    MNI_CUDA(cudaMemcpy(out, ptr, 8 * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    if (reset) MNI_CUDA(cudaMemset(ptr, 0, 8 * sizeof(uint64_t)));
    return MNI_B200_OK;
}

// The kernel's view of a problem.  An output with few rows and many columns would fill at most half of
// every 128-row MMA; with the operands exchanged the kernel computes C^T in 64-wide tiles instead and its
// epilogue stores the 32 x 32 patches transposed, so C is written in place as before.
GemmProblem kernel_view(const GemmProblem &p, bool *transposed) {
    *transposed = false;
    const bool storable = (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 && p.ldc % 4 == 0 && p.c_bstride % 4 == 0 &&
                          p.N % 4 == 0 && env_int("MNI_B200_NO_TMA_STORE", 0) == 0 && env_int("MNI_B200_EPI_VECTOR", 0) == 0;
    if (p.D != nullptr || p.M > 64 || p.N < 256 || !storable || env_int("MNI_B200_TRANSPOSE_OUT", 1) == 0) return p;
    GemmProblem q = p;
    std::swap(q.A, q.B);
    std::swap(q.M, q.N);
    *transposed = true;
    return q;
}

bool gemm_tc_can_fuse_activation(const GemmProblem &p, int sm_count) {
    const Plan pl = make_plan(p, sm_count);
    auto aligned = [&](const float *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    return pl.splits == 1 && p.ldc % 4 == 0 && p.c_bstride % 4 == 0 && aligned(p.D) && (p.C == nullptr || aligned(p.C)) &&
           env_int("MNI_B200_NO_TMA_STORE", 0) == 0 && env_int("MNI_B200_EPI_VECTOR", 0) == 0;
}

size_t gemm_tc_partial_bytes(const GemmProblem &p0, int sm_count) {
    bool transposed = false;
    const GemmProblem p = kernel_view(p0, &transposed);
    const Plan pl = make_plan(p, sm_count);
    if (pl.sk) return static_cast<size_t>(pl.grid) * 2 * BM * pl.bn * sizeof(float);   // two parked accumulators per CTA
    if (pl.splits <= 1) return 0;
    return static_cast<size_t>(pl.splits) * p.batch * p.M * p.N * sizeof(float);
}

std::string gemm_tc_describe(const GemmProblem &p0, int sm_count) {
    bool transposed = false;
    const GemmProblem p = kernel_view(p0, &transposed);
    const Plan pl = make_plan(p, sm_count);
    const int chunk_k = env_int("MNI_B200_CHUNK_K", 1024);
    // pieces a whole unit's contraction is summed in (the kernel's first_piece rule)
    const long long iters = p.fold * ((p.K + pl.bk - 1) / pl.bk);
    const long long len = (iters + pl.splits - 1) / pl.splits;
    const long long ci = (chunk_k > 0 && p.D == nullptr) ? std::max(1, chunk_k / pl.bk) : 0;
    const int pieces = (ci > 0 && len > ci + ci / 2) ? static_cast<int>((len + ci - 1) / ci) : 1;
    char buf[320];
    snprintf(buf, sizeof(buf),
             "tensor m=%lld n=%lld k=%lld batch=%lld fold=%lld bn=%d bk=%d pair=%d tmem_a=%d stages=%d splits=%d "
             "tail=%d grid=%d exchanged=%d single_pass=%d pieces=%d mma_n=%d",
             static_cast<long long>(p.M), static_cast<long long>(p.N), static_cast<long long>(p.K),
             static_cast<long long>(p.batch), static_cast<long long>(p.fold), pl.bn, pl.bk, pl.cg == 2 ? 1 : 0,
             pl.ta ? 1 : 0, pl.stages, pl.splits, pl.sk ? 1 : 0, pl.grid, transposed ? 1 : 0, p.fast_tf32 ? 1 : 0,
             pieces, mma_n_for(p, pl));
    return buf;
}

int launch_gemm_tc(const GemmProblem &p0, float *partial, uint32_t *err_word, int sm_count,
                   cudaStream_t stream) {
    if (p0.M <= 0 || p0.N <= 0 || p0.batch <= 0) return MNI_B200_OK;
    bool transposed = false;
    const GemmProblem p = kernel_view(p0, &transposed);       // p.M / p.N are the kernel's; oM / oN the output's
    const int64_t oM = p0.M, oN = p0.N;
    const Plan pl = make_plan(p, sm_count);
    if (p.K <= 0) return fail(MNI_B200_ERR_ARG, "empty contraction reached the tensor-core launcher");
    if ((pl.splits > 1 || pl.sk) && partial == nullptr)
        return fail(MNI_B200_ERR_WORKSPACE, "split-K launch without partial storage");

    KParams k{};
    CUtensorMap tmA, tmB, tmC, tmD;
    if (p.D != nullptr && !gemm_tc_can_fuse_activation(p, sm_count))
        return fail(MNI_B200_ERR_ARG, "fused activation requested for a problem that cannot carry it");
    int rc = make_operand_map(&tmA, p.A, BM, pl.bk, &k.a_mode);
    if (rc) return rc;
    // B rows that exist in a tile wider than the output: with a K-major B (one box of whole rows) only those are
    // loaded, split and multiplied; the shared memory behind them is never read.
    const int mma_n = mma_n_for(p, pl);
    k.b_rows_live = (p.B.k_major && mma_n < pl.bn) ? mma_n : pl.bn / pl.cg;
    rc = make_operand_map(&tmB, p.B, k.b_rows_live, pl.bk, &k.b_mode);
    if (rc) return rc;

    // Epilogue: TMA store when the destination rows are 16-byte aligned, plain stores otherwise.
    float *dst = pl.splits > 1 ? partial : p.C;
    const int64_t dst_ld = pl.splits > 1 ? oN : p.ldc;
    const int64_t dst_bs = pl.splits > 1 ? p.M * p.N : p.c_bstride;
    const int64_t dst_batches = pl.splits > 1 ? static_cast<int64_t>(pl.splits) * p.batch : p.batch;
    const bool tma_ok = (reinterpret_cast<uintptr_t>(dst) & 15) == 0 && dst_ld % 4 == 0 && dst_bs % 4 == 0 &&
                        env_int("MNI_B200_NO_TMA_STORE", 0) == 0;
    k.epi_mode = kEpiPlainStores;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(dst) & 31) == 0 && dst_ld % 8 == 0 && dst_bs % 8 == 0;
    if (vec_ok && env_int("MNI_B200_EPI_VECTOR", 0) != 0) {
        k.epi_mode = kEpiVectorStores;
        tmC = tmA;
    } else if (tma_ok && (dst != nullptr || p.D != nullptr)) {
        if (dst != nullptr) {
            rc = make_output_map(&tmC, dst, oN, oM, dst_batches, dst_ld, dst_bs);
            if (rc) return rc;
        } else {
            tmC = tmA;
        }
        k.epi_mode = (p.accumulate && pl.splits == 1) ? kEpiTmaReduce : kEpiTmaStore;
    } else {
        tmC = tmA;   // unused by the plain-store epilogue, but must be a valid object
    }
    tmD = tmC;
    if (p.D != nullptr) {
        rc = make_output_map(&tmD, p.D, p.N, p.M, p.batch, p.ldc, p.c_bstride);
        if (rc) return rc;
        k.act = 1;
        k.store_pre = p.C != nullptr ? 1 : 0;
    }

    k.M = static_cast<int>(p.M);
    k.N = static_cast<int>(p.N);
    k.transpose_out = transposed ? 1 : 0;
    k.tiles_m = pl.tiles_m;
    k.tiles_n = pl.tiles_n;
    k.group_m = std::max(1, std::min(pl.tiles_m, env_int("MNI_B200_GROUP_M", 16)));
    k.batch = static_cast<int>(p.batch);
    k.kiters = static_cast<int>((p.K + pl.bk - 1) / pl.bk);
    k.fold = static_cast<int>(p.fold);
    k.splits = pl.splits;
    k.dep_mode = p.dep_mode;
    {
        // Longest accumulation chain in tensor memory, in contraction elements (MNI_B200_CHUNK_K, 0 = unlimited).
        // The fused activation needs the whole sum in one accumulator.
        const int chunk_k = env_int("MNI_B200_CHUNK_K", 1024);
        k.chunk_iters = (chunk_k > 0 && p.D == nullptr) ? std::max(1, chunk_k / pl.bk) : 0;
    }
    k.a_batch = static_cast<int>(p.A.batch);
    k.a_d1 = static_cast<int>(p.A.bshape[1]);
    k.a_d2 = static_cast<int>(p.A.bshape[2]);
    k.b_batch = static_cast<int>(p.B.batch);
    k.b_d1 = static_cast<int>(p.B.bshape[1]);
    k.b_d2 = static_cast<int>(p.B.bshape[2]);
    {
        const int last_gm = k.tiles_m % k.group_m == 0 ? k.group_m : k.tiles_m % k.group_m;
        k.fd_splits = make_fastdiv(k.splits);
        k.fd_per_batch = make_fastdiv(static_cast<long long>(k.tiles_m) * k.tiles_n);
        k.fd_group_sz = make_fastdiv(static_cast<long long>(k.group_m) * k.tiles_n);
        k.fd_group_m = make_fastdiv(k.group_m);
        k.fd_last_gm = make_fastdiv(last_gm);
        k.fd_a_cnt = make_fastdiv(k.a_batch); k.fd_a_d1 = make_fastdiv(k.a_d1); k.fd_a_d2 = make_fastdiv(k.a_d2);
        k.fd_b_cnt = make_fastdiv(k.b_batch); k.fd_b_d1 = make_fastdiv(k.b_d1); k.fd_b_d2 = make_fastdiv(k.b_d2);
    }
    k.stages = pl.stages;
    k.epi_patches = pl.patches;
    k.idesc = (1u << 4) | (2u << 7) | (2u << 10) | (((p.A.k_major || pl.ta) ? 0u : 1u) << 15) |
              ((p.B.k_major ? 0u : 1u) << 16) | (static_cast<uint32_t>(mma_n >> 3) << 17) |
              (static_cast<uint32_t>((BM * pl.cg) >> 4) << 24);
    // K-major tile: rows of BK floats, 8-row groups SBO apart, swizzle span = one row.
    // MN-major tile: 32-float chunks of BK k-rows (LBO apart); the 32-byte-unit swizzle repeats every
    // 4 k-rows (SBO = 512), and one 8-deep k-step spans two such groups (1024 bytes).
    const uint32_t k_layout = pl.bk == 32 ? 2u : 4u;   // SWIZZLE_128B : SWIZZLE_64B
    const uint32_t k_sbo = static_cast<uint32_t>(8 * pl.bk * 4);
    const uint32_t mn_lbo = static_cast<uint32_t>(pl.bk * 128);
    const uint32_t mn_sbo = 512, mn_layout = 1;        // SWIZZLE_128B_BASE32B
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
    {
        // Tests shorten the limit of the device-side waits; the withhold hook (a stage that never fills, so
        // that the waits do run out) is honoured only together with a limit of at most ~0.1 s.
        const char *w = getenv("MNI_B200_WAIT_CYCLES");
        const long long wc = w && *w ? atoll(w) : 0;
        k.wait_cycles = wc > 0 ? wc : kWaitCycles;
        k.withhold_at = k.wait_cycles <= 200000000LL ? env_int("MNI_B200_TEST_WITHHOLD_KBLOCK", 0) : 0;
    }
    k.prof = env_int("MNI_B200_ROLE_WAITS", 0) ? role_wait_ptr() : nullptr;
    k.sk = pl.sk ? 1 : 0;
    k.sk_first_tile = pl.sk_first_tile;
    k.sk_partial = pl.sk ? partial : nullptr;
    k.sk_flags = nullptr;
    if (pl.sk) {
        k.sk_flags = sk_flags_ptr();
        if (!k.sk_flags) return fail(MNI_B200_ERR_CUDA, "balanced-tail flags unavailable");
        k.sk_flags += (p.flag_bank > 0 ? 1 : 0) * kSkFlagCount;
        // ready flags for 2 parking places per CTA, then one ticket per region of a tail tile (fewer tiles than CTAs)
        if (pl.grid * 3 * kEpiWarps > kSkFlagCount) return fail(MNI_B200_ERR_CUDA, "balanced-tail flag array too small");
    }

    // Two split groups pay when the k-loop is long enough for the second k-block in flight to matter (measured:
    // K = 512 per unit 33.6 -> 32.8 us per attention-shaped product, 128 k-blocks 57.9 -> 54.4 us; four k-blocks per
    // unit are no faster).  MNI_B200_SPLIT_GROUPS=1/2 forces either.
    int split_groups = 1;
    if (pl.ta) {
        const long long unit_iters = (static_cast<long long>(k.fold) * k.kiters + pl.splits - 1) / pl.splits;
        const int sg_env = env_int("MNI_B200_SPLIT_GROUPS", 0);
        split_groups = (sg_env == 1 || sg_env == 2) ? sg_env : (unit_iters >= 12 ? 2 : 1);
    }
    cudaError_t e = cudaErrorInvalidValue;
    if (pl.sk) {
        if (pl.ta && pl.bn == 64 && split_groups == 2) e = launch_variant<64, 32, false, 8, 1, true, true, 2>(pl, tmA, tmB, tmC, tmD, k, stream);
        else if (pl.ta && pl.bn == 64) e = launch_variant<64, 32, false, 8, 1, true, true>(pl, tmA, tmB, tmC, tmD, k, stream);
        else if (pl.ta && pl.bn == 128 && split_groups == 2) e = launch_variant<128, 32, false, 8, 1, true, true, 2>(pl, tmA, tmB, tmC, tmD, k, stream);
        else if (pl.ta && pl.bn == 128) e = launch_variant<128, 32, false, 8, 1, true, true>(pl, tmA, tmB, tmC, tmD, k, stream);
        else if (!p.fast_tf32 && pl.bk == 16) e = launch_variant<256, 16, false, 8, 2, false, true>(pl, tmA, tmB, tmC, tmD, k, stream);
        else if (!p.fast_tf32 && pl.bk == 32) e = launch_variant<256, 32, false, 8, 2, false, true>(pl, tmA, tmB, tmC, tmD, k, stream);
        else if (pl.bk == 16) e = launch_variant<256, 16, true, 4, 2, false, true>(pl, tmA, tmB, tmC, tmD, k, stream);
        else e = launch_variant<256, 32, true, 4, 2, false, true>(pl, tmA, tmB, tmC, tmD, k, stream);
    } else if (pl.ta) {
        if (pl.bn == 64 && split_groups == 2) e = launch_variant<64, 32, false, 8, 1, true, false, 2>(pl, tmA, tmB, tmC, tmD, k, stream);
        else if (pl.bn == 64) e = launch_variant<64, 32, false, 8, 1, true>(pl, tmA, tmB, tmC, tmD, k, stream);
        else if (split_groups == 2) e = launch_variant<128, 32, false, 8, 1, true, false, 2>(pl, tmA, tmB, tmC, tmD, k, stream);
        else e = launch_variant<128, 32, false, 8, 1, true>(pl, tmA, tmB, tmC, tmD, k, stream);
    }
#define MNI_VARIANT(BN_, BK_)                                                                         \
    if (pl.cg == 1 && !pl.ta && pl.bn == BN_ && pl.bk == BK_) {                                                 \
        if (p.fast_tf32) e = launch_variant<BN_, BK_, true, 4, 1>(pl, tmA, tmB, tmC, tmD, k, stream);      \
        else e = launch_variant<BN_, BK_, false, 8, 1>(pl, tmA, tmB, tmC, tmD, k, stream);                 \
    }
#define MNI_PAIR_VARIANT(BN_, BK_)                                                                    \
    if (pl.cg == 2 && !pl.sk && pl.bn == BN_ && pl.bk == BK_) {                                                 \
        if (p.fast_tf32) e = launch_variant<BN_, BK_, true, 4, 2>(pl, tmA, tmB, tmC, tmD, k, stream);      \
        else e = launch_variant<BN_, BK_, false, 8, 2>(pl, tmA, tmB, tmC, tmD, k, stream);                 \
    }
    MNI_PAIR_VARIANT(64, 32) MNI_PAIR_VARIANT(128, 32) MNI_PAIR_VARIANT(256, 16) MNI_PAIR_VARIANT(256, 32)
#undef MNI_PAIR_VARIANT
    MNI_VARIANT(64, 32) MNI_VARIANT(128, 32) MNI_VARIANT(256, 16) MNI_VARIANT(256, 32)
#undef MNI_VARIANT
    if (e != cudaSuccess) return fail(MNI_B200_ERR_CUDA, "gemm_tc_kernel set-up failed: %s", cudaGetErrorString(e));
    MNI_LAUNCH_CHECK("gemm_tc_kernel");
    if (pl.splits > 1) {
        const long long rows = static_cast<long long>(p.batch) * oM;
        const bool vec = oN % 4 == 0 && p.ldc % 4 == 0 && p.c_bstride % 4 == 0 &&
                         ((reinterpret_cast<uintptr_t>(p.C) | reinterpret_cast<uintptr_t>(partial) |
                           reinterpret_cast<uintptr_t>(p.bias)) & 15) == 0;
        const long long items = rows * (vec ? oN / 4 : oN);
        const unsigned blocks = static_cast<unsigned>((items + 255) / 256);
        const bool small = items < (1LL << 31) - 256;
#define MNI_REDUCE(V_, I_)                                                                                          \
    e = launch_dependent(splitk_reduce_kernel<V_, I_>, dim3(blocks), dim3(256), 0, stream, partial, p.C, p.ldc,        \
                         p.c_bstride, p.bias, p.accumulate ? 1 : 0, pl.splits, rows, static_cast<int>(oM),          \
                         static_cast<int>(oN))
        if (vec && small) MNI_REDUCE(float4, unsigned);
        else if (vec) MNI_REDUCE(float4, long long);
        else if (small) MNI_REDUCE(float, unsigned);
        else MNI_REDUCE(float, long long);
#undef MNI_REDUCE
        if (e != cudaSuccess) return fail(MNI_B200_ERR_CUDA, "splitk_reduce_kernel launch failed: %s", cudaGetErrorString(e));
        MNI_LAUNCH_CHECK("splitk_reduce_kernel");
    }
    return MNI_B200_OK;
}

}  // namespace mni
