// C ABI of libmni_b200.so: argument checking, view classification, path selection and
// scratch management.  All arithmetic happens in the kernels of gemm_tcgen05.cu,
// skinny.cu and pointwise.cu; there is no host or library (cuBLAS) fallback.
#include "internal.h"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <vector>

namespace mni {

std::atomic<uint64_t> g_launches{0};

namespace {

thread_local char t_error[512] = "";

__device__ unsigned int g_err_word;   // first timeout code recorded by any kernel of the library

constexpr int kMaxDevices = 64;

struct DeviceState {
    std::mutex mu;
    bool init = false;
    int sm_count = 0;
    int sm_reserve = 0;           // SMs the tensor-core launches leave free (mni_b200_sm_reserve)
    int cc_major = 0;
    uint8_t *ws = nullptr;        // library-owned scratch
    size_t ws_bytes = 0;
    uint8_t *user_ws = nullptr;   // caller-provided scratch (takes precedence)
    size_t user_bytes = 0;
    unsigned int *err_word = nullptr;
    // Second stream of small backward calls: dA and dB of a small problem each occupy a fraction of
    // the GPU, so they are issued side by side (fork / join through events; also under stream capture).
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
};
DeviceState g_dev[kMaxDevices];

int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

// x^n in f32 the way Rust's f32::powi evaluates it (ops/optimizer.rs:26-27 call it for the bias corrections):
// binary exponentiation from the lowest exponent bit up -- multiply the result in when the bit is set,
// square the base between bits -- every product rounded to f32.  O(log n) and, from n = 4 on, rounded
// differently from n successive multiplications.
float powi_f32(float x, uint32_t n) {
    float r = 1.0f;
    while (true) {
        if (n & 1u) r *= x;
        n >>= 1;
        if (n == 0) break;
        x *= x;
    }
    return r;
}

// Largest M*N*K*batch for which the two gradient products of a backward call are issued side by side.
double overlap_work_limit() {
    const char *v = getenv("MNI_B200_BWD_OVERLAP_WORK");
    return v && *v ? atof(v) : 4.0e9;   // measured: helps up to the attention-shaped products (1.6e9), neutral beyond
}

// Row counts up to which the streaming kernels beat the tensor path (measured at K = N = 4096 with a weight
// that is not in L2: dx 19.4 vs 23.6 us at 5 rows and 31.0 vs 23.7 at 8; dW 13.5 vs 16.9 at 8 rows and 21.8 vs
// 17.0 at 12).  The forward's limit depends on which of its two kernels can run: skinny_fwd_row_limit.
constexpr int64_t kSkinnyDxRows = 5, kSkinnyDwRows = 8;

bool env_flag(const char *name, int dflt) {
    const char *v = getenv(name);
    return (v && *v ? atoi(v) : dflt) != 0;
}

// Bump allocator over the device's scratch.  In dry mode nothing is touched: the
// same host logic runs and only the byte count is produced (workspace_query).
struct Arena {
    DeviceState *st = nullptr;
    bool dry = false;
    size_t used = 0;
    std::vector<std::pair<size_t, size_t>> blocks;   // (offset, bytes) in request order
    size_t reserve(size_t bytes) {
        const size_t off = used;
        used += (bytes + 255) & ~static_cast<size_t>(255);
        return off;
    }
};

int device_state(DeviceState **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(MNI_B200_ERR_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(MNI_B200_ERR_DEVICE, "device ordinal %d out of range", dev);
    DeviceState &st = g_dev[dev];
    // First use of a device: under the device's lock, so that two host threads that make their first
    // call together initialise it once (init is only ever read or written with the lock held).
    std::lock_guard<std::mutex> lock(st.mu);
    if (!st.init) {
        cudaDeviceProp prop;
        e = cudaGetDeviceProperties(&prop, dev);
        if (e != cudaSuccess) return fail(MNI_B200_ERR_DEVICE, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
        if (prop.major != 10)
            return fail(MNI_B200_ERR_DEVICE,
                        "device %d is compute capability %d.%d; this library only carries sm_100a code", dev,
                        prop.major, prop.minor);
        st.sm_count = prop.multiProcessorCount;
        st.cc_major = prop.major;
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_err_word);
        if (e != cudaSuccess) return fail(MNI_B200_ERR_CUDA, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        st.err_word = static_cast<unsigned int *>(p);
        e = cudaMemset(st.err_word, 0, sizeof(unsigned int));
        if (e != cudaSuccess) return fail(MNI_B200_ERR_CUDA, "cudaMemset: %s", cudaGetErrorString(e));
        if (!st.side) e = cudaStreamCreateWithFlags(&st.side, cudaStreamNonBlocking);
        if (e == cudaSuccess && !st.ev_fork) e = cudaEventCreateWithFlags(&st.ev_fork, cudaEventDisableTiming);
        if (e == cudaSuccess && !st.ev_join) e = cudaEventCreateWithFlags(&st.ev_join, cudaEventDisableTiming);
        if (e != cudaSuccess) return fail(MNI_B200_ERR_CUDA, "side stream set-up: %s", cudaGetErrorString(e));
        st.init = true;
    }
    *out = &st;
    return MNI_B200_OK;
}

// True while `stream` records into a CUDA graph.
bool stream_is_capturing(cudaStream_t stream) {
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &status) != cudaSuccess) {
        cudaGetLastError();   // the legacy stream beside another stream's capture: not capturing itself
        return false;
    }
    return status != cudaStreamCaptureStatusNone;
}

// Makes `bytes` of scratch available and returns its base.
int scratch_base(DeviceState &st, size_t bytes, cudaStream_t stream, uint8_t **base) {
    if (st.user_ws) {
        if (bytes > st.user_bytes)
            return fail(MNI_B200_ERR_WORKSPACE, "caller-provided scratch holds %zu bytes, %zu needed", st.user_bytes,
                        bytes);
        *base = st.user_ws;
        return MNI_B200_OK;
    }
    if (bytes > st.ws_bytes) {
        const size_t want = bytes + bytes / 4 + (1u << 20);
        // Growing frees the old buffer, which a capturing stream must not do (it would end the capture in
        // an error) and which would leave the nodes already recorded with a dangling address.
        if (st.ws && stream_is_capturing(stream))
            return fail(MNI_B200_ERR_WORKSPACE,
                        "scratch would have to grow from %zu to %zu bytes while the stream is capturing: run the call "
                        "once before the capture, or hand the library a buffer (mni_b200_workspace_set)",
                        st.ws_bytes, bytes);
        if (st.ws) {
            // cudaFree waits for work that may still read the old buffer.
            cudaError_t e = cudaFree(st.ws);
            st.ws = nullptr;
            st.ws_bytes = 0;
            if (e != cudaSuccess) return fail(MNI_B200_ERR_WORKSPACE, "cudaFree(scratch): %s", cudaGetErrorString(e));
        }
        void *p = nullptr;
        cudaError_t e = cudaMalloc(&p, want);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(MNI_B200_ERR_WORKSPACE, "cudaMalloc(%zu) for scratch failed: %s", want, cudaGetErrorString(e));
        }
        st.ws = static_cast<uint8_t *>(p);
        st.ws_bytes = want;
    }
    *base = st.ws;
    return MNI_B200_OK;
}

// ------------------------------------------------------------------ shapes
int64_t prod(const int64_t *s, int n) {
    int64_t p = 1;
    for (int i = 0; i < n; ++i) p *= s[i];
    return p;
}

// utils.rs:3-20
int broadcast_shape(const int64_t *a, int an, const int64_t *b, int bn, int64_t *out) {
    const int nd = std::max(an, bn);
    for (int i = 0; i < nd; ++i) {
        const int64_t da = i < nd - an ? 1 : a[i - (nd - an)];
        const int64_t db = i < nd - bn ? 1 : b[i - (nd - bn)];
        if (da == db) out[i] = da;
        else if (da == 1) out[i] = db;
        else if (db == 1) out[i] = da;
        else return -1;
    }
    return nd;
}

int check_view(const mni_b200_view *v, const char *name, int min_nd) {
    if (!v) return fail(MNI_B200_ERR_ARG, "%s is null", name);
    if (v->ndim < min_nd) return fail(MNI_B200_ERR_NDIM, "matmul requires at least 2D tensors (%s has %d)", name, v->ndim);
    if (v->ndim > MNI_B200_MAX_DIMS) return fail(MNI_B200_ERR_ARG, "%s has %d dims (max %d)", name, v->ndim, MNI_B200_MAX_DIMS);
    for (int d = 0; d < v->ndim; ++d) {
        if (v->shape[d] < 0 || v->stride[d] < 0) return fail(MNI_B200_ERR_ARG, "%s has a negative extent or stride", name);
        if (v->shape[d] > 0x7fffffffLL) return fail(MNI_B200_ERR_TOO_LARGE, "%s dim %d = %lld exceeds 2^31-1", name, d, (long long)v->shape[d]);
    }
    if (!v->ptr && prod(v->shape, v->ndim) > 0) return fail(MNI_B200_ERR_ARG, "%s has a null data pointer", name);
    return MNI_B200_OK;
}

// A matrix operand read through a TMA descriptor.  `transposed` selects which of the
// view's last two dims is the contraction dim: false -> [.., rows, k], true -> [.., k, rows].
// Returns false if the view cannot be described (then the caller packs it first).
bool view_to_operand(const mni_b200_view &v, bool transposed, Operand &op) {
    const int nd = v.ndim;
    const int64_t s_r = transposed ? v.stride[nd - 1] : v.stride[nd - 2];
    const int64_t s_k = transposed ? v.stride[nd - 2] : v.stride[nd - 1];
    op.ptr = v.ptr;
    op.rows = transposed ? v.shape[nd - 1] : v.shape[nd - 2];
    op.kdim = transposed ? v.shape[nd - 2] : v.shape[nd - 1];
    if ((reinterpret_cast<uintptr_t>(v.ptr) & 15) != 0) return false;
    const bool k_ok = (s_k == 1 || op.kdim == 1) && (op.rows == 1 || (s_r > 0 && s_r % 4 == 0));
    const bool mn_ok = (s_r == 1 || op.rows == 1) && (op.kdim == 1 || (s_k > 0 && s_k % 4 == 0));
    if (k_ok) {
        op.k_major = true;
        op.ld = s_r;
    } else if (mn_ok) {
        op.k_major = false;
        op.ld = s_k;
    } else {
        return false;
    }
    // Batch dims: drop extent-1 dims, merge dims that are contiguous with each other.
    int64_t bs[MNI_B200_MAX_DIMS], bt[MNI_B200_MAX_DIMS];
    int nb = 0;
    op.batch = 1;
    for (int d = 0; d < nd - 2; ++d) {
        op.batch *= v.shape[d];
        if (v.shape[d] == 1) continue;
        if (nb > 0 && bt[nb - 1] == v.stride[d] * v.shape[d]) {
            bs[nb - 1] *= v.shape[d];
            bt[nb - 1] = v.stride[d];
        } else {
            bs[nb] = v.shape[d];
            bt[nb] = v.stride[d];
            ++nb;
        }
    }
    if (nb > 3) return false;
    for (int i = 0; i < 3; ++i) { op.bshape[i] = 1; op.bstride[i] = 0; }
    for (int i = 0; i < nb; ++i) {
        if (bt[i] <= 0 || bt[i] % 4 != 0) return false;
        if (bs[i] > 0x7fffffffLL) return false;
        op.bshape[3 - nb + i] = bs[i];
        op.bstride[3 - nb + i] = bt[i];
    }
    return true;
}

struct Call {
    DeviceState *st;
    Arena arena;
    cudaStream_t stream;
    uint32_t flags;
    uint8_t *base = nullptr;   // resolved scratch base (real mode, second pass)
    int flag_bank = 0;         // 1 while launches go to the library's side stream / for the second product of a pair
    int dep_mode = 0;          // GemmProblem::dep_mode of the tensor-path launches issued now
    int sm_share = 1;          // 2 while grad_a and grad_b run side by side: each is planned for half of the SMs
    std::string *plan_log = nullptr;   // mni_b200_plan_describe: one line per launch the call would make
    const char *label = "";            // which product the launches logged now belong to
    void note(const std::string &what) const {
        if (plan_log) *plan_log += std::string(label) + what + "\n";
    }
    // SMs the persistent tensor-core grids are planned for: all of them minus the caller's reservation, divided
    // between the products that run at the same time (kept even, CTA pairs take two)
    int gemm_sms() const { return std::max(8, ((st->sm_count - st->sm_reserve) / sm_share) & ~1); }
    bool dry() const { return arena.dry; }
    float *at(size_t off) const { return reinterpret_cast<float *>(base + off); }
};

// Gathers a view into scratch as [batch_flat, R, C] with the last dim padded to a multiple of 4.
int pack_view(Call &c, const mni_b200_view &v, mni_b200_view *packed, size_t *offset) {
    const int nd = v.ndim;
    const int64_t cols = v.shape[nd - 1], rows = v.shape[nd - 2];
    const int64_t ld = std::max<int64_t>(4, round_up(cols, 4));
    const int64_t batch = prod(v.shape, nd - 2);
    const size_t bytes = static_cast<size_t>(batch * rows * ld) * sizeof(float);
    const size_t off = c.arena.reserve(bytes);
    *offset = off;
    packed->ndim = 3;
    packed->shape[0] = batch; packed->shape[1] = rows; packed->shape[2] = cols;
    packed->stride[0] = rows * ld; packed->stride[1] = ld; packed->stride[2] = 1;
    packed->ptr = c.dry() ? reinterpret_cast<const float *>(static_cast<uintptr_t>(256)) : c.at(off);
    c.note("gather of a strided operand into scratch");
    if (c.dry()) return MNI_B200_OK;
    return launch_pack(v, c.at(off), ld, c.stream);
}

// Operand from a view, packing it into scratch when TMA cannot describe it.
int make_operand(Call &c, const mni_b200_view &v, bool transposed, Operand &op) {
    const bool force_pack = (c.flags & MNI_B200_FORCE_PACK) != 0;
    if (!force_pack && view_to_operand(v, transposed, op)) return MNI_B200_OK;
    mni_b200_view packed;
    size_t off;
    int rc = pack_view(c, v, &packed, &off);
    if (rc) return rc;
    if (!view_to_operand(packed, transposed, op)) return fail(MNI_B200_ERR_ARG, "packed operand is not describable");
    // The packed copy is flat in the batch: keep the original flat batch count.
    return MNI_B200_OK;
}

int run_gemm(Call &c, GemmProblem &p) {
    p.fast_tf32 = (c.flags & MNI_B200_PRECISION_TF32) != 0;
    p.force_splits = static_cast<int>((c.flags >> 16) & 0xffu);
    p.flag_bank = c.flag_bank;
    p.dep_mode = c.dep_mode;
    if (p.M > 0x7fffffffLL || p.N > 0x7fffffffLL || p.K > 0x7fffffffLL || p.batch * p.fold > 0x7fffffffLL ||
        p.batch * ((p.M + 127) / 128) * ((p.N + 63) / 64) > 0x3fffffffLL)
        return fail(MNI_B200_ERR_TOO_LARGE, "GEMM %lld x %lld x %lld (batch %lld) exceeds the kernels' int32 indexing",
                    (long long)p.M, (long long)p.N, (long long)p.K, (long long)p.batch);
    const size_t pbytes = gemm_tc_partial_bytes(p, c.gemm_sms());
    size_t poff = 0;
    if (pbytes) poff = c.arena.reserve(pbytes);
    if (c.plan_log) c.note(gemm_tc_describe(p, c.gemm_sms()));
    if (c.dry()) return MNI_B200_OK;
    return launch_gemm_tc(p, pbytes ? c.at(poff) : nullptr, c.st->err_word, c.gemm_sms(), c.stream);
}

int zero_or_bias_fill(Call &c, float *out, int64_t rows, int64_t n, const float *bias, bool accumulate) {
    if (c.dry() || rows * n == 0) return MNI_B200_OK;
    if (!accumulate) MNI_CUDA(cudaMemsetAsync(out, 0, static_cast<size_t>(rows * n) * sizeof(float), c.stream));
    if (bias) return launch_add_bias(out, bias, out, rows, n, c.stream);
    return MNI_B200_OK;
}

struct Shapes {
    int64_t M, K, N;
    int64_t out_batch[MNI_B200_MAX_DIMS];
    int out_nb;
    int64_t batch, a_batch, b_batch;
};

int analyse(const mni_b200_view *a, const mni_b200_view *b, Shapes &s) {
    int rc = check_view(a, "a", 2);
    if (rc) return rc;
    rc = check_view(b, "b", 2);
    if (rc) return rc;
    s.M = a->shape[a->ndim - 2];
    s.K = a->shape[a->ndim - 1];
    s.N = b->shape[b->ndim - 1];
    if (b->shape[b->ndim - 2] != s.K)
        return fail(MNI_B200_ERR_INNER_DIM, "matmul inner dimensions must match: %lld vs %lld", (long long)s.K,
                    (long long)b->shape[b->ndim - 2]);
    s.out_nb = broadcast_shape(a->shape, a->ndim - 2, b->shape, b->ndim - 2, s.out_batch);
    if (s.out_nb < 0) return fail(MNI_B200_ERR_BROADCAST, "batch shapes are not broadcastable");
    s.batch = prod(s.out_batch, s.out_nb);
    s.a_batch = prod(a->shape, a->ndim - 2);
    s.b_batch = prod(b->shape, b->ndim - 2);
    return MNI_B200_OK;
}

// ------------------------------------------------------------------ forward
int fwd_body(Call &c, const mni_b200_view *a, const mni_b200_view *b, float *out, const float *bias) {
    Shapes s;
    int rc = analyse(a, b, s);
    if (rc) return rc;
    if (!out && s.batch * s.M * s.N > 0) return fail(MNI_B200_ERR_ARG, "c is null");
    const bool accumulate = (c.flags & MNI_B200_ACCUMULATE_C) != 0;
    if (s.batch * s.M * s.N == 0) return MNI_B200_OK;
    if (s.K == 0) return zero_or_bias_fill(c, out, s.batch * s.M, s.N, bias, accumulate);

    if (!*c.label) c.label = "forward: ";
    const bool want_skinny = (c.flags & MNI_B200_FORCE_SKINNY_PATH) != 0 ||
                             ((c.flags & MNI_B200_FORCE_TENSOR_PATH) == 0 && s.M <= skinny_fwd_row_limit(s.N));
    if (want_skinny && s.batch == 1 && skinny_fwd_supported(s.M, s.N, s.K)) {
        const int an = a->ndim, bn = b->ndim;
        const bool a_ok = a->stride[an - 1] == 1 || s.K == 1;
        const bool b_ok = (b->stride[bn - 1] == 1 || s.N == 1) && (b->stride[bn - 2] % 4 == 0 || s.K == 1) &&
                          (reinterpret_cast<uintptr_t>(b->ptr) & 15) == 0;
        if (a_ok && b_ok) {
            const size_t pbytes = skinny_fwd_partial_bytes(s.M, s.N, s.K, c.st->sm_count);
            const size_t poff = c.arena.reserve(pbytes);
            c.note("streaming (skinny) forward kernel");
            if (c.dry()) return MNI_B200_OK;
            const int64_t ldw = s.K == 1 ? round_up(s.N, 4) : b->stride[bn - 2];
            return launch_skinny_fwd(a->ptr, a->stride[an - 2], b->ptr, ldw, out, s.N, bias, accumulate, s.M, s.N,
                                     s.K, c.at(poff), c.st->sm_count, c.stream);
        }
    }

    GemmProblem p;
    rc = make_operand(c, *a, false, p.A);
    if (rc) return rc;
    rc = make_operand(c, *b, true, p.B);
    if (rc) return rc;
    p.A.batch = s.a_batch;
    p.B.batch = s.b_batch;
    p.M = s.M; p.N = s.N; p.K = s.K;
    p.batch = s.batch;
    p.fold = 1;
    p.C = out;
    p.ldc = s.N;
    p.c_bstride = s.M * s.N;
    p.bias = bias;
    p.accumulate = accumulate;
    return run_gemm(c, p);
}

// Forward with the bias + GELU epilogue: pre = a . b (optional output), out = gelu(pre + bias).
int fwd_gelu_body(Call &c, const mni_b200_view *a, const mni_b200_view *b, const float *bias, float *pre,
                  float *out) {
    Shapes s;
    int rc = analyse(a, b, s);
    if (rc) return rc;
    const int64_t rows = s.batch * s.M;
    if (rows * s.N == 0) return MNI_B200_OK;
    if (!bias || !out) return fail(MNI_B200_ERR_ARG, "bias and out must not be null");
    const uint32_t saved_flags = c.flags;
    c.flags &= ~static_cast<uint32_t>(MNI_B200_ACCUMULATE_C);
    const bool skinny = (c.flags & MNI_B200_FORCE_SKINNY_PATH) != 0 ||
                        ((c.flags & MNI_B200_FORCE_TENSOR_PATH) == 0 && s.M <= skinny_fwd_row_limit(s.N));
    if (s.K > 0 && !skinny) {
        GemmProblem p;
        rc = make_operand(c, *a, false, p.A);
        if (rc) return rc;
        rc = make_operand(c, *b, true, p.B);
        if (rc) return rc;
        p.A.batch = s.a_batch;
        p.B.batch = s.b_batch;
        p.M = s.M; p.N = s.N; p.K = s.K;
        p.batch = s.batch;
        p.C = pre; p.D = out;
        p.ldc = s.N; p.c_bstride = s.M * s.N;
        p.bias = bias;
        p.fast_tf32 = (c.flags & MNI_B200_PRECISION_TF32) != 0;
        p.force_splits = static_cast<int>((c.flags >> 16) & 0xffu);
        if (gemm_tc_can_fuse_activation(p, c.gemm_sms())) {
            rc = run_gemm(c, p);
            c.flags = saved_flags;
            return rc;
        }
    }
    // Not fusable (split-K, skinny rows, unaligned rows): the product first, then the pointwise kernel.
    float *tmp = pre;
    size_t off = 0;
    if (!tmp) off = c.arena.reserve(static_cast<size_t>(rows * s.N) * sizeof(float));
    if (!tmp && !c.dry()) tmp = c.at(off);
    rc = fwd_body(c, a, b, c.dry() && !tmp ? reinterpret_cast<float *>(static_cast<uintptr_t>(256)) : tmp, nullptr);
    c.flags = saved_flags;
    if (rc || c.dry()) return rc;
    return launch_bias_gelu(tmp, bias, out, rows, s.N, c.stream);
}

// ------------------------------------------------------------------ backward
// One gradient: G[ob.., R, Cn] = X . Y (a GEMM over `kdim`) reduced to `target`'s shape.
//   X supplies the rows, Y the columns; both already as Operands with flat batch counts.
int grad_gemm(Call &c, Operand X, Operand Y, int64_t R, int64_t Cn, int64_t kdim, const int64_t *ob, int onb,
              const mni_b200_view &target, float *out, bool accumulate) {
    const int64_t obatch = prod(ob, onb);
    const int tnb = target.ndim - 2;
    const int64_t tbatch = prod(target.shape, tnb);
    bool same = true;
    {   // target batch dims, right-aligned against ob, all equal?
        if (tnb > onb) same = false;
        for (int i = 0; same && i < onb; ++i) {
            const int64_t td = i < onb - tnb ? 1 : target.shape[i - (onb - tnb)];
            if (td != ob[i]) same = false;
        }
    }
    GemmProblem p;
    p.A = X; p.B = Y;
    p.M = R; p.N = Cn; p.K = kdim;
    p.bias = nullptr;
    if (same || obatch == 1) {
        p.batch = obatch; p.fold = 1;
        p.C = out; p.ldc = Cn; p.c_bstride = R * Cn; p.accumulate = accumulate;
        return run_gemm(c, p);
    }
    if (tbatch == 1) {
        // The operand was broadcast over every batch: sum the batches inside the contraction.
        p.batch = 1; p.fold = obatch;
        p.C = out; p.ldc = Cn; p.c_bstride = R * Cn; p.accumulate = accumulate;
        return run_gemm(c, p);
    }
    // Partial broadcast: full batched product into scratch, then the device-side unbroadcast.
    const size_t bytes = static_cast<size_t>(obatch * R * Cn) * sizeof(float);
    const size_t off = c.arena.reserve(bytes);
    p.batch = obatch; p.fold = 1;
    p.C = c.dry() ? nullptr : c.at(off);
    p.ldc = Cn; p.c_bstride = R * Cn; p.accumulate = false;
    int rc = run_gemm(c, p);
    c.note("sum over the broadcast batch dims (unbroadcast kernel)");
    if (rc || c.dry()) return rc;
    int64_t gshape[MNI_B200_MAX_DIMS + 2];
    for (int i = 0; i < onb; ++i) gshape[i] = ob[i];
    gshape[onb] = R; gshape[onb + 1] = Cn;
    return launch_unbroadcast(c.at(off), gshape, onb + 2, target.shape, target.ndim, out, accumulate, c.stream);
}

int bwd_body(Call &c, const mni_b200_view *a, const mni_b200_view *b, const mni_b200_view *dc, float *da,
             float *db, float *dbias) {
    Shapes s;
    int rc = analyse(a, b, s);
    if (rc) return rc;
    rc = check_view(dc, "dc", 2);
    if (rc) return rc;
    const int gn = dc->ndim;
    if (dc->shape[gn - 2] != s.M || dc->shape[gn - 1] != s.N)
        return fail(MNI_B200_ERR_ARG, "dc is [.., %lld, %lld] but the forward output is [.., %lld, %lld]",
                    (long long)dc->shape[gn - 2], (long long)dc->shape[gn - 1], (long long)s.M, (long long)s.N);
    const int64_t g_batch = prod(dc->shape, gn - 2);
    const bool acc_da = (c.flags & MNI_B200_ACCUMULATE_DA) != 0;
    const bool acc_db = (c.flags & MNI_B200_ACCUMULATE_DB) != 0;
    const bool acc_dbias = (c.flags & MNI_B200_ACCUMULATE_DBIAS) != 0;
    const int64_t a_elems = s.a_batch * s.M * s.K, b_elems = s.b_batch * s.K * s.N;

    // Which kernel each gradient takes.
    const bool da_wanted = da && a_elems > 0 && s.N > 0 && g_batch > 0;
    const bool db_wanted = db && b_elems > 0 && s.M > 0 && g_batch > 0;
    const bool skinny_dx = da_wanted &&
                           ((c.flags & MNI_B200_FORCE_SKINNY_PATH) != 0 ||
                            ((c.flags & MNI_B200_FORCE_TENSOR_PATH) == 0 && s.M <= kSkinnyDxRows)) &&
                           s.batch == 1 && g_batch == 1 && s.a_batch == 1 && s.b_batch == 1 &&
                           dc->stride[gn - 1] == 1 && b->stride[b->ndim - 1] == 1 && s.K > 1 &&
                           skinny_dx_supported(dc->ptr, dc->stride[gn - 2], b->ptr, b->stride[b->ndim - 2], s.M, s.N);
    const bool skinny_dw = db_wanted &&
                           ((c.flags & MNI_B200_FORCE_SKINNY_PATH) != 0 ||
                            ((c.flags & MNI_B200_FORCE_TENSOR_PATH) == 0 && s.M <= kSkinnyDwRows)) &&
                           s.batch == 1 && g_batch == 1 && s.M <= 16 && (a->stride[a->ndim - 1] == 1 || s.K == 1) &&
                           (dc->stride[gn - 1] == 1 || s.N == 1);

    // grad_a and grad_b do not depend on each other.  grad_b of a small problem goes to the library's side stream
    // next to grad_a and is joined before returning (event fork / join, also valid under stream capture).  The
    // column sums of the bias gradient are HBM-bound and always go to the side stream, where they run beside the
    // tensor-bound products instead of in front of them.
    // MNI_B200_BWD_PAIR=1 selects the one-stream alternative for two tensor-core products: launched back to back
    // as an independent pair (GemmProblem::dep_mode), the second starts on the SMs the first leaves free with no
    // event in between.  Measured, it does not pay: 512^3 30.9 vs 28.8 us per step under graph replay (the second
    // product can only start once every CTA of the first has passed its own dependency wait), 58.9 vs 60.8 us
    // eager, the Linear step 406 vs 405 us -- so it stays off.
    const double work = static_cast<double>(s.M) * static_cast<double>(s.N) * static_cast<double>(s.K) *
                        static_cast<double>(std::max<int64_t>(g_batch, 1));
    // The decisions are the same in the sizing pass and in the real pass (they change the plans, hence the scratch);
    // only the stream operations are skipped while sizing.
    const bool side_on = env_flag("MNI_B200_BWD_OVERLAP", 1);
    const bool pair = side_on && da_wanted && db_wanted && !skinny_dx && !skinny_dw && env_flag("MNI_B200_BWD_PAIR", 0);
    const bool overlap = side_on && !pair && da && db && a_elems > 0 && b_elems > 0 && work > 0 && work <= overlap_work_limit();
    const bool side_dbias = side_on && dbias && (da || db) && work > 0;
    // Two tensor-core products side by side: each persistent grid is planned for half of the SMs, so that both are
    // resident at once instead of the second queueing behind the first's CTAs (measured under graph replay: 512^3
    // 29.2 -> 24.6 us per step, 1024^3 55.3 -> 45.3 us).
    const bool share_sms = overlap && da_wanted && db_wanted && !skinny_dx && !skinny_dw && env_flag("MNI_B200_BWD_SHARE_SMS", 1);
    if (share_sms) c.sm_share = 2;
    cudaStream_t const main_stream = c.stream;
    const bool fork = !c.dry() && (overlap || side_dbias);
    if (fork) {
        MNI_CUDA(cudaEventRecord(c.st->ev_fork, main_stream));
        MNI_CUDA(cudaStreamWaitEvent(c.st->side, c.st->ev_fork, 0));
    }
    struct Join {      // joins the side stream on every exit path once it has been forked
        Call &c; cudaStream_t main; bool on;
        ~Join() {
            c.flag_bank = 0;
            c.dep_mode = 0;
            c.sm_share = 1;
            c.label = "";
            if (!on) return;
            c.stream = main;
            if (cudaEventRecord(c.st->ev_join, c.st->side) == cudaSuccess) cudaStreamWaitEvent(main, c.st->ev_join, 0);
        }
    } join{c, main_stream, fork};

    if (share_sms) c.note("grad_a and grad_b side by side, each planned for half of the SMs");
    else if (overlap) c.note("grad_b on the side stream beside grad_a");
    if (dbias) {
        // Column sums over every row of dc (ops/elementwise.rs:224-229 via utils::unbroadcast).
        c.label = "grad_bias: ";
        if (side_dbias && !c.dry()) c.stream = c.st->side;
        const int64_t rows = g_batch * s.M;
        if (rows == 0 || s.N == 0) {
            rc = zero_or_bias_fill(c, dbias, 1, s.N, nullptr, acc_dbias);
            if (rc) return rc;
        } else {
            mni_b200_view flat = *dc;
            const float *src = dc->ptr;
            int64_t ld = s.N;
            bool contiguous = true;
            {
                int64_t expect = 1;
                for (int d = gn - 1; d >= 0; --d) {
                    if (dc->shape[d] != 1 && dc->stride[d] != expect) contiguous = false;
                    expect *= dc->shape[d];
                }
            }
            if (!contiguous) {
                size_t off;
                rc = pack_view(c, *dc, &flat, &off);
                if (rc) return rc;
                src = flat.ptr;
                ld = flat.stride[1];
            }
            const size_t pbytes = colsum_partial_bytes(rows, s.N, c.st->sm_count);
            const size_t poff = c.arena.reserve(pbytes);
            c.note(side_dbias ? "column sums, on the side stream" : "column sums");
            if (!c.dry()) {
                rc = launch_colsum(src, ld, dbias, rows, s.N, acc_dbias, c.at(poff), c.st->sm_count, c.stream);
                if (rc) return rc;
            }
        }
    }

    c.stream = main_stream;

    // grad_a = unbroadcast(dc . b^T, a.shape)   (ops/matmul.rs:231-240)
    c.label = "grad_a: ";
    if (da && a_elems > 0) {
        if (!da_wanted) {
            rc = zero_or_bias_fill(c, da, a_elems, 1, nullptr, acc_da);
            if (rc) return rc;
        } else if (skinny_dx) {
            c.note("streaming (skinny) input-gradient kernel");
            if (!c.dry()) {
                rc = launch_skinny_dx(dc->ptr, dc->stride[gn - 2], b->ptr, b->stride[b->ndim - 2], da, s.K, acc_da,
                                      s.M, s.N, s.K, c.stream);
                if (rc) return rc;
            }
        } else {
            int64_t ob[MNI_B200_MAX_DIMS];
            const int onb = broadcast_shape(dc->shape, gn - 2, b->shape, b->ndim - 2, ob);
            if (onb < 0) return fail(MNI_B200_ERR_BROADCAST, "dc and b batch shapes are not broadcastable");
            Operand X, Y;
            rc = make_operand(c, *dc, false, X);   // rows M, contraction N
            if (rc) return rc;
            rc = make_operand(c, *b, false, Y);    // rows K, contraction N
            if (rc) return rc;
            X.batch = g_batch;
            Y.batch = s.b_batch;
            c.dep_mode = pair ? 1 : 0;
            rc = grad_gemm(c, X, Y, s.M, s.K, s.N, ob, onb, *a, da, acc_da);
            c.dep_mode = 0;
            if (rc) return rc;
        }
    }

    // grad_b = unbroadcast(a^T . dc, b.shape)   (ops/matmul.rs:242-251)
    if (overlap) { if (!c.dry()) c.stream = c.st->side; c.flag_bank = 1; }
    c.label = "grad_b: ";
    if (db && b_elems > 0) {
        if (!db_wanted) {
            rc = zero_or_bias_fill(c, db, b_elems, 1, nullptr, acc_db);
            if (rc) return rc;
        } else if (skinny_dw) {
            c.note("streaming (skinny) weight-gradient kernel");
            if (!c.dry()) {
                rc = launch_skinny_dw(a->ptr, a->stride[a->ndim - 2], dc->ptr, dc->stride[gn - 2], db, s.N, acc_db,
                                      s.M, s.N, s.K, c.stream);
                if (rc) return rc;
            }
        } else {
            int64_t ob[MNI_B200_MAX_DIMS];
            const int onb = broadcast_shape(a->shape, a->ndim - 2, dc->shape, gn - 2, ob);
            if (onb < 0) return fail(MNI_B200_ERR_BROADCAST, "a and dc batch shapes are not broadcastable");
            Operand X, Y;
            const size_t used_before = c.arena.used;
            rc = make_operand(c, *a, true, X);     // rows K, contraction M
            if (rc) return rc;
            rc = make_operand(c, *dc, true, Y);    // rows N, contraction M
            if (rc) return rc;
            X.batch = s.a_batch;
            Y.batch = g_batch;
            // An operand that had to be gathered first makes this product depend on the gather kernel just
            // launched: then it waits like any other launch.
            if (pair && c.arena.used == used_before) { c.dep_mode = 2; c.flag_bank = 1; }
            rc = grad_gemm(c, X, Y, s.K, s.N, s.M, ob, onb, *b, db, acc_db);
            c.dep_mode = 0;
            if (rc) return rc;
        }
    }
    return MNI_B200_OK;
}

// Runs `body` twice: a dry pass that sizes the scratch, then the real pass.
template <class Body>
int with_scratch(uint32_t flags, void *stream, Body body) {
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(st->mu);
    Call dry;
    dry.st = st; dry.arena.st = st; dry.arena.dry = true; dry.stream = static_cast<cudaStream_t>(stream); dry.flags = flags;
    rc = body(dry);
    if (rc) return rc;
    Call real;
    real.st = st; real.arena.st = st; real.arena.dry = false; real.stream = static_cast<cudaStream_t>(stream); real.flags = flags;
    if (dry.arena.used > 0) {
        rc = scratch_base(*st, dry.arena.used, real.stream, &real.base);
        if (rc) return rc;
    }
    rc = body(real);
    // Both passes must have planned the same launches: a real pass that asked for more scratch than was sized
    // would have written past it.
    if (rc == MNI_B200_OK && real.arena.used > dry.arena.used)
        return fail(MNI_B200_ERR_WORKSPACE, "internal: the call used %zu bytes of scratch, %zu were sized", real.arena.used,
                    dry.arena.used);
    return rc;
}

}  // namespace

int device_sm_count() {
    static std::atomic<int> cache[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    int n = cache[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

bool pdl_enabled() {
    static const bool on = env_flag("MNI_B200_PDL", 1);
    return on;
}

int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    return status;
}

}  // namespace mni

using namespace mni;

extern "C" {

int mni_b200_version(void) { return 100; }

const char *mni_b200_last_error(void) { return t_error; }

uint64_t mni_b200_launch_count(void) { return g_launches.load(); }

int mni_b200_matmul_fwd(const mni_b200_view *a, const mni_b200_view *b, float *c, const float *bias,
                        uint32_t flags, void *stream) {
    Shapes s;   // argument errors are reported before any device is touched
    int rc = analyse(a, b, s);
    if (rc) return rc;
    return with_scratch(flags, stream, [&](Call &call) { return fwd_body(call, a, b, c, bias); });
}

int mni_b200_matmul_bias_gelu_fwd(const mni_b200_view *a, const mni_b200_view *b, const float *bias, float *pre,
                                  float *out, uint32_t flags, void *stream) {
    Shapes s;
    int rc = analyse(a, b, s);
    if (rc) return rc;
    return with_scratch(flags, stream, [&](Call &call) { return fwd_gelu_body(call, a, b, bias, pre, out); });
}

int mni_b200_matmul_bwd(const mni_b200_view *a, const mni_b200_view *b, const mni_b200_view *dc, float *da,
                        float *db, float *dbias, uint32_t flags, void *stream) {
    Shapes s;
    int rc = analyse(a, b, s);
    if (rc) return rc;
    rc = check_view(dc, "dc", 2);
    if (rc) return rc;
    if (dc->shape[dc->ndim - 2] != s.M || dc->shape[dc->ndim - 1] != s.N)
        return fail(MNI_B200_ERR_ARG, "dc is [.., %lld, %lld] but the forward output is [.., %lld, %lld]",
                    (long long)dc->shape[dc->ndim - 2], (long long)dc->shape[dc->ndim - 1], (long long)s.M,
                    (long long)s.N);
    return with_scratch(flags, stream, [&](Call &call) { return bwd_body(call, a, b, dc, da, db, dbias); });
}

int mni_b200_add_bias(const float *y, const float *bias, float *out, int64_t rows, int64_t n, void *stream) {
    if (rows < 0 || n < 0) return fail(MNI_B200_ERR_ARG, "negative extent");
    if (rows * n == 0) return MNI_B200_OK;
    if (!y || !bias || !out) return fail(MNI_B200_ERR_ARG, "null pointer");
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    return launch_add_bias(y, bias, out, rows, n, static_cast<cudaStream_t>(stream));
}

int mni_b200_add_bias_bwd(const float *dy, float *d_y, float *dbias, int64_t rows, int64_t n, uint32_t flags,
                          void *stream) {
    if (rows < 0 || n < 0) return fail(MNI_B200_ERR_ARG, "negative extent");
    if (!dy && rows * n > 0) return fail(MNI_B200_ERR_ARG, "dy is null");
    return with_scratch(flags, stream, [&](Call &c) -> int {
        if (d_y && d_y != dy && !c.dry()) {
            int rc = launch_copy(dy, d_y, rows * n, c.stream);
            if (rc) return rc;
        }
        if (!dbias || n == 0) return MNI_B200_OK;
        const bool acc = (flags & MNI_B200_ACCUMULATE_DBIAS) != 0;
        if (rows == 0) return zero_or_bias_fill(c, dbias, 1, n, nullptr, acc);
        const size_t poff = c.arena.reserve(colsum_partial_bytes(rows, n, c.st->sm_count));
        if (c.dry()) return MNI_B200_OK;
        return launch_colsum(dy, n, dbias, rows, n, acc, c.at(poff), c.st->sm_count, c.stream);
    });
}

int mni_b200_bias_gelu(const float *x, const float *bias, float *out, int64_t rows, int64_t n, void *stream) {
    if (rows < 0 || n < 0) return fail(MNI_B200_ERR_ARG, "negative extent");
    if (rows * n == 0) return MNI_B200_OK;
    if (!x || !bias || !out) return fail(MNI_B200_ERR_ARG, "null pointer");
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    return launch_bias_gelu(x, bias, out, rows, n, static_cast<cudaStream_t>(stream));
}

int mni_b200_bias_gelu_bwd(const float *grad, const float *x, const float *bias, float *dx, float *dbias,
                           int64_t rows, int64_t n, uint32_t flags, void *stream) {
    if (rows < 0 || n < 0) return fail(MNI_B200_ERR_ARG, "negative extent");
    if (rows * n > 0 && (!grad || !x || !bias || !dx)) return fail(MNI_B200_ERR_ARG, "null pointer");
    if (n > 0 && !dbias) return fail(MNI_B200_ERR_ARG, "dbias is null");
    return with_scratch(flags, stream, [&](Call &c) -> int {
        const bool acc = (flags & MNI_B200_ACCUMULATE_DBIAS) != 0;
        if (n == 0) return MNI_B200_OK;
        if (rows == 0) return zero_or_bias_fill(c, dbias, 1, n, nullptr, acc);
        const size_t poff = c.arena.reserve(colsum_partial_bytes(rows, n, c.st->sm_count));
        if (c.dry()) return MNI_B200_OK;
        return launch_bias_gelu_bwd(grad, x, bias, dx, dbias, rows, n, acc, c.at(poff), c.st->sm_count, c.stream);
    });
}

static int softmax_args(const void *p0, const void *p1, const void *p2, int64_t outer, int64_t dim, int64_t inner) {
    if (outer < 0 || dim < 0 || inner < 0) return fail(MNI_B200_ERR_ARG, "negative extent");
    if (outer == 0 || dim == 0 || inner == 0) return MNI_B200_OK;
    if (!p0 || !p1 || !p2) return fail(MNI_B200_ERR_ARG, "null pointer");
    if (outer > 0x7fffffffLL || inner > 0x7fffffffLL || dim > (INT64_MAX / outer) / inner ||
        (inner > 1 && outer * inner / 32 >= 0x7fffffffLL))
        return fail(MNI_B200_ERR_TOO_LARGE, "softmax extent too large");
    return MNI_B200_OK;
}

int mni_b200_softmax_fwd(const float *x, float *out, int64_t outer, int64_t dim_size, int64_t inner, void *stream) {
    int rc = softmax_args(x, out, out, outer, dim_size, inner);
    if (rc || outer * dim_size * inner == 0) return rc;
    DeviceState *st = nullptr;
    rc = device_state(&st);
    if (rc) return rc;
    return launch_softmax_fwd(x, out, outer, dim_size, inner, static_cast<cudaStream_t>(stream));
}

int mni_b200_softmax_bwd(const float *grad, const float *out, float *dx, int64_t outer, int64_t dim_size,
                         int64_t inner, void *stream) {
    int rc = softmax_args(grad, out, dx, outer, dim_size, inner);
    if (rc || outer * dim_size * inner == 0) return rc;
    DeviceState *st = nullptr;
    rc = device_state(&st);
    if (rc) return rc;
    return launch_softmax_bwd(grad, out, dx, outer, dim_size, inner, static_cast<cudaStream_t>(stream));
}

int mni_b200_grad_sumsq(const float *grad, int64_t n, double *sumsq, uint32_t flags, void *stream) {
    if (n < 0) return fail(MNI_B200_ERR_ARG, "negative extent");
    if (!sumsq) return fail(MNI_B200_ERR_ARG, "sumsq is null");
    if (n > 0 && !grad) return fail(MNI_B200_ERR_ARG, "grad is null");
    return with_scratch(flags, stream, [&](Call &c) -> int {
        const size_t poff = c.arena.reserve(sumsq_partial_bytes(n, c.st->sm_count));
        if (c.dry()) return MNI_B200_OK;
        return launch_sumsq(grad, n, sumsq, (flags & MNI_B200_ACCUMULATE_C) != 0, c.at(poff), c.st->sm_count, c.stream);
    });
}

int mni_b200_adamw_step(float *param, float *m, float *v, float *grad, int64_t n, float lr, float beta1, float beta2,
                        float eps, float weight_decay, uint32_t step, const double *grad_sumsq, float max_grad_norm,
                        int write_clipped_grad, void *stream) {
    if (n < 0) return fail(MNI_B200_ERR_ARG, "negative extent");
    if (n == 0) return MNI_B200_OK;
    if (!param || !m || !v || !grad) return fail(MNI_B200_ERR_ARG, "null pointer");
    if (step == 0) return fail(MNI_B200_ERR_ARG, "step counts from 1");
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    // bias corrections of ops/optimizer.rs:26-27: 1 - beta.powi(step) in f32
    const float p1 = powi_f32(beta1, step), p2 = powi_f32(beta2, step);
    return launch_adamw(param, m, v, grad, n, lr, beta1, beta2, eps, weight_decay, 1.0f - p1, 1.0f - p2, grad_sumsq,
                        max_grad_norm, write_clipped_grad != 0, static_cast<cudaStream_t>(stream));
}

int mni_b200_contiguous(const mni_b200_view *src, float *dst, void *stream) {
    int rc = check_view(src, "src", 1);
    if (rc) return rc;
    if (prod(src->shape, src->ndim) == 0) return MNI_B200_OK;
    if (!dst) return fail(MNI_B200_ERR_ARG, "dst is null");
    DeviceState *st = nullptr;
    rc = device_state(&st);
    if (rc) return rc;
    return launch_pack(*src, dst, src->shape[src->ndim - 1], static_cast<cudaStream_t>(stream));
}

int mni_b200_sm_reserve(int sms) {
    if (sms < 0) return fail(MNI_B200_ERR_ARG, "negative SM count");
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(st->mu);
    st->sm_reserve = std::min(sms, std::max(0, st->sm_count - 8));
    return MNI_B200_OK;
}

int mni_b200_workspace_set(void *ptr, size_t bytes) {
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(st->mu);
    if (!ptr || bytes == 0) { st->user_ws = nullptr; st->user_bytes = 0; return MNI_B200_OK; }
    if ((reinterpret_cast<uintptr_t>(ptr) & 255) != 0) return fail(MNI_B200_ERR_ARG, "scratch must be 256-byte aligned");
    st->user_ws = static_cast<uint8_t *>(ptr);
    st->user_bytes = bytes;
    return MNI_B200_OK;
}

int mni_b200_workspace_query(const mni_b200_view *a, const mni_b200_view *b, uint32_t flags, size_t *bytes) {
    if (!bytes) return fail(MNI_B200_ERR_ARG, "bytes is null");
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    Shapes s;
    rc = analyse(a, b, s);
    if (rc) return rc;
    // The forward output's gradient, broadcast batch + [M, N], in the two forms that bound what a real one can
    // need: contiguous and 256-byte aligned (read in place), and a view no descriptor covers (neither matrix
    // dim has unit stride), which is gathered into scratch once for each of its three uses.
    mni_b200_view dc{};
    dc.ptr = reinterpret_cast<const float *>(static_cast<uintptr_t>(256));
    dc.ndim = s.out_nb + 2;
    for (int i = 0; i < s.out_nb; ++i) dc.shape[i] = s.out_batch[i];
    dc.shape[s.out_nb] = s.M; dc.shape[s.out_nb + 1] = s.N;
    int64_t acc = 1;
    for (int d = dc.ndim - 1; d >= 0; --d) { dc.stride[d] = acc; acc *= dc.shape[d]; }
    mni_b200_view dc_strided = dc;
    for (int d = 0; d < dc.ndim; ++d) dc_strided.stride[d] = dc.stride[d] * 2;
    float *fake = reinterpret_cast<float *>(static_cast<uintptr_t>(256));
    size_t need = 0;
    auto dry = [&](auto body) -> int {
        Call c;
        c.st = st; c.arena.dry = true; c.stream = nullptr; c.flags = flags;
        const int r = body(c);
        need = std::max(need, c.arena.used);
        return r;
    };
    rc = dry([&](Call &c) { return fwd_body(c, a, b, fake, nullptr); });
    if (rc) return rc;
    rc = dry([&](Call &c) { return bwd_body(c, a, b, &dc, fake, fake, fake); });
    if (rc) return rc;
    rc = dry([&](Call &c) { return bwd_body(c, a, b, &dc_strided, fake, fake, fake); });
    if (rc) return rc;
    // bias + GELU forward without a `pre` output: when the epilogue cannot be fused the product needs a temporary
    rc = dry([&](Call &c) { return fwd_gelu_body(c, a, b, fake, nullptr, fake); });
    if (rc) return rc;
    // the pointwise entry points on the forward output: column-sum partials, gradient-norm partials
    const int64_t rows = s.batch * s.M;
    need = std::max(need, (colsum_partial_bytes(std::max<int64_t>(rows, 1), std::max<int64_t>(s.N, 1), st->sm_count) + 255) &
                              ~static_cast<size_t>(255));
    const int64_t biggest = std::max({s.a_batch * s.M * s.K, s.b_batch * s.K * s.N, rows * s.N, int64_t{1}});
    need = std::max(need, (sumsq_partial_bytes(biggest, st->sm_count) + 255) & ~static_cast<size_t>(255));
    *bytes = need;
    return MNI_B200_OK;
}

int mni_b200_plan_describe(const mni_b200_view *a, const mni_b200_view *b, int backward, uint32_t flags, int sm_count,
                           char *out, size_t out_len) {
    if (!out || out_len == 0) return fail(MNI_B200_ERR_ARG, "out is null or empty");
    if (sm_count < 8 || sm_count > 4096) return fail(MNI_B200_ERR_ARG, "sm_count %d out of range", sm_count);
    out[0] = 0;
    Shapes s;
    int rc = analyse(a, b, s);
    if (rc) return rc;
    // A stand-in for the device: the plans depend on its SM count only.
    DeviceState st;
    st.sm_count = sm_count;
    std::string log;
    Call c;
    c.st = &st; c.arena.dry = true; c.stream = nullptr; c.flags = flags; c.plan_log = &log;
    float *fake = reinterpret_cast<float *>(static_cast<uintptr_t>(256));
    if (!backward) {
        rc = fwd_body(c, a, b, fake, nullptr);
    } else {
        // the forward output's gradient: contiguous, broadcast batch + [M, N]
        mni_b200_view dc{};
        dc.ptr = fake;
        dc.ndim = s.out_nb + 2;
        for (int i = 0; i < s.out_nb; ++i) dc.shape[i] = s.out_batch[i];
        dc.shape[s.out_nb] = s.M; dc.shape[s.out_nb + 1] = s.N;
        int64_t acc = 1;
        for (int d = dc.ndim - 1; d >= 0; --d) { dc.stride[d] = acc; acc *= dc.shape[d]; }
        rc = bwd_body(c, a, b, &dc, fake, fake, backward > 1 ? fake : nullptr);
    }
    if (rc) return rc;
    if (log.size() + 1 > out_len)
        return fail(MNI_B200_ERR_ARG, "the description needs %zu bytes, %zu given", log.size() + 1, out_len);
    memcpy(out, log.c_str(), log.size() + 1);
    return MNI_B200_OK;
}

int mni_b200_device_status(void *stream, uint32_t *detail) {
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    MNI_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    unsigned int word = 0;
    MNI_CUDA(cudaMemcpy(&word, st->err_word, sizeof(word), cudaMemcpyDeviceToHost));
    if (detail) *detail = word;
    if (word != 0) {
        MNI_CUDA(cudaMemset(st->err_word, 0, sizeof(word)));
        return fail(MNI_B200_ERR_TIMEOUT, "a kernel gave up on a bounded wait (code 0x%x: role %u, slot %u)", word,
                    word >> 8, word & 0xffu);
    }
    return MNI_B200_OK;
}

int mni_b200_role_wait_cycles(uint64_t out[8], int reset) {
    if (!out) return fail(MNI_B200_ERR_ARG, "out is null");
    return read_role_waits(out, reset);
}

int mni_b200_release(void) {
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(st->mu);
    if (st->ws) {
        MNI_CUDA(cudaDeviceSynchronize());
        MNI_CUDA(cudaFree(st->ws));
        st->ws = nullptr;
        st->ws_bytes = 0;
    }
    return MNI_B200_OK;
}

}  // extern "C"
