/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the matmul hot path.
 *
 * A plain-C restatement of the reference's CPU backend (Rust) for
 * Tensor.matmul forward / backward and the bias add.  It exists so that the
 * CUDA library can be checked against the reference's own arithmetic; nothing
 * in the product path may call it.  The reference itself (Rust + Node N-API)
 * cannot be compiled in this environment, so parity is pinned by
 *   (1) the known-answer cases of the reference's own tests
 *       (test/tensor.test.ts:221-240, test/autograd.test.ts:41-46), and
 *   (2) line-by-line correspondence with the reference source cited on every
 *       function below.
 *
 * Numerics preserved from the reference: f32 accumulator, contraction index
 * ascending, a separate multiply and add per term (the Rust loop
 * `out[..] += a_val * b[..]` is not contracted to an FMA), single pass.  Build
 * with -ffp-contract=off and without -ffast-math (see oracle/Makefile).
 *
 * Every entry point takes `threads`.  threads == 1 is the faithful
 * single-threaded loop nest of the reference (used for the timed CPU
 * baseline).  threads > 1 distributes whole output rows (matmul) or whole
 * destination elements' owners over OpenMP threads; each output element is
 * still produced by exactly the same sequence of f32 operations, so results
 * are bit-identical (tests/test_oracle.py checks this).
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <math.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_MAX_DIMS 8

/* tensor.rs:19-21  shape_size = product of dims, at least 1 */
static int64_t shape_size(const int64_t *shape, int ndim) {
    int64_t n = 1;
    for (int i = 0; i < ndim; ++i) n *= shape[i];
    return n < 1 ? 1 : n;
}

/* tensor.rs:7-17  row-major strides in elements */
static void compute_strides(const int64_t *shape, int ndim, int64_t *strides) {
    if (ndim == 0) return;
    strides[ndim - 1] = 1;
    for (int i = ndim - 2; i >= 0; --i) strides[i] = strides[i + 1] * shape[i + 1];
}

/* utils.rs:3-20  NumPy-style right-aligned broadcast; returns -1 where the
 * reference panics ("shapes ... are not broadcastable"). */
int oracle_broadcast_shape(const int64_t *a, int a_nd, const int64_t *b, int b_nd,
                           int64_t *out) {
    int nd = a_nd > b_nd ? a_nd : b_nd;
    for (int i = 0; i < nd; ++i) {
        int64_t da = i < nd - a_nd ? 1 : a[i - (nd - a_nd)];
        int64_t db = i < nd - b_nd ? 1 : b[i - (nd - b_nd)];
        if (da == db) out[i] = da;
        else if (da == 1) out[i] = db;
        else if (db == 1) out[i] = da;
        else return -1;
    }
    return nd;
}

/* tensor.rs:292-309  make_contiguous_data: gather a strided view into a fresh
 * row-major buffer (flat output index -> coordinates -> source offset). */
void oracle_make_contiguous(const float *data, const int64_t *shape,
                            const int64_t *strides, int ndim, float *out) {
    int64_t size = shape_size(shape, ndim);
    int64_t ostr[ORACLE_MAX_DIMS];
    compute_strides(shape, ndim, ostr);
    for (int64_t i = 0; i < size; ++i) {
        int64_t src = 0, rem = i;
        for (int d = 0; d < ndim; ++d) {
            int64_t c = rem / ostr[d];
            rem %= ostr[d];
            src += c * strides[d];
        }
        out[i] = data[src];
    }
}

/* ops/matmul.rs:45-70  the hot loop, operands already contiguous.
 * a: [a_batch, m, k]  b: [b_batch, k, n]  out: [batch, m, n] (zero-filled here,
 * ops/matmul.rs:48).  Operand batch index = batch % operand batch size (:55-56). */
void oracle_matmul_contig(const float *a, const float *b, float *out,
                          int64_t batch, int64_t a_batch, int64_t b_batch,
                          int64_t m, int64_t k, int64_t n, int threads) {
    const int64_t a_mat = m * k, b_mat = k * n, c_mat = m * n;
    const int64_t rows = batch * m;
    if (threads < 1) threads = 1;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1)
#endif
    for (int64_t r = 0; r < rows; ++r) {
        const int64_t bt = r / m, i = r % m;
        const int64_t ab = a_batch == 1 ? 0 : bt % a_batch;
        const int64_t bb = b_batch == 1 ? 0 : bt % b_batch;
        const float *ap = a + ab * a_mat + i * k;
        const float *bp = b + bb * b_mat;
        float *op = out + bt * c_mat + i * n;
        for (int64_t j = 0; j < n; ++j) op[j] = 0.0f;
        for (int64_t kk = 0; kk < k; ++kk) {
            const float av = ap[kk];
            const float *brow = bp + kk * n;
            for (int64_t j = 0; j < n; ++j) op[j] += av * brow[j];
        }
    }
}

/* ops/matmul.rs:259-284  materialised swap of the last two dims of a
 * contiguous [batch, m, n] tensor. */
void oracle_transpose_last2(const float *data, float *out, int64_t batch,
                            int64_t m, int64_t n, int threads) {
    if (threads < 1) threads = 1;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1)
#endif
    for (int64_t b = 0; b < batch; ++b) {
        const int64_t off = b * m * n;
        for (int64_t i = 0; i < m; ++i)
            for (int64_t j = 0; j < n; ++j) out[off + j * m + i] = data[off + i * n + j];
    }
}

/* utils.rs:39-66  unbroadcast: scan the gradient in ascending flat order and
 * `+=` each element into the clamped coordinate of the original shape.  With
 * threads > 1 each thread owns a disjoint range of destination elements and
 * scans the sources that map to them in the same ascending order, so every
 * destination sees the same sequence of additions. */
void oracle_unbroadcast(const float *grad, const int64_t *gshape, int gnd,
                        const int64_t *oshape, int ond, float *out, int threads) {
    int same = gnd == ond;
    for (int d = 0; same && d < gnd; ++d) same = gshape[d] == oshape[d];
    int64_t gsize = shape_size(gshape, gnd), osize = shape_size(oshape, ond);
    if (same) { memcpy(out, grad, (size_t)gsize * sizeof(float)); return; }
    int64_t gstr[ORACLE_MAX_DIMS], ostr[ORACLE_MAX_DIMS];
    compute_strides(gshape, gnd, gstr);
    compute_strides(oshape, ond, ostr);
    const int off = gnd - ond;
    if (threads < 1) threads = 1;
    memset(out, 0, (size_t)osize * sizeof(float));
    if (threads == 1) {
        for (int64_t i = 0; i < gsize; ++i) {
            int64_t rem = i, oi = 0;
            for (int d = 0; d < gnd; ++d) {
                int64_t c = rem / gstr[d];
                rem %= gstr[d];
                if (d >= off && oshape[d - off] != 1) oi += c * ostr[d - off];
            }
            out[oi] += grad[i];
        }
        return;
    }
#ifdef _OPENMP
#pragma omp parallel num_threads(threads)
    {
        const int t = omp_get_thread_num(), nt = omp_get_num_threads();
        const int64_t lo = osize * t / nt, hi = osize * (t + 1) / nt;
        for (int64_t i = 0; i < gsize; ++i) {
            int64_t rem = i, oi = 0;
            for (int d = 0; d < gnd; ++d) {
                int64_t c = rem / gstr[d];
                rem %= gstr[d];
                if (d >= off && oshape[d - off] != 1) oi += c * ostr[d - off];
            }
            if (oi >= lo && oi < hi) out[oi] += grad[i];
        }
    }
#endif
}

/* ops/matmul.rs:19-78  forward on strided views: ensure_contiguous both
 * operands, broadcast the batch dims, run the loop.  `out` holds
 * prod(broadcast batch) * m * n floats.  Returns 0, -1 (ndim < 2, :25),
 * -2 (inner dims differ, :30), -3 (batch dims not broadcastable, utils.rs:16). */
int oracle_matmul_fwd(const float *a, const int64_t *a_shape, const int64_t *a_strides, int a_nd,
                      const float *b, const int64_t *b_shape, const int64_t *b_strides, int b_nd,
                      float *out, int threads) {
    if (a_nd < 2 || b_nd < 2) return -1;
    const int64_t m = a_shape[a_nd - 2], k = a_shape[a_nd - 1];
    const int64_t k2 = b_shape[b_nd - 2], n = b_shape[b_nd - 1];
    if (k != k2) return -2;
    int64_t ob[ORACLE_MAX_DIMS];
    int ond = oracle_broadcast_shape(a_shape, a_nd - 2, b_shape, b_nd - 2, ob);
    if (ond < 0) return -3;
    const int64_t batch = shape_size(ob, ond);
    const int64_t a_batch = shape_size(a_shape, a_nd - 2), b_batch = shape_size(b_shape, b_nd - 2);
    float *ac = (float *)malloc((size_t)shape_size(a_shape, a_nd) * sizeof(float));
    float *bc = (float *)malloc((size_t)shape_size(b_shape, b_nd) * sizeof(float));
    if (!ac || !bc) { free(ac); free(bc); return -4; }
    oracle_make_contiguous(a, a_shape, a_strides, a_nd, ac);
    oracle_make_contiguous(b, b_shape, b_strides, b_nd, bc);
    oracle_matmul_contig(ac, bc, out, batch, a_batch, b_batch, m, k, n, threads);
    free(ac); free(bc);
    return 0;
}

/* ops/matmul.rs:200-222  backward on strided views:
 *   grad_a = unbroadcast(grad . transpose_last2(b), a.shape)
 *   grad_b = unbroadcast(transpose_last2(a) . grad, b.shape)
 * grad is contiguous in the forward output's shape.  da / db are contiguous in
 * the operands' logical shapes (from_vec, :211 / :218). */
int oracle_matmul_bwd(const float *grad, const int64_t *g_shape, int g_nd,
                      const float *a, const int64_t *a_shape, const int64_t *a_strides, int a_nd,
                      const float *b, const int64_t *b_shape, const int64_t *b_strides, int b_nd,
                      float *da, float *db, int threads) {
    if (a_nd < 2 || b_nd < 2 || g_nd < 2) return -1;
    const int64_t m = a_shape[a_nd - 2], k = a_shape[a_nd - 1], n = b_shape[b_nd - 1];
    if (b_shape[b_nd - 2] != k) return -2;
    const int64_t a_batch = shape_size(a_shape, a_nd - 2), b_batch = shape_size(b_shape, b_nd - 2);
    const int64_t g_batch = shape_size(g_shape, g_nd - 2);
    const int64_t a_size = a_batch * m * k, b_size = b_batch * k * n;
    float *ac = (float *)malloc((size_t)a_size * sizeof(float));
    float *bc = (float *)malloc((size_t)b_size * sizeof(float));
    float *tr = (float *)malloc((size_t)(a_size > b_size ? a_size : b_size) * sizeof(float));
    if (!ac || !bc || !tr) { free(ac); free(bc); free(tr); return -4; }
    oracle_make_contiguous(a, a_shape, a_strides, a_nd, ac);
    oracle_make_contiguous(b, b_shape, b_strides, b_nd, bc);
    int rc = 0;

    /* grad_a: grad [.., m, n] . b_t [.., n, k] */
    {
        oracle_transpose_last2(bc, tr, b_batch, k, n, threads);
        int64_t ob[ORACLE_MAX_DIMS], gs[ORACLE_MAX_DIMS];
        int ond = oracle_broadcast_shape(g_shape, g_nd - 2, b_shape, b_nd - 2, ob);
        if (ond < 0) { rc = -3; goto done; }
        const int64_t batch = shape_size(ob, ond);
        float *ga = (float *)malloc((size_t)(batch * m * k) * sizeof(float));
        if (!ga) { rc = -4; goto done; }
        oracle_matmul_contig(grad, tr, ga, batch, g_batch, b_batch, m, n, k, threads);
        for (int d = 0; d < ond; ++d) gs[d] = ob[d];
        gs[ond] = m; gs[ond + 1] = k;
        oracle_unbroadcast(ga, gs, ond + 2, a_shape, a_nd, da, threads);
        free(ga);
    }
    /* grad_b: a_t [.., k, m] . grad [.., m, n] */
    {
        oracle_transpose_last2(ac, tr, a_batch, m, k, threads);
        int64_t ob[ORACLE_MAX_DIMS], gs[ORACLE_MAX_DIMS];
        int ond = oracle_broadcast_shape(a_shape, a_nd - 2, g_shape, g_nd - 2, ob);
        if (ond < 0) { rc = -3; goto done; }
        const int64_t batch = shape_size(ob, ond);
        float *gb = (float *)malloc((size_t)(batch * k * n) * sizeof(float));
        if (!gb) { rc = -4; goto done; }
        oracle_matmul_contig(tr, grad, gb, batch, a_batch, g_batch, k, m, n, threads);
        for (int d = 0; d < ond; ++d) gs[d] = ob[d];
        gs[ond] = k; gs[ond + 1] = n;
        oracle_unbroadcast(gb, gs, ond + 2, b_shape, b_nd, db, threads);
        free(gb);
    }
done:
    free(ac); free(bc); free(tr);
    return rc;
}

/* ops/elementwise.rs:21-56, :62-73  broadcast add of two contiguous tensors
 * (the Linear bias add is a [.., N] + [N] instance). */
int oracle_add(const float *a, const int64_t *a_shape, int a_nd,
               const float *b, const int64_t *b_shape, int b_nd, float *out) {
    int64_t os[ORACLE_MAX_DIMS], ostr[ORACLE_MAX_DIMS], astr[ORACLE_MAX_DIMS], bstr[ORACLE_MAX_DIMS];
    int nd = oracle_broadcast_shape(a_shape, a_nd, b_shape, b_nd, os);
    if (nd < 0) return -3;
    compute_strides(os, nd, ostr);
    compute_strides(a_shape, a_nd, astr);
    compute_strides(b_shape, b_nd, bstr);
    const int64_t size = shape_size(os, nd);
    const int aoff = nd - a_nd, boff = nd - b_nd;
    for (int64_t i = 0; i < size; ++i) {
        int64_t rem = i, ai = 0, bi = 0;
        for (int d = 0; d < nd; ++d) {
            int64_t c = rem / ostr[d];
            rem %= ostr[d];
            if (d >= aoff && a_shape[d - aoff] != 1) ai += c * astr[d - aoff];
            if (d >= boff && b_shape[d - boff] != 1) bi += c * bstr[d - boff];
        }
        out[i] = a[ai] + b[bi];
    }
    return 0;
}

/* ops/elementwise.rs:199-211  add backward: both input gradients are the
 * output gradient unbroadcast to the input's shape. */
void oracle_add_bwd(const float *grad, const int64_t *g_shape, int g_nd,
                    const int64_t *a_shape, int a_nd, const int64_t *b_shape, int b_nd,
                    float *da, float *db, int threads) {
    oracle_unbroadcast(grad, g_shape, g_nd, a_shape, a_nd, da, threads);
    oracle_unbroadcast(grad, g_shape, g_nd, b_shape, b_nd, db, threads);
}

/* ops/layout.rs:162-195  permute backward: scatter the contiguous gradient of
 * the permuted tensor back into the original layout with the inverse order. */
void oracle_permute_bwd(const float *grad, const int64_t *g_shape, int nd,
                        const int64_t *order, const int64_t *orig_shape, float *out) {
    int64_t inv[ORACLE_MAX_DIMS], sstr[ORACLE_MAX_DIMS], ostr[ORACLE_MAX_DIMS], coord[ORACLE_MAX_DIMS];
    for (int i = 0; i < nd; ++i) inv[order[i]] = i;
    compute_strides(g_shape, nd, sstr);
    compute_strides(orig_shape, nd, ostr);
    const int64_t size = shape_size(g_shape, nd);
    for (int64_t i = 0; i < size; ++i) {
        int64_t rem = i, oi = 0;
        for (int d = 0; d < nd; ++d) { coord[d] = rem / sstr[d]; rem %= sstr[d]; }
        for (int d = 0; d < nd; ++d) oi += coord[inv[d]] * ostr[d];
        out[oi] = grad[i];
    }
}

/* ops/fused.rs:251-277  fused bias + GELU (tanh form), CPU backend: the constant is the Rust
 * literal 0.7978845608_f32, evaluated in f32 exactly as written there. */
void oracle_bias_gelu(const float *x, const float *bias, float *out, int64_t total, int64_t c) {
    for (int64_t i = 0; i < total; ++i) {
        const float val = x[i] + bias[i % c];
        const float inner = 0.7978845608f * (val + 0.044715f * val * val * val);
        out[i] = 0.5f * val * (1.0f + tanhf(inner));
    }
}

/* ops/fused.rs:317-352  backward: dx = grad * gelu'(x + bias); dbias[j] += dx in ascending row order. */
void oracle_bias_gelu_bwd(const float *grad, const float *x, const float *bias, float *dx, float *dbias,
                          int64_t total, int64_t c) {
    for (int64_t j = 0; j < c; ++j) dbias[j] = 0.0f;
    for (int64_t i = 0; i < total; ++i) {
        const int64_t j = i % c;
        const float val = x[i] + bias[j];
        const float inner = 0.7978845608f * (val + 0.044715f * val * val * val);
        const float th = tanhf(inner);
        const float sech2 = 1.0f - th * th;
        const float d_inner = 0.7978845608f * (1.0f + 3.0f * 0.044715f * val * val);
        const float dgelu = 0.5f * (1.0f + th) + 0.5f * val * sech2 * d_inner;
        const float g = grad[i] * dgelu;
        dx[i] = g;
        dbias[j] += g;
    }
}

/* ops/norm.rs:10-50  softmax over dimension d of a row-major tensor seen as [outer, dim, inner]. */
void oracle_softmax(const float *a, float *out, int64_t outer, int64_t dim, int64_t inner) {
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t i = 0; i < inner; ++i) {
            float max_val = -INFINITY;
            for (int64_t s = 0; s < dim; ++s) max_val = fmaxf(max_val, a[o * dim * inner + s * inner + i]);
            float sum = 0.0f;
            for (int64_t s = 0; s < dim; ++s) {
                const int64_t idx = o * dim * inner + s * inner + i;
                const float e = expf(a[idx] - max_val);
                out[idx] = e;
                sum += e;
            }
            for (int64_t s = 0; s < dim; ++s) out[o * dim * inner + s * inner + i] /= sum;
        }
}

/* ops/norm.rs:95-123  softmax backward from the saved output: dot = sum(grad * sm); out = sm * (grad - dot). */
void oracle_softmax_bwd(const float *grad, const float *sm, float *out, int64_t outer, int64_t dim, int64_t inner) {
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t i = 0; i < inner; ++i) {
            float dot = 0.0f;
            for (int64_t s = 0; s < dim; ++s) {
                const int64_t idx = o * dim * inner + s * inner + i;
                dot += grad[idx] * sm[idx];
            }
            for (int64_t s = 0; s < dim; ++s) {
                const int64_t idx = o * dim * inner + s * inner + i;
                out[idx] = sm[idx] * (grad[idx] - dot);
            }
        }
}

/* f32::powi as the reference's build evaluates it (ops/optimizer.rs:26-27): binary exponentiation,
 * lowest exponent bit first, each product rounded to f32. */
float oracle_powi(float x, int n) {
    float r = 1.0f;
    unsigned int e = n < 0 ? 0u - (unsigned int)n : (unsigned int)n;
    for (;;) {
        if (e & 1u) r *= x;
        e >>= 1;
        if (e == 0) break;
        x *= x;
    }
    return n < 0 ? 1.0f / r : r;
}

/* ops/optimizer.rs:22-65  AdamW on one parameter, CPU backend: decoupled decay first (only if
 * weight_decay > 0), then the moment updates and the bias-corrected step.  bc = 1 - beta.powi(step). */
void oracle_adamw_step(float *data, float *m, float *v, const float *grad, int64_t n, float lr, float beta1,
                       float beta2, float eps, float weight_decay, int step) {
    const float bc1 = 1.0f - oracle_powi(beta1, step), bc2 = 1.0f - oracle_powi(beta2, step);
    for (int64_t i = 0; i < n; ++i) {
        const float g = grad[i];
        if (weight_decay > 0.0f) data[i] *= 1.0f - lr * weight_decay;
        m[i] = beta1 * m[i] + (1.0f - beta1) * g;
        v[i] = beta2 * v[i] + (1.0f - beta2) * g * g;
        const float m_hat = m[i] / bc1;
        const float v_hat = v[i] / bc2;
        data[i] -= lr * m_hat / (sqrtf(v_hat) + eps);
    }
}

/* ops/optimizer.rs:126-138  global gradient norm: f64 sum of squares over the gradients in order,
 * rounded to f32, then sqrt. */
float oracle_grad_norm(const float *const *grads, const int64_t *sizes, int count) {
    double norm_sq = 0.0;
    for (int p = 0; p < count; ++p)
        for (int64_t i = 0; i < sizes[p]; ++i) norm_sq += (double)grads[p][i] * (double)grads[p][i];
    return sqrtf((float)norm_sq);
}

/* ops/optimizer.rs:226-245  clip_and_step, CPU backend: norm, in-place scaling of every gradient when
 * max_grad_norm > 0 and norm > max_grad_norm, then AdamW on each parameter; returns the norm. */
float oracle_clip_and_step(float *const *params, float *const *ms, float *const *vs, float *const *grads,
                           const int64_t *sizes, int count, float lr, float beta1, float beta2, float eps,
                           float weight_decay, int step, float max_grad_norm) {
    const float norm = oracle_grad_norm((const float *const *)grads, sizes, count);
    if (max_grad_norm > 0.0f && norm > max_grad_norm) {
        const float scale = max_grad_norm / norm;
        for (int p = 0; p < count; ++p)
            for (int64_t i = 0; i < sizes[p]; ++i) grads[p][i] *= scale;
    }
    for (int p = 0; p < count; ++p)
        oracle_adamw_step(params[p], ms[p], vs[p], grads[p], sizes[p], lr, beta1, beta2, eps, weight_decay, step);
    return norm;
}

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
