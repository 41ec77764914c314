/*
 * mni_b200.h -- C ABI of the sm_100a matmul library (libmni_b200.so).
 *
 * The library replaces the `#[cfg(feature = "cuda")]` bodies of the reference's
 * matmul op and of the Linear bias add.  The reference keeps doing what it does
 * today around the call: shape asserts, output allocation (`store.zeros`, whose
 * buffers may hold stale data -- allocator.rs:61-66 -- so every output here is
 * fully overwritten unless an ACCUMULATE flag is given) and `tape.record`.
 *
 * Conventions
 *   - f32 only.  Pointers are device pointers on the CURRENT device; the
 *     reference passes what GpuDevice::ptr / TensorStore::dev_ptr return
 *     (device.rs:205-211, tensor.rs:359-362).
 *   - `mni_b200_view` is what a GpuTensor carries: shape and strides in
 *     ELEMENTS (tensor.rs:63-73).  Stride 0 is allowed on batch dims.
 *   - All work is enqueued on `stream` (a cudaStream_t / CUstream passed as
 *     void*; NULL = the legacy default stream, which is what cudarc's
 *     default_stream() of device.rs:37 resolves to).  No call synchronises the
 *     device except the ones documented to.
 *   - Every function returns an mni_b200_status; mni_b200_last_error() gives the
 *     message of the calling thread's last failure.  Nothing aborts or traps.
 *   - Outputs are contiguous row-major in the logical shape the reference
 *     expects (ops/matmul.rs:145, :211, :218).
 *   - No cuBLAS, no CPU fallback: if the device is not sm_100 the calls fail
 *     with MNI_B200_ERR_DEVICE.
 *   - Threads and streams.  Calls may come from any host thread; state is per
 *     device and guarded by a per-device lock.  The scratch buffer, the finish
 *     tickets of the split-K / streaming kernels and the flags of the balanced
 *     tail are ONE set per device, shared by every stream: two calls whose
 *     kernels can run at the same time on one device (different streams with no
 *     event between them) race on them.  Keep a device's calls on one stream --
 *     what the reference does (device.rs:37) -- or order the streams with events.
 *     The library's own side stream is forked from and joined to the caller's
 *     stream inside one call and never overlaps the next call's kernels.
 */
#ifndef MNI_B200_H
#define MNI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MNI_B200_MAX_DIMS 8

/* Exported symbols (the library is built with hidden default visibility). */
#if defined(__GNUC__)
#define MNI_B200_API __attribute__((visibility("default")))
#else
#define MNI_B200_API
#endif

typedef struct mni_b200_view {
    const float *ptr;
    int32_t ndim;                        /* 1..8 (matmul operands: 2..8)          */
    int64_t shape[MNI_B200_MAX_DIMS];
    int64_t stride[MNI_B200_MAX_DIMS];   /* elements                                */
} mni_b200_view;

typedef enum mni_b200_status {
    MNI_B200_OK = 0,
    MNI_B200_ERR_NDIM = 1,        /* "matmul requires at least 2D tensors" (ops/matmul.rs:89)      */
    MNI_B200_ERR_INNER_DIM = 2,   /* "matmul inner dimensions must match"  (ops/matmul.rs:94)      */
    MNI_B200_ERR_BROADCAST = 3,   /* batch dims not broadcastable (utils.rs:16)                     */
    MNI_B200_ERR_ARG = 4,         /* null pointer, negative size, bad flag, shape mismatch          */
    MNI_B200_ERR_DEVICE = 5,      /* no CUDA device / not compute capability 10.x                   */
    MNI_B200_ERR_CUDA = 6,        /* a CUDA runtime/driver call failed (message has the detail)     */
    MNI_B200_ERR_WORKSPACE = 7,   /* scratch memory could not be grown / caller's is too small      */
    MNI_B200_ERR_TIMEOUT = 8,     /* a bounded device-side wait gave up (see mni_b200_device_status) */
    MNI_B200_ERR_TOO_LARGE = 9    /* a dimension exceeds what the kernels index (2^31-1)            */
} mni_b200_status;

/* flags (OR together) */
#define MNI_B200_PRECISION_3XTF32   0u        /* default: hi/lo split, 3 tensor-core passes, ~f32 accuracy  */
#define MNI_B200_PRECISION_TF32     (1u << 0) /* fast mode: one TF32 pass                                   */
#define MNI_B200_ACCUMULATE_C       (1u << 1) /* fwd: c  += a.b (+bias)   instead of overwrite              */
#define MNI_B200_ACCUMULATE_DA      (1u << 2) /* bwd: da += ...                                             */
#define MNI_B200_ACCUMULATE_DB      (1u << 3) /* bwd: db += ...                                             */
#define MNI_B200_ACCUMULATE_DBIAS   (1u << 4) /* bwd: dbias += ...                                          */
#define MNI_B200_FORCE_TENSOR_PATH  (1u << 8) /* tests: never take the skinny CUDA-core path                */
#define MNI_B200_FORCE_SKINNY_PATH  (1u << 9) /* tests: take the skinny path whenever its kernel can run    */
#define MNI_B200_FORCE_PACK         (1u << 10)/* tests: copy strided operands to scratch first              */
#define MNI_B200_FORCE_SPLIT_K(s)   (((uint32_t)(s) & 0xffu) << 16) /* tests: split the contraction s ways  */

/* Library version: major*10000 + minor*100 + patch. */
MNI_B200_API int mni_b200_version(void);

/* sha256 (hex) of the source files this binary was built from, so that a loader can refuse a stale build.
 * (No counterpart in the reference.) */
MNI_B200_API const char *mni_b200_build_id(void);

/* Message of the calling thread's most recent failing call ("" if none). */
MNI_B200_API const char *mni_b200_last_error(void);

/*
 * Forward.  Replaces the cuBLAS gemm / gemm_strided_batched calls of
 * ops/matmul.rs:145-190 and, for strided operands, the ensure_contiguous
 * round trip of ops/matmul.rs:84-85 / tensor.rs:510-517.
 *
 *   c[batch..., M, N] = a[..., M, K] . b[..., K, N]  (+ bias[N] if bias != NULL)
 *
 * Batch dims broadcast as utils.rs:3-20; an operand whose flat batch count
 * differs from the output's is indexed `batch % operand_batch` exactly as
 * ops/matmul.rs:123-124 does.  `c` is contiguous.  A non-NULL `bias` fuses
 * the Linear bias add (src/nn.ts:23-25) into the epilogue.
 */
MNI_B200_API int mni_b200_matmul_fwd(const mni_b200_view *a, const mni_b200_view *b, float *c,
                        const float *bias, uint32_t flags, void *stream);

/*
 * Forward with the bias + GELU epilogue (the MLP up-projection): one call for what the reference runs
 * as matmul (ops/matmul.rs:83-197) followed by bias_gelu (ops/fused.rs:279-314):
 *   pre[batch..., M, N] = a . b            (written only if pre != NULL; it is what the tape saves)
 *   out[batch..., M, N] = gelu(pre + bias[N])
 * Both outputs leave the GEMM epilogue in the same pass over the accumulator.
 */
MNI_B200_API int mni_b200_matmul_bias_gelu_fwd(const mni_b200_view *a, const mni_b200_view *b, const float *bias,
                                               float *pre, float *out, uint32_t flags, void *stream);

/*
 * Backward.  Replaces ops/matmul.rs:224-255: both transpose_last2 calls
 * (:231, :242), both matmul_no_grad calls (:232, :243) and the device->host
 * unbroadcast round trips (:234-240, :245-251).
 *
 *   da = unbroadcast(dc . b^T, a.shape)      db = unbroadcast(a^T . dc, b.shape)
 *   dbias[N] = column sums of dc             (only if dbias != NULL)
 *
 * `dc` is the gradient of the forward output (shape = broadcast batch + [M,N],
 * any strides).  da / db are contiguous in a's / b's logical shape; either may
 * be NULL to skip it.  Transposes are never materialised; a gradient whose
 * operand was broadcast over the batch is reduced inside the GEMM.
 */
MNI_B200_API int mni_b200_matmul_bwd(const mni_b200_view *a, const mni_b200_view *b, const mni_b200_view *dc,
                        float *da, float *db, float *dbias, uint32_t flags, void *stream);

/*
 * Stand-alone bias add for the drop-in Linear path, where matmul and add are
 * two separate N-API calls.  Replaces the add_bias_f32 launch of
 * ops/elementwise.rs:105-130 (kernels/elementwise.cu:43-47):
 *   out[r, j] = y[r, j] + bias[j],  r < rows, j < n.   out may alias y.
 */
MNI_B200_API int mni_b200_add_bias(const float *y, const float *bias, float *out, int64_t rows, int64_t n,
                      void *stream);

/*
 * Backward of the bias add.  Replaces the device->host->device path of
 * ops/elementwise.rs:224-229: d_y = copy of dy (skipped if d_y is NULL or
 * equals dy), dbias[j] = sum over rows of dy[r, j].
 */
MNI_B200_API int mni_b200_add_bias_bwd(const float *dy, float *d_y, float *dbias, int64_t rows, int64_t n,
                          uint32_t flags, void *stream);

/*
 * Fused bias + GELU (tanh form), the pointwise op that follows the MLP up-projection.  Replaces the
 * bias_gelu_forward_f32 launch of ops/fused.rs:279-314 (kernels/fused_ops.cu:66-82):
 *   out[r, j] = gelu(x[r, j] + bias[j]).
 */
MNI_B200_API int mni_b200_bias_gelu(const float *x, const float *bias, float *out, int64_t rows, int64_t n,
                                    void *stream);

/*
 * Backward of bias + GELU.  Replaces ops/fused.rs:354-392 (kernels/fused_ops.cu:84-110, whose dbias is an
 * atomicAdd in arbitrary order): dx = grad * gelu'(x + bias) and dbias[j] = sum over rows of dx[r, j],
 * summed in a fixed order.  MNI_B200_ACCUMULATE_DBIAS adds into dbias.
 */
MNI_B200_API int mni_b200_bias_gelu_bwd(const float *grad, const float *x, const float *bias, float *dx,
                                        float *dbias, int64_t rows, int64_t n, uint32_t flags, void *stream);

/*
 * Softmax over one dimension of a contiguous tensor seen as [outer, dim_size, inner], and its backward
 * from the saved output.  Replace the softmax_forward_f32 / softmax_backward_f32 launches of
 * ops/norm.rs:52-89 and :125-163 (kernels/softmax.cu); arithmetic as the CPU backend (ops/norm.rs:10-50,
 * :95-123): subtract the maximum, exp, divide by the sum; dx = out * (grad - sum(grad * out)).
 */
MNI_B200_API int mni_b200_softmax_fwd(const float *x, float *out, int64_t outer, int64_t dim_size, int64_t inner,
                                      void *stream);
MNI_B200_API int mni_b200_softmax_bwd(const float *grad, const float *out, float *dx, int64_t outer,
                                      int64_t dim_size, int64_t inner, void *stream);

/*
 * Sum of squares of one gradient in f64, into a device double: the per-parameter term of grad_norm
 * (ops/optimizer.rs:126-171, kernel grad_norm_sq_partial_f32).  With MNI_B200_ACCUMULATE_C the term
 * is added to *sumsq, so a loop over the parameters leaves the squared global norm on the device and
 * no host read sits between the norm and the step.  Fixed grid and summation order: reproducible.
 */
MNI_B200_API int mni_b200_grad_sumsq(const float *grad, int64_t n, double *sumsq, uint32_t flags, void *stream);

/*
 * AdamW step on one parameter, the consumer of the weight gradient.  Replaces the adamw_step_f32 launch
 * of ops/optimizer.rs:67-120 (kernels/adamw.cu): m, v and param are updated in place from grad in one
 * pass; `step` counts from 1 and sets the bias corrections 1 - beta^step.  m and v start as zeros.
 * With grad_sumsq non-null and max_grad_norm > 0 this is clip_and_step (ops/optimizer.rs:247-276):
 * norm = sqrt((float)*grad_sumsq); when norm > max_grad_norm every gradient element is multiplied by
 * max_grad_norm / norm before use, and written back to grad when write_clipped_grad is non-zero (the
 * reference's grad_clip_f32 pass leaves the gradients scaled).
 */
MNI_B200_API int mni_b200_adamw_step(float *param, float *m, float *v, float *grad, int64_t n, float lr, float beta1,
                                     float beta2, float eps, float weight_decay, uint32_t step,
                                     const double *grad_sumsq, float max_grad_norm, int write_clipped_grad,
                                     void *stream);

/*
 * Same result as mni_b200_add_bias_bwd, for callers that must never see this library
 * allocate device memory: a runtime that owns the device's memory budget through its own
 * allocator, or a step loop that cannot take the device-wide stall of cudaMalloc/cudaFree.
 * (No counterpart in the reference: it is an addition of this library.)
 *
 * The partial column sums live in a fixed 1 MiB array inside the library's device image
 * instead of the growable scratch buffer, so this call performs no allocation of any kind.
 *   - Sizes whose partial sums exceed 1 MiB are refused with MNI_B200_ERR_WORKSPACE before
 *     anything is launched (every n <= 262144 fits).
 *   - All calls on a device share that array and it keeps the previous call's contents;
 *     no slot needs to start at zero, each call overwrites what it later reads.
 *   - Calls that overlap on the GPU (other streams / unordered threads) race on the array:
 *     keep them on one stream or order them with events.
 *   - The first call on each device resolves and caches the array's device address; make
 *     that call at start-up, before any stream capture begins on that device.
 */
MNI_B200_API int mni_b200_add_bias_bwd_noalloc(const float *dy, float *d_y, float *dbias, int64_t rows,
                                               int64_t n, uint32_t flags, void *stream);

/*
 * Device-side gather of a strided view into a contiguous row-major buffer.
 * Replaces TensorStore::ensure_contiguous on the CUDA backend
 * (tensor.rs:510-517, a device->host->device round trip in the reference).
 */
MNI_B200_API int mni_b200_contiguous(const mni_b200_view *src, float *dst, void *stream);

/*
 * Scratch memory.  By default the library owns one lazily grown buffer per
 * device.  mni_b200_workspace_set hands it a caller-owned buffer instead
 * (bytes == 0 / ptr == NULL returns to the library-owned one); calls then fail
 * with MNI_B200_ERR_WORKSPACE rather than allocate.  mni_b200_workspace_query
 * returns an upper bound, for operands a and b as given (their strides and
 * alignment count), over: mni_b200_matmul_fwd; mni_b200_matmul_bias_gelu_fwd
 * with or without a `pre` output; mni_b200_matmul_bwd with da, db and dbias and
 * ANY view of the output gradient (contiguous, or strided so that it has to be
 * gathered first); and the pointwise entry points (add_bias_bwd, bias_gelu_bwd,
 * grad_sumsq) applied to tensors no larger than a, b or the forward output.
 * The flags given are the flags the later calls must use.
 *
 * CUDA graphs.  Every call may be recorded by a capturing stream (the side stream
 * is forked and joined with events, which capture follows).  The recorded nodes
 * hold the scratch address of the moment: a library-owned buffer that grows later
 * is freed and leaves such a graph with a dangling address, and it cannot grow
 * during a capture at all (the call then fails with MNI_B200_ERR_WORKSPACE and
 * records nothing).  A caller that replays graphs hands the library a buffer of
 * the queried size with mni_b200_workspace_set and keeps it for the graph's life,
 * or runs each captured call once beforehand and makes no larger call afterwards.
 */
MNI_B200_API int mni_b200_workspace_set(void *ptr, size_t bytes);
MNI_B200_API int mni_b200_workspace_query(const mni_b200_view *a, const mni_b200_view *b, uint32_t flags,
                             size_t *bytes);

/*
 * Leaves `sms` SMs of the current device out of the tensor-core kernels' persistent grids from now on
 * (0 = use every SM again).  For a caller that runs something else beside a matmul call -- a collective
 * that sums the weight gradient over GPUs while the input gradient is computed: the persistent grid is one
 * CTA per SM with all of its shared memory, so a co-running kernel that takes k SMs would otherwise push k
 * CTAs of the grid into a second wave that starts when that kernel ends.  (No counterpart in the reference,
 * which is single-GPU.)
 */
MNI_B200_API int mni_b200_sm_reserve(int sms);

/*
 * Diagnostics: which kernels mni_b200_matmul_fwd (backward = 0) or mni_b200_matmul_bwd with a contiguous
 * output gradient and both gradients (backward = 1; 2 = with the bias gradient too) would launch for
 * these operands and flags on a device with `sm_count` SMs -- one line of text per launch: the product
 * it belongs to, the kernel, and for the tensor-core kernel its tile width, CTA pairing, contraction
 * split, balanced tail, grid and the number of pieces a long contraction is summed in.  Operand
 * pointers are only inspected for alignment.  Pure host arithmetic: touches no device, so the planner
 * can be checked where there is none.  (No counterpart in the reference.)
 */
MNI_B200_API int mni_b200_plan_describe(const mni_b200_view *a, const mni_b200_view *b, int backward,
                                        uint32_t flags, int sm_count, char *out, size_t out_len);

/*
 * Synchronises `stream` and reports whether any kernel of this library gave up
 * on a bounded wait since the last call (MNI_B200_ERR_TIMEOUT, with the
 * recorded role/stage word in *detail if detail != NULL).  Clears the record.
 */
MNI_B200_API int mni_b200_device_status(void *stream, uint32_t *detail);

/*
 * Diagnostics for the tensor-core kernel.  While the environment variable
 * MNI_B200_ROLE_WAITS=1 is set, every launch adds, summed over its CTAs, the clock cycles each
 * warp role spent blocked: out[0] TMA producer waiting for a free stage, out[1] MMA issuer
 * waiting for a free accumulator, out[2] MMA issuer waiting for operands, out[3] split warps
 * waiting for TMA data, out[4] epilogue waiting for a finished accumulator, out[5] total CTA
 * cycles, out[6] CTAs counted.  Synchronises the device.  (No counterpart in the reference.)
 */
MNI_B200_API int mni_b200_role_wait_cycles(uint64_t out[8], int reset);

/* Number of kernels this library has launched in this process (all threads). */
MNI_B200_API uint64_t mni_b200_launch_count(void);

/* Releases the library-owned scratch of the current device (synchronises it). */
MNI_B200_API int mni_b200_release(void);

#ifdef __cplusplus
}
#endif
#endif /* MNI_B200_H */
