// Internal interfaces between the C-ABI host logic (api.cu) and the kernel
// launchers.  Nothing here is exported.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <string>

#include "mni_b200.h"

namespace mni {

// ---------------------------------------------------------------------------
// programmatic dependent launch
// ---------------------------------------------------------------------------
// Short kernels that follow one another in a stream (GEMM -> split-K finish -> GEMM, the three skinny
// products of a step) are launched with programmatic stream serialization: the next grid may be scheduled,
// and run its set-up, while its predecessor still runs; before it touches global memory it executes
// griddepcontrol.wait, which returns once the predecessor has completed and its writes are visible.
// MNI_B200_PDL=0 turns the attribute off (the device-side instructions are then no-ops).
bool pdl_enabled();
#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_trigger() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// ---------------------------------------------------------------------------
// error plumbing
// ---------------------------------------------------------------------------
int fail(int status, const char *fmt, ...);          // records the thread-local message, returns status
int device_sm_count();                                // SM count of the current device (cached per device)
extern std::atomic<uint64_t> g_launches;              // kernels launched by this library

#define MNI_CUDA(call)                                                                   \
    do {                                                                                 \
        cudaError_t e__ = (call);                                                        \
        if (e__ != cudaSuccess)                                                          \
            return ::mni::fail(MNI_B200_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

#define MNI_LAUNCH_CHECK(name)                                                           \
    do {                                                                                 \
        ::mni::g_launches.fetch_add(1, std::memory_order_relaxed);                       \
        cudaError_t e__ = cudaGetLastError();                                            \
        if (e__ != cudaSuccess)                                                          \
            return ::mni::fail(MNI_B200_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)

// ---------------------------------------------------------------------------
// One GEMM operand as the tensor-core kernel reads it through a TMA descriptor.
// "rows" is the operand's non-contraction extent (M for A, N for B), "kdim" the
// contraction extent of one batch.  Exactly one of the two matrix dims has unit
// stride: k_major says which.
// ---------------------------------------------------------------------------
struct Operand {
    const float *ptr = nullptr;
    bool k_major = true;
    int64_t rows = 0, kdim = 0;
    int64_t ld = 0;                // element stride of the non-unit matrix dim
    int64_t bshape[3] = {1, 1, 1}; // operand batch dims, outermost first (front-padded with 1)
    int64_t bstride[3] = {0, 0, 0};
    int64_t batch = 1;             // product of bshape
};

struct GemmProblem {
    Operand A, B;                  // C[M,N] = sum_k A[m,k] * B[n,k]
    int64_t M = 0, N = 0, K = 0;
    int64_t batch = 1;             // output batches
    int64_t fold = 1;              // batches summed inside the contraction (weight-gradient reduce)
    float *C = nullptr;
    int64_t ldc = 0, c_bstride = 0;
    const float *bias = nullptr;   // per output column, may be null
    bool accumulate = false;       // C += ...
    bool fast_tf32 = false;        // one TF32 pass instead of the 3-pass split
    int force_splits = 0;          // tests
    // Two products of one call that do not depend on each other (grad_a and grad_b) are launched back to back on
    // one stream as a pair: the first (1) lets its dependent start only after its own wait for earlier work has
    // returned, the second (2) skips that wait, runs beside the first -- on free SMs, or on the SMs its tail
    // leaves -- and waits for it just before it ends, so stream order holds for everything after the pair.
    int dep_mode = 0;
    int flag_bank = 0;             // 1 for launches on the library's side stream: their own set of balanced-tail flags
    // Optional second output D = gelu(C + bias) written by the same epilogue (C itself is skipped if null).
    float *D = nullptr;
};

// Bytes of split-K partial storage launch_gemm_tc would use for this problem (0 if none).
size_t gemm_tc_partial_bytes(const GemmProblem &p, int sm_count);

// Tensor-core path: TMA -> smem -> (hi/lo split) -> tcgen05.mma -> TMEM -> global.
// `partial` must hold gemm_tc_partial_bytes() bytes when that is non-zero.
int launch_gemm_tc(const GemmProblem &p, float *partial, uint32_t *err_word, int sm_count,
                   cudaStream_t stream);
// One line of text naming the kernel variant, tiling, split and grid launch_gemm_tc would use for this problem
// on a device with `sm_count` SMs.  Pure host arithmetic: touches no device.
std::string gemm_tc_describe(const GemmProblem &p, int sm_count);
// True if the fused second output (GemmProblem::D) can be produced for this problem: no split-K and a
// 16-byte aligned row pitch.  Otherwise the caller runs the GEMM and the pointwise kernel separately.
bool gemm_tc_can_fuse_activation(const GemmProblem &p, int sm_count);

// Diagnostics: copies the 8 role wait counters of the current device (collected only while
// MNI_B200_ROLE_WAITS=1 is set in the environment) and optionally clears them.
int read_role_waits(uint64_t out[8], int reset);

// Skinny path (few output rows, HBM-bound): CUDA-core fp32 FMA kernels.
//   y[M,N] = x[M,K] . W[K,N]          (W row-major, ldw)           M <= 16
int64_t skinny_fwd_row_limit(int64_t N);
bool skinny_fwd_supported(int64_t M, int64_t N, int64_t K);
size_t skinny_fwd_partial_bytes(int64_t M, int64_t N, int64_t K, int sm_count);
int launch_skinny_fwd(const float *x, int64_t ldx, const float *W, int64_t ldw, float *y, int64_t ldy,
                      const float *bias, bool accumulate, int64_t M, int64_t N, int64_t K,
                      float *partial, int sm_count, cudaStream_t stream);
//   dx[M,K] = dy[M,N] . W[K,N]^T                                    M <= 8
bool skinny_dx_supported(const float *dy, int64_t lddy, const float *W, int64_t ldw, int64_t M, int64_t N);
int launch_skinny_dx(const float *dy, int64_t lddy, const float *W, int64_t ldw, float *dx, int64_t lddx,
                     bool accumulate, int64_t M, int64_t N, int64_t K, cudaStream_t stream);
//   dW[K,N] = x[M,K]^T . dy[M,N]                                     M <= 16
int launch_skinny_dw(const float *x, int64_t ldx, const float *dy, int64_t lddy, float *dW, int64_t lddw,
                     bool accumulate, int64_t M, int64_t N, int64_t K, cudaStream_t stream);

// Pointwise / reduction helpers.
int launch_add_bias(const float *y, const float *bias, float *out, int64_t rows, int64_t n,
                    cudaStream_t stream);
size_t colsum_partial_bytes(int64_t rows, int64_t n, int sm_count);
int launch_colsum(const float *dy, int64_t ld, float *out, int64_t rows, int64_t n, bool accumulate,
                  float *partial, int sm_count, cudaStream_t stream);
int launch_copy(const float *src, float *dst, int64_t n, cudaStream_t stream);
int launch_adamw(float *param, float *m, float *v, float *grad, int64_t n, float lr, float beta1, float beta2,
                 float eps, float weight_decay, float bc1, float bc2, const double *sumsq, float max_norm,
                 bool write_grad, cudaStream_t stream);
int launch_softmax_fwd(const float *x, float *out, int64_t outer, int64_t dim, int64_t inner, cudaStream_t stream);
int launch_softmax_bwd(const float *dy, const float *out, float *dx, int64_t outer, int64_t dim, int64_t inner,
                       cudaStream_t stream);
size_t sumsq_partial_bytes(int64_t n, int sm_count);
int launch_sumsq(const float *grad, int64_t n, double *out, bool accumulate, void *partial, int sm_count,
                 cudaStream_t stream);
// out = gelu_tanh(x + bias[col]);  dx = grad * gelu'(x + bias), dbias = column sums of dx (partial: colsum_partial_bytes)
int launch_bias_gelu(const float *x, const float *bias, float *out, int64_t rows, int64_t n, cudaStream_t stream);
int launch_bias_gelu_bwd(const float *grad, const float *x, const float *bias, float *dx, float *dbias,
                         int64_t rows, int64_t n, bool accumulate, float *partial, int sm_count,
                         cudaStream_t stream);
// dst[row-major, ld_dst on the last dim] = gather of a strided view
int launch_pack(const mni_b200_view &src, float *dst, int64_t ld_dst, cudaStream_t stream);
// device-side utils::unbroadcast: out[orig] (+)= sum over broadcast dims of grad[gshape]
int launch_unbroadcast(const float *grad, const int64_t *gshape, int gnd, const int64_t *oshape, int ond,
                       float *out, bool accumulate, cudaStream_t stream);

}  // namespace mni
