/*
 * flashnystrom_b200 -- C ABI of the sm_100a Nystrom-attention library.
 *
 * Every entry point takes plain pointers and sizes; the caller (PyTorch host code through
 * ctypes, or any FFI) owns all memory.  Unless a comment says otherwise a call
 *   - allocates nothing and frees nothing,
 *   - does not synchronise the host with the device,
 *   - enqueues all work on the cudaStream_t it is given (passed as void*),
 *   - keeps no thread-affine state,
 * and returns 0 on success or a negative fnb_status; fnb_last_error() then holds the text.
 *
 * Each declaration names the interface of the reference project (athrva98/FlashNystrom) it
 * stands in for, as file:line inside that project.
 */
#ifndef FLASHNYSTROM_B200_H_
#define FLASHNYSTROM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FNB_ABI_VERSION 2

#if defined(__GNUC__)
#define FNB_API __attribute__((visibility("default")))
#else
#define FNB_API
#endif

enum fnb_status {
  FNB_OK = 0,
  FNB_ERR_INVALID_ARGUMENT = -1, /* a shape / dtype / pointer check failed               */
  FNB_ERR_WORKSPACE = -2,        /* workspace pointer null or smaller than required       */
  FNB_ERR_CUDA = -3,             /* a CUDA runtime call or launch failed                  */
  FNB_ERR_UNSUPPORTED_DEVICE = -4, /* the device is not compute capability 10.x           */
  FNB_ERR_SMEM = -5,             /* "insufficient smem": kernel needs more shared memory  */
  FNB_ERR_DEVICE_STATUS = -6     /* a bounded device-side wait expired (status word set)  */
};

enum fnb_dtype { FNB_F32 = 0, FNB_F16 = 1, FNB_BF16 = 2 };

/* Memory layout of the (B,H,N,D) tensors q, k, v, out, d_out, dq, dk, dv (all eight share it).
 * FNB_LAYOUT_BHND: contiguous (B,H,N,D), what the reference's kernels require
 *   (csrc/flash_nystrom.cu:45-56).
 * FNB_LAYOUT_BNHD: element (b,h,n,d) at ((b*N + n)*H + h)*D + d, i.e. the head-split view of a
 *   contiguous (B,N,H*D) projection output.  The reference's module makes four transposing copies
 *   to get from this to BHND and back (flash_nystrom/flash_nystrom.py:271-292); with this layout
 *   none is needed.  Tensor-core path only (16-bit dtypes, head_dim 64 with num_landmarks <= 64 or
 *   head_dim 128 with num_landmarks <= 128); other shapes are refused with
 *   FNB_ERR_INVALID_ARGUMENT, and so are the sequence-parallel entry points. */
enum fnb_layout { FNB_LAYOUT_BHND = 0, FNB_LAYOUT_BNHD = 1 };

/* flags */
#define FNB_FLAG_FORCE_GENERIC 1u /* use the CUDA-core FP32 kernels even where a tensor-core
                                     kernel exists (verification, like the reference's
                                     FP32 scalar twins csrc/kernels/kernel1_scalar.cuh:18-92) */
#define FNB_FLAG_TEST_DROP_LOAD 0x100u /* tests only: in fnb_forward on the tensor-core path one CTA
                                     of the output pass never issues the copy of its last tile, so
                                     a bounded device-side wait runs out; the call still returns,
                                     `out` is invalid and the status word is set.  No counterpart
                                     in the reference (its kernels have no waits to bound). */

/* Problem description shared by all entry points.
 * Mirrors the scalar fields of NystromParams (csrc/flash_nystrom.h:21-88). */
typedef struct fnb_shape {
  int64_t batch;          /* B                                                    */
  int64_t heads;          /* H                                                    */
  int64_t seq_len;        /* N  (N >= num_landmarks)                              */
  int32_t head_dim;       /* D  (16, 32, 64 or 128)                               */
  int32_t num_landmarks;  /* m  (1..128)                                          */
  int32_t newton_iter;    /* J  (1..20)                                           */
  int32_t dtype;          /* fnb_dtype of q, k, v, out, dO, dQ, dK, dV            */
  float kappa_star;       /* Tikhonov ridge target condition number, 0 = no ridge */
  uint32_t flags;
  int32_t layout;         /* fnb_layout of the eight (B,H,N,D) tensors            */
  int32_t reserved;       /* 0                                                    */
} fnb_shape;

/* Forward.  Replaces nystrom_fwd + run_nystrom_fwd (csrc/flash_nystrom.cu:30-172,
 * csrc/flash_nystrom_kernels.cu:188-251) and the kernels they launch.
 * All tensors are contiguous row-major device memory.  Small saved tensors are FP32. */
typedef struct fnb_fwd_args {
  fnb_shape shape;
  const void* q;        /* (B,H,N,D) dtype, read-only */
  const void* k;        /* (B,H,N,D) dtype, read-only */
  const void* v;        /* (B,H,N,D) dtype, read-only */
  void* out;            /* (B,H,N,D) dtype                                            */
  float* lse1;          /* (B,H,N)   log-sum-exp of softmax(Q Kt^T) rows              */
  float* q_landmarks;   /* (B,H,m,D) D^-1/4-scaled segment means of Q                 */
  float* k_landmarks;   /* (B,H,m,D) same for K                                       */
  float* k2;            /* (B,H,m,m) softmax(Qt Kt^T), without ridge                  */
  float* lse2;          /* (B,H,m)                                                    */
  float* ns_iterates;   /* (B,H,J+1,m,m) Newton-Schulz iterates Z_0..Z_J              */
  float* k2_inv;        /* (B,H,m,m) pseudoinverse used by the output                 */
  float* bmat;          /* (B,H,m,D) softmax(Qt K^T) V                                */
  float* lse3;          /* (B,H,m)                                                    */
  float* step2;         /* (B,H,m,D) k2_inv * bmat                                    */
  void* workspace;      /* >= fnb_fwd_workspace_bytes(), 256-byte aligned             */
  size_t workspace_bytes;
  int32_t device;       /* CUDA device ordinal all pointers live on                   */
  void* stream;         /* cudaStream_t                                               */
  int32_t* device_status; /* optional device word, zeroed by the caller.  The first kernel that
                             meets one of these conditions stores (code<<24 | location):
                               1  a bounded device-side wait ran out (results invalid; the
                                  kernel released its resources and returned)
                               2  the kernel's shared-memory window was not 1024-byte aligned
                               3  fp16 only: a non-finite softmax-Jacobian value met the range
                                  rescaling of the backward column pass (inf / NaN in the
                                  inputs or in dO; the values go through as they are)
                             The library never synchronises, so it cannot return
                             FNB_ERR_DEVICE_STATUS itself: the host reads the word after the
                             stream has drained (the Python shim's check_device_status). */
} fnb_fwd_args;

/* Backward.  Replaces nystrom_bwd + run_nystrom_bwd_impl (csrc/flash_nystrom.cu:177-415,
 * csrc/flash_nystrom_kernels.cu:313-391), including the cuBLAS + CUDA-graph
 * Newton-Schulz backward (csrc/kernels/backward/kernel2_inv_bwd.cu:794-1058).
 * dq, dk, dv need not be zeroed and must not alias any input.  dv is written once; on the
 * tensor-core path (16-bit dtypes, head_dim 64, num_landmarks <= 64) dq and dk first hold the
 * 16-bit softmax-Jacobian tiles of their rows and are turned into the gradients in place by the
 * last kernel of the call, so their contents are defined only when the call's work on `stream`
 * has completed.  Kernels of one call may also run on a library-owned side stream, forked from
 * and joined back into `stream` with events (capturable into a CUDA graph). */
typedef struct fnb_bwd_args {
  fnb_shape shape;
  const void* q;
  const void* k;
  const void* v;
  const void* d_out;    /* (B,H,N,D) dtype */
  const float* lse1;
  const float* q_landmarks;
  const float* k_landmarks;
  const float* k2;
  const float* ns_iterates;
  const float* k2_inv;
  const float* bmat;
  const float* lse3;
  const float* step2;
  void* dq;             /* (B,H,N,D) dtype */
  void* dk;
  void* dv;
  void* workspace;      /* >= fnb_bwd_workspace_bytes(), 256-byte aligned */
  size_t workspace_bytes;
  int32_t device;
  void* stream;
  int32_t* device_status; /* as in fnb_fwd_args */
} fnb_bwd_args;

typedef struct fnb_caps {
  int32_t abi_version;
  int32_t cc_major, cc_minor;
  int32_t sm_count;
  int32_t max_smem_per_block;  /* opt-in bytes */
  int64_t l2_bytes;
  int64_t total_mem_bytes;
} fnb_caps;

/* Text of the last failure on the calling thread (thread-local, never NULL).
 * Stands in for the std::runtime_error text of csrc/utils.h:23-61. */
FNB_API const char* fnb_last_error(void);

/* Library ABI version (FNB_ABI_VERSION).  No counterpart in the reference. */
FNB_API int fnb_version(void);

/* Device properties; FNB_ERR_UNSUPPORTED_DEVICE unless the device is sm_100.
 * Stands in for query_sm_limits (csrc/flash_nystrom.cu:693-726). */
FNB_API int fnb_capabilities(int device, fnb_caps* caps);

/* Scratch sizes in bytes for one call of the given shape.  The reference allocates its
 * scratch itself (csrc/flash_nystrom.cu:292-333, kernel3_output_fused.cuh:1033-1047). */
FNB_API size_t fnb_fwd_workspace_bytes(const fnb_shape* shape);
FNB_API size_t fnb_bwd_workspace_bytes(const fnb_shape* shape);

/* Validate a shape exactly as fnb_forward would (csrc/flash_nystrom.cu:45-79). */
FNB_API int fnb_check_shape(const fnb_shape* shape);

FNB_API int fnb_forward(const fnb_fwd_args* args);
FNB_API int fnb_backward(const fnb_bwd_args* args);

/* ---- sequence parallelism (no counterpart in the reference) -------------------------------
 * The sequence of every (b,h) slice is cut into `world` equal contiguous shards, one per rank;
 * shape.seq_len is the LOCAL length, seq_len_global = world * seq_len.  Requirements:
 * num_landmarks % world == 0 and seq_len_global % num_landmarks == 0, so every landmark
 * segment lives on one rank.  A forward or backward is three calls (stage 0, 1, 2) with the
 * same arguments and workspace; between stages the caller runs one collective on `xfer`
 * (FP32, device memory):
 *   forward  after stage 0: all-reduce(sum) of xfer[0 .. 2*BH*m*D)
 *            after stage 1: all-gather of this rank's BH*m*(D+2) floats into world * that many,
 *                           rank-major, passed as xfer of stage 2
 *   backward after stage 0: all-reduce(sum) of xfer[0 .. 2*BH*m*D)
 *            after stage 1: all-reduce(sum) of xfer[0 .. BH*m*D)
 * Saved tensors are replicated (identical on every rank) except lse1, which is per local row.
 * The collectives carry m x D tiles per slice: they are latency-bound, not bandwidth-bound. */
typedef struct fnb_sp_info {
  int32_t rank, world, stage;
  int64_t seq_len_global;
  float* xfer;
  size_t xfer_floats;    /* capacity of xfer, checked against fnb_sp_xfer_floats */
} fnb_sp_info;
/* Floats needed in xfer for (is_backward, stage); stage 2 of the forward wants world x stage 1. */
FNB_API size_t fnb_sp_xfer_floats(const fnb_shape* shape, int world, int is_backward, int stage);
FNB_API int fnb_sp_forward(const fnb_fwd_args* args, const fnb_sp_info* sp);
FNB_API int fnb_sp_backward(const fnb_bwd_args* args, const fnb_sp_info* sp);

/* Isolation hooks for the Newton-Schulz kernels; (BH,m,m) FP32 device tensors.
 * Stand in for debug_kernel2_inv_bwd_full / debug_ns_bwd_* (csrc/flash_nystrom.cu:629-690).
 *
 * fnb_debug_pinv_forward: k2 (already a softmax matrix) -> ns_iterates, k2_inv.
 * fnb_debug_pinv_backward: (k2, ns_iterates, d_k2_inv) -> d_k2  (gradient w.r.t. the
 *   softmax matrix, before the softmax Jacobian). */
FNB_API int fnb_debug_pinv_forward(int64_t bh, int32_t m, int32_t newton_iter, float kappa_star,
                           const float* k2, float* ns_iterates, float* k2_inv,
                           void* workspace, size_t workspace_bytes, int32_t device,
                           void* stream);
FNB_API int fnb_debug_pinv_backward(int64_t bh, int32_t m, int32_t newton_iter, float kappa_star,
                            const float* k2, const float* ns_iterates, const float* d_k2_inv,
                            float* d_k2, void* workspace, size_t workspace_bytes,
                            int32_t device, void* stream);
FNB_API size_t fnb_debug_pinv_workspace_bytes(int64_t bh, int32_t m);

/* One backward iteration of the Newton-Schulz unroll, run by the product's tensor-core kernel
 * (num_landmarks <= 64, no ridge): from K2, the iterate Z_j and dL/dZ_{j+1} to dL/dZ_j and this
 * iteration's contribution to dL/dK2.  (BH,m,m) FP32 device tensors.
 * Stands in for debug_ns_bwd_step (csrc/flash_nystrom.cu:422-456). */
FNB_API int fnb_debug_ns_bwd_step(int64_t bh, int32_t m, const float* k2, const float* z_j, const float* d_z_next,
                                  float* d_z_out, float* d_k2_acc, int32_t device, void* stream);

/* The tail of the backward in isolation (num_landmarks <= 64, no ridge): dL/dZ_0 and the dL/dK2
 * accumulated over the iterations -> complete dL/dK2 (d_k2_out), then through the softmax-2
 * Jacobian to dQt = dS2 Kt and dKt = dS2^T Qt.  zeros_md: (m, D) floats of zeros.
 * Stands in for debug_ns_bwd_final (csrc/flash_nystrom.cu:474-520). */
FNB_API int fnb_debug_ns_bwd_final(int64_t bh, int32_t m, int32_t head_dim, const float* q_landmarks,
                                   const float* k_landmarks, const float* k2, const float* d_z0, const float* d_k2_in,
                                   const float* zeros_md, float* d_q_landmarks, float* d_k_landmarks, float* d_k2_out,
                                   int32_t device, void* stream);

/* Resources and occupancy of the hot-path kernels on `device`: registers per thread, static and
 * dynamic shared memory, local (spill) bytes per thread, threads per CTA and how many CTAs fit on
 * one SM.  Writes up to `cap` entries, returns how many.  Stands in for probe_occupancy
 * (csrc/occupancy_probe.h:89-142). */
typedef struct fnb_kernel_info {
  char name[48];
  int32_t registers, static_smem_bytes, dynamic_smem_bytes, local_bytes_per_thread, threads, blocks_per_sm;
} fnb_kernel_info;
FNB_API int fnb_kernel_report(int device, fnb_kernel_info* out, int cap);

/* Gradient of the pseudoinverse for callers that must not allocate: what
 * fnb_debug_pinv_backward computes, but without a workspace argument.  It always runs the FP32
 * CUDA-core kernel (fnb_debug_pinv_backward prefers the tensor-core kernel for num_landmarks
 * <= 64), so the two agree to FP32 rounding, not bit for bit; without the ridge the row of
 * ||K2||_inf is decided by round-off (row sums of a softmax matrix tie at 1), so compare them
 * after the softmax Jacobian, which removes that row-constant term.  It has no counterpart in the
 * reference.  It is meant for hosts whose device memory is handed out once at start-up and
 * then frozen - a plugin inside a serving process with a fixed memory plan, say - where a
 * cudaMalloc in the request path is forbidden (it may fail, and it stalls the device).  The
 * scratch the kernel needs (one m x m FP32 block per slice, used with the ridge) lives in a
 * 1 MiB array compiled into the library; every GPU that loads the library carries it until the
 * process exits.  Limits: at most 64 slices per call and num_landmarks <= 64; larger requests
 * are refused with FNB_ERR_INVALID_ARGUMENT.  The call allocates and frees nothing.  The first
 * call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call before any stream capture begins.  All calls share the one
 * array and it keeps whatever the last call left in it (nothing needs clearing: every block is
 * written before it is read); two calls whose kernels overlap on the GPU - different streams -
 * would race on it, so keep them ordered. */
FNB_API int fnb_pinv_backward_noalloc(int64_t bh, int32_t m, int32_t newton_iter, float kappa_star,
                                      const float* k2, const float* ns_iterates, const float* d_k2_inv,
                                      float* d_k2, int32_t device, void* stream);

/* ---- depthwise convolution residual of the attention module ----------------------------------
 * Replaces _depthwise_conv_residual (flash_nystrom/flash_nystrom.py:19-55: two transposing copies
 * around a grouped F.conv1d) together with the addition to the attention output that follows the
 * kernel call in flash_nystrom_attention, and what autograd derives from them.  Every head has one
 * 1-D kernel of odd length kernel_size (<= 127), shared by its head_dim channels; zero padding of
 * kernel_size / 2 rows on either side of the sequence:
 *     result[b,h,n,:] = base[b,h,n,:] + sum_j weight[h][j] * v[b,h,n + j - kernel_size/2,:]
 * with transposed != 0 the taps are reversed (the operator the backward applies to dOut to get the
 * contribution to dV).  v, base (may be NULL: nothing is added) and result are (B,H,N,D) tensors of
 * `dtype` in `layout`, 16-byte aligned; result must not alias v (it may alias base).  weight is FP32
 * [heads][kernel_size] on the device.  head_dim in {16, 32, 64, 128}.  One kernel on `stream`, no
 * synchronisation, no allocation. */
typedef struct fnb_conv_args {
  int64_t batch, heads, seq_len;
  int32_t head_dim, kernel_size, dtype, layout;
  const void* v;
  const void* base;
  void* result;
  const float* weight;
  int32_t transposed;
  int32_t device;
  void* stream;
} fnb_conv_args;
FNB_API int fnb_conv_residual(const fnb_conv_args* args);

/* Gradient of the convolution residual with respect to the weights:
 *     d_weight[h][j] = sum over b, n, d of d_out[b,h,n,d] * v[b,h,n + j - kernel_size/2,d]
 * (FP32, summed in a fixed order: two calls give identical bits).  workspace: device memory of at
 * least fnb_conv_dweight_workspace_bytes(...) bytes, 16-byte aligned.  Two kernels on `stream`. */
typedef struct fnb_conv_dw_args {
  int64_t batch, heads, seq_len;
  int32_t head_dim, kernel_size, dtype, layout;
  const void* v;
  const void* d_out;
  float* d_weight;
  void* workspace;
  size_t workspace_bytes;
  int32_t device;
  void* stream;
} fnb_conv_dw_args;
FNB_API size_t fnb_conv_dweight_workspace_bytes(int64_t batch, int64_t heads, int64_t seq_len, int32_t kernel_size);
FNB_API int fnb_conv_residual_dweight(const fnb_conv_dw_args* args);

/* Tests only: the time limit of every bounded device-side wait on `device` (default 1500 ms),
 * so that a test of the expiry path does not take seconds.  1..10000 ms.  No counterpart in the
 * reference. */
FNB_API int fnb_debug_set_wait_limit_ms(int device, int ms);

/* Per-kernel timing.  Off unless the environment variable FNB_PROFILE=1 was set when the
 * library was loaded or fnb_set_profiling(1) was called (process-wide switch; returns the
 * previous mode).  While on, fnb_forward / fnb_backward bracket every kernel with CUDA events on
 * the caller's stream; the call itself still does not synchronise.  fnb_last_profile() waits for
 * the events of the most recent call made on this thread and writes up to `cap` entries.
 * Stands in for KernelProfiler (csrc/profile.h:44-106). */
typedef struct fnb_kernel_time { char name[48]; float ms; } fnb_kernel_time;
FNB_API int fnb_set_profiling(int mode);
FNB_API int fnb_last_profile(fnb_kernel_time* out, int cap);

#ifdef __cplusplus
}
#endif
#endif /* FLASHNYSTROM_B200_H_ */
