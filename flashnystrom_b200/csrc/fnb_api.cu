// C ABI of flashnystrom_b200: argument validation, workspace carving and the ordered kernel
// launches of the forward and backward passes.  See include/flashnystrom_b200.h for the
// contract of every entry point.
#include "../../include/flashnystrom_b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <vector>
#include <map>
#include <mutex>
#include <utility>
#include <string>

#include "common.cuh"
#include "mid_kernels.cuh"
#include "generic_kernels.cuh"
#include "tc_host.cuh"
#include "ns_kernels.cuh"
#include "ns_tc_kernels.cuh"
#include "conv_kernels.cuh"
#include <type_traits>
#include <algorithm>

namespace fnb {

// Scratch of fnb_pinv_backward_noalloc: one (64 x 64) FP32 matrix per slice for up to 64 slices
// (1 MiB), resident in every device that loads this library until the process exits.
constexpr int kNoAllocMaxSlices = 64;
constexpr int kNoAllocMaxM = 64;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocMaxSlices * kNoAllocMaxM * kNoAllocMaxM];

static thread_local char g_err[512] = "";
static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define FNB_CUDA(expr)                                                                     \
  do {                                                                                     \
    cudaError_t e_ = (expr);                                                               \
    if (e_ != cudaSuccess)                                                                 \
      return fail(FNB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_),    \
                  __FILE__, __LINE__);                                                     \
  } while (0)

// ---- optional per-kernel profiler -----------------------------------------------------------
// Off by default.  FNB_PROFILE=1 in the environment at load, or fnb_set_profiling(1), brackets
// every kernel with a pair of CUDA events on the caller's stream (no host synchronisation in the
// call itself); fnb_last_profile() waits for the last event and reads the times back.
static int g_profile = [] {
  const char* e = getenv("FNB_PROFILE");
  return (e && e[0] == '1') ? 1 : 0;
}();
struct ProfState {
  int device = -1;
  std::vector<cudaEvent_t> pool;      // reused across calls on this thread
  std::vector<std::string> names;     // kernels of the most recent call
  size_t used = 0;
  cudaEvent_t get(int dev) {
    if (dev != device) {
      for (cudaEvent_t e : pool) cudaEventDestroy(e);
      pool.clear();
      device = dev;
      used = 0;
    }
    if (used == pool.size()) {
      cudaEvent_t e = nullptr;
      cudaEventCreate(&e);
      pool.push_back(e);
    }
    return pool[used++];
  }
};
static thread_local ProfState g_prof;

struct Launcher {
  cudaStream_t stream;
  int device;
  bool prof;
  int status = 0;
  Launcher(cudaStream_t s, int dev) : stream(s), device(dev), prof(g_profile != 0) {
    if (prof) {
      g_prof.names.clear();
      g_prof.used = 0;
    }
  }
  void begin() {
    if (prof) cudaEventRecord(g_prof.get(device), stream);
  }
  int end(const char* name) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
      cudaGetLastError();
      return status = fail(FNB_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e));
    }
    if (prof) {
      cudaEventRecord(g_prof.get(device), stream);
      g_prof.names.push_back(name);
    }
    return 0;
  }
};

// Side stream for work that can run beside the caller's stream inside one call.  One side stream
// and two events per host thread and device, created on first use and kept for the life of the
// thread; fork/join are event record + wait pairs, so a caller capturing its stream into a CUDA
// graph captures the fork as well.
struct SideStream {
  int device = -1;
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  bool get(int dev) {
    if (dev == device && stream) return true;
    if (stream) { cudaStreamDestroy(stream); cudaEventDestroy(fork); cudaEventDestroy(join); stream = nullptr; }
    if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) { stream = nullptr; return false; }
    cudaEventCreateWithFlags(&fork, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&join, cudaEventDisableTiming);
    device = dev;
    return true;
  }
};
static thread_local SideStream g_side;

struct Fork {
  cudaStream_t main;
  bool enabled, forked = false, ended = false;
  Fork(cudaStream_t st, int dev, bool want) : main(st), enabled(want && g_side.get(dev)) {}
  cudaStream_t begin() {            // work launched on the returned stream runs beside `main`
    if (!enabled) return main;
    cudaEventRecord(g_side.fork, main);
    cudaStreamWaitEvent(g_side.stream, g_side.fork, 0);
    forked = true;
    return g_side.stream;
  }
  void end() { if (forked && !ended) { cudaEventRecord(g_side.join, g_side.stream); ended = true; } }
  void join() {                     // `main` waits for the side work
    if (forked) {
      end();                        // an early error return never reached end(): close the fork now
      cudaStreamWaitEvent(main, g_side.join, 0);
      forked = false;
    }
  }
  ~Fork() { join(); }
};

// The two function attributes below are per kernel and device and stay until the context ends:
// they are set once (again only if a later call needs more), not on every launch.
static std::mutex g_smem_mutex;
static std::map<std::pair<const void*, int>, size_t> g_smem_set;

// Raises a kernel's opt-in dynamic shared memory size to `bytes` (never lowers it: the largest size asked
// for so far is remembered per kernel and device, and launches that need less skip the call).
static cudaError_t raise_smem(const void* kernel, size_t bytes) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) device = -1;
  const std::pair<const void*, int> key(kernel, device);
  if (device >= 0) {
    std::lock_guard<std::mutex> lock(g_smem_mutex);
    auto it = g_smem_set.find(key);
    if (it != g_smem_set.end() && it->second >= bytes) return cudaSuccess;
  }
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  // ask for the largest shared-memory carveout so that co-residency is limited by the kernel's
  // own footprint, not by the driver's default split between L1 and shared memory
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e == cudaSuccess && device >= 0) {
    std::lock_guard<std::mutex> lock(g_smem_mutex);
    size_t& cur = g_smem_set[key];
    if (cur < bytes) cur = bytes;
  }
  return e;
}

template <class K>
static int set_smem(K kernel, size_t bytes, int max_optin, const char* name) {
  if ((long long)bytes > (long long)max_optin)
    return fail(FNB_ERR_SMEM, "insufficient smem for %s: needs %zu bytes, device allows %d", name,
                bytes, max_optin);
  cudaError_t e = raise_smem(reinterpret_cast<const void*>(kernel), bytes);
  if (e != cudaSuccess)
    return fail(FNB_ERR_CUDA, "cudaFuncSetAttribute(%s, %zu) failed: %s", name, bytes,
                cudaGetErrorString(e));
  return 0;
}

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    // Always (re)select: besides switching devices this binds the device's primary context to
    // the calling thread, which the driver-level tensor-map encoder needs (an autograd worker
    // thread may not have touched the runtime yet).
    if (cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
  }
};

static int device_limits(int device, int* max_smem, int* cc_major, int* sm_count) {
  // attribute queries are cheap and keep the call free of cached, thread-affine state
  FNB_CUDA(cudaDeviceGetAttribute(max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  FNB_CUDA(cudaDeviceGetAttribute(cc_major, cudaDevAttrComputeCapabilityMajor, device));
  FNB_CUDA(cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, device));
  if (*cc_major != 10)
    return fail(FNB_ERR_UNSUPPORTED_DEVICE,
                "device %d has compute capability %d.x; this library is built for sm_100a only",
                device, *cc_major);
  return 0;
}

static int check_shape(const fnb_shape* s) {
  if (!s) return fail(FNB_ERR_INVALID_ARGUMENT, "shape is NULL");
  if (s->batch <= 0 || s->heads <= 0)
    return fail(FNB_ERR_INVALID_ARGUMENT, "batch_size and num_heads must be positive (got B=%lld, H=%lld)",
                (long long)s->batch, (long long)s->heads);
  if (s->dtype != FNB_F32 && s->dtype != FNB_F16 && s->dtype != FNB_BF16)
    return fail(FNB_ERR_INVALID_ARGUMENT, "Supported dtypes: float32, float16, bfloat16 (got code %d)", s->dtype);
  if (s->num_landmarks < 1 || s->num_landmarks > kMaxM)
    return fail(FNB_ERR_INVALID_ARGUMENT, "num_landmarks must be in [1, %d], got %d", kMaxM, s->num_landmarks);
  if (s->seq_len < s->num_landmarks)
    return fail(FNB_ERR_INVALID_ARGUMENT, "seq_len (%lld) must be >= num_landmarks (%d)",
                (long long)s->seq_len, s->num_landmarks);
  if (!(s->head_dim == 16 || s->head_dim == 32 || s->head_dim == 64 || s->head_dim == 128))
    return fail(FNB_ERR_INVALID_ARGUMENT, "head_dim must be 16, 32, 64 or 128, got %d", s->head_dim);
  if (s->newton_iter < 1 || s->newton_iter > 20)
    return fail(FNB_ERR_INVALID_ARGUMENT, "newton_iter must be in [1, 20], got %d", s->newton_iter);
  if (!std::isfinite(s->kappa_star) || s->kappa_star < 0.f)
    return fail(FNB_ERR_INVALID_ARGUMENT,
                "kappa_star must be finite and >= 0 (got %g); 0 disables the Tikhonov ridge",
                (double)s->kappa_star);
  if (s->layout != FNB_LAYOUT_BHND && s->layout != FNB_LAYOUT_BNHD)
    return fail(FNB_ERR_INVALID_ARGUMENT, "layout must be FNB_LAYOUT_BHND (0) or FNB_LAYOUT_BNHD (1), got %d", s->layout);
  if (s->batch * s->heads > (int64_t)1 << 24)
    return fail(FNB_ERR_INVALID_ARGUMENT, "batch * heads (%lld) exceeds 2^24", (long long)(s->batch * s->heads));
  return 0;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct FwdWs {
  float *land_partial, *part_acc, *part_max, *part_sum, *pinv;
  void *qt16, *kt16, *st16;   // 16-bit operand copies for the tensor-core kernels
  float* st_scale;            // [BH] power-of-two normalisation of the step2 copy
  size_t bytes;
};
static FwdWs carve_fwd(const Plan& p, void* base) {
  char* b = (char*)base;
  size_t off = 0;
  auto take = [&](size_t nfloat) { float* r = (float*)(b + off); off += align256(nfloat * sizeof(float)); return r; };
  FwdWs w;
  w.land_partial = take((size_t)2 * p.BH * p.m * p.lm_chunks * p.D);
  w.part_acc = take((size_t)p.BH * p.nchunk * p.m * p.D);
  w.part_max = take((size_t)p.BH * p.nchunk * p.m);
  w.part_sum = take((size_t)p.BH * p.nchunk * p.m);
  w.pinv = take((size_t)p.BH * kPinvFwdBufs * p.m * p.m);
  const int MP = p.m <= 64 ? 64 : 128;
  const size_t op16 = ((size_t)p.BH * MP * p.D + 1) / 2;   // 16-bit elements, counted in floats
  w.qt16 = take(op16); w.kt16 = take(op16); w.st16 = take(op16);
  w.st_scale = take((size_t)p.BH);
  w.bytes = off;
  return w;
}

struct BwdWs {
  float *partA, *partB, *dstep2, *dkt_a, *dO3, *dqt_ns, *dkt_tot, *dqt_tot, *D3, *G, *dK2, *pinv;
  void* op16[8];              // 16-bit operand copies for the tensor-core kernels
  float *st_scale, *do3_scale, *rows_q, *rows_k;
  float* partA_red;           // [BH][2][m][D]: pass-A partials summed over the chunks
  float* tile_scale;          // [BH][ceil(N / 128)]: factor the column pass stored each dS' tile with
  size_t bytes;
};
static BwdWs carve_bwd(const Plan& p, void* base) {
  char* b = (char*)base;
  size_t off = 0;
  auto take = [&](size_t nfloat) { float* r = (float*)(b + off); off += align256(nfloat * sizeof(float)); return r; };
  BwdWs w;
  const size_t md = (size_t)p.BH * p.m * p.D, mm = (size_t)p.BH * p.m * p.m;
  w.partA = take((size_t)p.nchunk * 2 * md);
  w.partB = take((size_t)p.nchunk * md);
  w.dstep2 = take(md); w.dkt_a = take(md); w.dO3 = take(md);
  w.dqt_ns = take(md); w.dkt_tot = take(md); w.dqt_tot = take(md);
  w.D3 = take((size_t)p.BH * p.m);
  w.G = take(mm); w.dK2 = take(mm);
  w.pinv = take((size_t)kPinvBwdBufs * mm);
  const int MP = p.m <= 64 ? 64 : 128;
  const size_t op16 = ((size_t)p.BH * MP * p.D + 1) / 2;
  for (int i = 0; i < 8; ++i) w.op16[i] = take(op16);
  w.st_scale = take((size_t)p.BH); w.do3_scale = take((size_t)p.BH);
  w.rows_q = take(md); w.rows_k = take(md);
  w.partA_red = take(2 * md);
  w.tile_scale = take((size_t)p.BH * (size_t)((p.N + 127) / 128));
  w.bytes = off;
  return w;
}

static Plan plan_of(const fnb_shape& s) {
  return make_plan(s.batch * s.heads, s.seq_len, s.head_dim, s.num_landmarks, s.newton_iter);
}

// Sequence-parallel context.  stage < 0: ordinary single-device call.  Otherwise the call runs one
// stage of the sharded pipeline (the collectives between stages belong to the caller):
//   forward  0: local segment sums -> xfer [2][BH][m][D]                     (all-reduce, sum)
//            1: landmarks, pseudoinverse, column pass, local merge -> xfer    (all-gather)
//               [BH*m*D acc | BH*m max | BH*m sum]
//            2: merge of the gathered partials (xfer = world x that), step2, output pass
//   backward 0: row pass partials, local sum -> xfer [BH][2][m][D]            (all-reduce, sum)
//            1: middle (from xfer), pseudoinverse backward, column pass, local dQt sum
//               -> xfer [BH][m][D]                                            (all-reduce, sum)
//            2: dQ pass (dQt_tot = Newton-Schulz part + xfer)
struct SpCtx {
  int stage = -1, rank = 0, world = 1;
  int64_t N_global = 0;
  float* xfer = nullptr;
  bool on() const { return stage >= 0; }
  bool run(int k) const { return stage < 0 || stage == k; }
};

// ------------------------------------------------------------------------------------------
// Forward: pooling pass -> landmarks -> [pseudoinverse | softmax-3 column pass] -> combine ->
// output row pass.
// Launch with programmatic stream serialization: the kernel may be scheduled while its
// predecessor in the stream is still running (every kernel launched this way calls pdl_wait()
// before it touches global memory that other kernels of the stream produce or consume).
template <class... KArgs, class... Args>
static cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// Launch as thread-block clusters of `cs` CTAs along x (grid.x = number of clusters * cs).
template <class... KArgs, class... Args>
static cudaError_t launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, int cs,
                                  Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)cs; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = cs > 1 ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// CTAs per slice of the landmark-sized kernels for more than 64 landmarks when their products run on
// the tensor cores (a thread-block cluster shares every product by output columns): eight if the
// device can hold a cluster of eight for every slice at once (each CTA takes an SM to itself, and
// a cluster must fit into one GPC), else four.  FNB_MID_CLUSTER in the environment at load fixes the
// size (1, 2, 4 or 8; kept for A/B measurements).
template <class... KArgs>
static int mid_cluster_size(void (*kern)(KArgs...), int64_t slices, int device) {
  static const int forced = [] {
    const char* e = getenv("FNB_MID_CLUSTER");
    const int v = e ? atoi(e) : 0;
    return (v == 1 || v == 2 || v == 4 || v == 8) ? v : 0;
  }();
  if (forced) return forced;
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, int> fit8;   // (kernel, device) -> clusters of eight that fit at once
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_pair((const void*)kern, device);
  auto it = fit8.find(key);
  if (it == fit8.end()) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(8 * 64); cfg.blockDim = dim3(kMidTcThreads); cfg.dynamicSmemBytes = kTcGemmSmem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 8; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { n = 0; cudaGetLastError(); }
    it = fit8.emplace(key, n).first;
  }
  return slices <= it->second ? 8 : 4;
}

// The Newton-Schulz kernels for num_landmarks <= 64 run on the tensor cores (three-term bf16
// split, FP32-equivalent) unless the caller forces the CUDA-core path or FNB_NS_CUDA_CORES=1 is
// set in the environment (kept for A/B measurements).
static bool ns_on_tensor_cores(uint32_t flags) {
  static const bool env_off = [] {
    const char* e = getenv("FNB_NS_CUDA_CORES");
    return e && e[0] == '1';
  }();
  return !env_off && !(flags & FNB_FLAG_FORCE_GENERIC);
}

// How the streaming passes hand data to one another through the L2 cache (bit mask; FNB_L2 in
// the environment at load overrides the default, kept for A/B measurements):
//   1  tile order: the output pass, the first backward row pass and the backward column pass walk
//      their tiles strided, and a pass that re-reads what its predecessor touched walks backwards
//   2  evict-first hints on everything that is read or written for the last time
//   4  the in-place pass finishes dK (whose parked tiles the column pass has just written) before dQ
//  16  evict-last hints on what the next pass of the chain reads back
//  32  the forward column pass walks its tiles strided too
// Measured on a B200 at B=1, H=16, N=65536 (ms per forward + backward): 0: 0.543, 7: 0.524,
// 23: 0.526, 31: 0.530 (the in-place pass 102 -> 93 us, the first row pass 86 -> 83 us).
constexpr int kL2Default = 7;
static int l2_mode() {
  static const int mode = [] {
    const char* e = getenv("FNB_L2");
    return e ? atoi(e) : kL2Default;
  }();
  return mode;
}
static int hint_bits(int in0, int in1, int out0, int out1) { return in0 | (in1 << 2) | (out0 << 4) | (out1 << 6); }

// Calls f(std::integral_constant<int, D>) for the head dimensions the tensor-core kernels are
// instantiated for.
template <class F>
static int dispatch_head_dim(int D, F&& f) {
  if (D == 64) return f(std::integral_constant<int, 64>{});
  return f(std::integral_constant<int, 128>{});
}
// Calls f(D, MP as integral constants) for the (head_dim, padded landmark count) pairs the
// tensor-core kernels are instantiated for: (64, 64), (128, 64), (128, 128).
template <class F>
static int dispatch_tc(int D, int MP, F&& f) {
  if (D == 64) return f(std::integral_constant<int, 64>{}, std::integral_constant<int, 64>{});
  if (MP == 64) return f(std::integral_constant<int, 128>{}, std::integral_constant<int, 64>{});
  return f(std::integral_constant<int, 128>{}, std::integral_constant<int, 128>{});
}
// Co-resident tensor-core CTAs per SM: two for head_dim 64, one for head_dim 128 (shared memory).
static int tc_ctas_per_sm(int D) { return D == 64 ? 2 : 1; }

template <class T>
static int forward_impl(const fnb_fwd_args& a, const Plan& p, const FwdWs& w, int max_smem, int sms,
                        cudaStream_t st, bool allow_inner_fork, const SpCtx& S = SpCtx()) {
  Launcher L(st, a.device);
  const float scale = powf((float)p.D, -0.25f);
  constexpr bool k16 = !std::is_same<T, float>::value;
  tc::TcSched sch = tc::make_sched(p.BH, p.N, tc_ctas_per_sm(p.D) * sms);   // one wave
  const bool use_tc = k16 && tc::tc_supported(a.shape.dtype, p.D, p.m, a.shape.flags) && sch.nchunk <= p.nchunk;
  const tc::BigLayout big{a.shape.batch, a.shape.heads, p.N, p.D, a.shape.layout};
  if (a.shape.layout != FNB_LAYOUT_BHND && !use_tc)
    return fail(FNB_ERR_INVALID_ARGUMENT, "the (B,N,H,D) layout needs the tensor-core path (16-bit dtype, head_dim 64 with "
                "num_landmarks <= 64 or head_dim 128 with num_landmarks <= 128)");
  const int MP = p.m <= 64 ? 64 : 128;
  const bool smem_ns = p.m <= ns::kN;
  const int64_t seg_N = S.on() ? S.N_global : p.N, row_offset = S.on() ? (int64_t)S.rank * p.N : 0;
  sch.seg_N = seg_N; sch.row_offset = row_offset; sch.H = big.map_h();
  const int lmC = S.on() ? 1 : p.lm_chunks;
  float* land = S.on() ? S.xfer : w.land_partial;
  const int l2 = l2_mode();
  const int ef = (l2 & 2) ? 1 : 0, el = (l2 & 16) ? 2 : 0;
  tc::TcSched sch_fb = sch, sch_fc = sch;
  sch_fb.order = (l2 & 32) ? tc::kOrderStrided : 0;
  sch_fb.hint = hint_bits(ef, ef, 0, 0);                 // K (left in L2 by the pooling pass) and V die here
  sch_fc.order = (l2 & 1) ? tc::kOrderStrided : 0;
  sch_fc.hint = hint_bits(el, 0, ef, 0);                 // Q is read again by the backward; O is not
  sch_fc.test_drop = (a.shape.flags & FNB_FLAG_TEST_DROP_LOAD) ? 1 : 0;
  const int nchunk_b = use_tc ? sch.nchunk : p.nchunk;
  const size_t md_all = (size_t)p.BH * p.m * p.D, m_all = (size_t)p.BH * p.m;

  if (S.run(0)) {
    {
      L.begin();
      int64_t grid = std::min<int64_t>(2 * p.BH * p.m * lmC, (int64_t)sms * 4);
      auto pool = (a.shape.layout == FNB_LAYOUT_BNHD) ? landmark_partial_kernel<T, false> : landmark_partial_kernel<T, true>;
      launch_pdl(pool, dim3((unsigned)grid), dim3(kThreads), 0, st,
          (const T*)a.q, (const T*)a.k, land, p.BH, p.N, p.D, p.m, lmC, seg_N, row_offset, big.map_h(), big.row_stride(),
          big.head_stride(), big.batch_stride());
      if (L.end("landmark_partial")) return L.status;
    }
  }
  if (S.stage == 0) return 0;

  StreamParams sp;
  memset(&sp, 0, sizeof(sp));
  sp.q = a.q; sp.k = a.k; sp.v = a.v; sp.out = a.out; sp.lse1 = a.lse1;
  sp.qt = a.q_landmarks; sp.kt = a.k_landmarks; sp.step2 = a.step2;
  sp.part_acc = w.part_acc; sp.part_max = w.part_max; sp.part_sum = w.part_sum;
  sp.N = p.N; sp.rows_per_chunk = p.rows_per_chunk; sp.D = p.D; sp.m = p.m; sp.mpad = p.mpad;
  sp.nchunk = p.nchunk; sp.scale = scale; sp.seg_N = seg_N; sp.row_offset = row_offset;
  const unsigned sgrid = (unsigned)(p.BH * p.nchunk);
  auto combine_kern = p.D == 16 ? combine2_kernel<1> : p.D == 32 ? combine2_kernel<2> : p.D == 64 ? combine2_kernel<4>
                                                                                                : combine2_kernel<8>;

  if (S.run(1)) {
  Fork fork(st, a.device, smem_ns && !L.prof && allow_inner_fork);   // side stream for the pseudoinverse (off while profiling)
  // With the tensor-core kernels the landmarks are formed from the raw segment sums inside their
  // two consumers (the Newton-Schulz forward writes the FP32 copies, the column pass packs its own
  // 16-bit operand), so the finalize kernel is skipped.
  const bool fused_landmarks = smem_ns && use_tc && p.D == 64 && ns_on_tensor_cores(a.shape.flags);
  if (smem_ns) {
    if (!fused_landmarks) {
    L.begin();
    {
      LandmarkFinalizeParams lp;
      lp.land_partial = land; lp.C = lmC; lp.qt = a.q_landmarks; lp.kt = a.k_landmarks;
      lp.BH = p.BH; lp.N = seg_N; lp.m = p.m; lp.D = p.D; lp.scale = scale;
      lp.qt16 = use_tc ? w.qt16 : nullptr; lp.dtype = a.shape.dtype; lp.MP = MP; lp.qt16_mul = scale * tc::kLog2e;
      landmark_finalize_kernel<<<dim3((unsigned)p.BH, 16), kThreads, 0, st>>>(lp);
    }
    if (L.end("landmark_finalize")) return L.status;
    }
    // The pseudoinverse only feeds the combine step, so it runs beside the column pass.
    cudaStream_t ns_stream = fork.begin();
    L.begin();
    ns::NsFwdParams np;
    np.qt = a.q_landmarks; np.kt = a.k_landmarks; np.k2 = a.k2; np.lse2 = a.lse2;
    np.iterates = a.ns_iterates; np.k2inv = a.k2_inv; np.m = p.m; np.D = p.D; np.J = p.J;
    np.kappa = a.shape.kappa_star;
    np.land = fused_landmarks ? land : nullptr; np.C = lmC; np.BH = p.BH; np.seg_N = seg_N; np.scale = scale;
    np.qt_out = a.q_landmarks; np.kt_out = a.k_landmarks;
    if (ns_on_tensor_cores(a.shape.flags)) {
      if (int rc = set_smem(nstc::ns_fwd_tc_kernel, nstc::kFwdSmem, max_smem, "ns_fwd")) return rc;
      nstc::ns_fwd_tc_kernel<<<(unsigned)p.BH, nstc::kNsTcThreads, nstc::kFwdSmem, ns_stream>>>(np, a.device_status);
    } else {
      if (int rc = set_smem(ns::ns_fwd_kernel, ns::kFwdSmem, max_smem, "ns_fwd")) return rc;
      ns::ns_fwd_kernel<<<(unsigned)p.BH, kThreads, ns::kFwdSmem, ns_stream>>>(np);
    }
    if (L.end("ns_fwd")) return L.status;
    fork.end();
  } else {
    L.begin();
    MidFwdParams mp;
    mp.land_partial = land; mp.C = lmC;
    mp.qt = a.q_landmarks; mp.kt = a.k_landmarks; mp.k2 = a.k2; mp.lse2 = a.lse2;
    mp.iterates = a.ns_iterates; mp.k2inv = a.k2_inv; mp.scratch = w.pinv;
    mp.BH = p.BH; mp.N = seg_N; mp.m = p.m; mp.D = p.D; mp.J = p.J;
    mp.kappa = a.shape.kappa_star; mp.scale = scale;
    mp.landmarks_only = 0;
    mp.qt16 = use_tc ? w.qt16 : nullptr; mp.dtype = a.shape.dtype; mp.MP = MP;
    mp.qt16_mul = scale * tc::kLog2e;
    // products on the tensor cores unless the caller forces the CUDA-core path
    mp.use_tc = (a.shape.flags & FNB_FLAG_FORCE_GENERIC) ? 0 : 1;
    mp.status = a.device_status;
    const size_t mid_smem = mp.use_tc ? kTcGemmSmem : 0;
    if (mp.use_tc)
      if (int rc = set_smem(mid_fwd_kernel, mid_smem, max_smem, "mid_fwd")) return rc;
    if (mp.use_tc) {
      const int cs = mid_cluster_size(mid_fwd_kernel, p.BH, a.device);
      FNB_CUDA(launch_cluster(mid_fwd_kernel, dim3((unsigned)(p.BH * cs)), dim3(kMidTcThreads), mid_smem, st, cs, mp));
    } else {
      mid_fwd_kernel<<<(unsigned)p.BH, kThreads, mid_smem, st>>>(mp);
    }
    if (L.end("mid_fwd")) return L.status;
  }

  if constexpr (k16) {
    if (use_tc) {
      int rc = dispatch_tc(p.D, MP, [&](auto dtag, auto mtag) -> int {
        constexpr int D = decltype(dtag)::value, MPc = decltype(mtag)::value;
        CUtensorMap tm_k, tm_v, tm_qt;
        if (!tc::make_map_big(&tm_k, a.k, a.shape.dtype, big, tc::kTile) ||
            !tc::make_map_big(&tm_v, a.v, a.shape.dtype, big, tc::kTile) ||
            !tc::make_map_2d(&tm_qt, w.qt16, a.shape.dtype, p.BH * MPc, D, MPc))
          return fail(FNB_ERR_CUDA, "cuTensorMapEncodeTiled failed for the forward column pass");
        L.begin();
        auto kern = tc::tc_fwd_b_kernel<T, D, MPc>;
        size_t smem = tc::FwdBSmem<D, MPc>::kBytes;
        if (int rc2 = set_smem(kern, smem, max_smem, "tc_fwd_b")) return rc2;
        launch_pdl(kern, dim3((unsigned)(p.BH * sch.nchunk)), dim3(tc::kTcThreads), smem, st,
            tm_k, tm_v, tm_qt, fused_landmarks ? land : (const float*)nullptr, lmC, p.BH, scale, w.part_acc, w.part_max,
            w.part_sum, sch_fb, p.m, a.device_status);
        return L.end("tc_fwd_b");
      });
      if (rc) return rc;
    }
  }
  if (!use_tc) {
    L.begin();
    size_t smem = fwd_b_smem(p.mpad, p.D);
    if (int rc = set_smem(gen_fwd_b_kernel<T>, smem, max_smem, "gen_fwd_b")) return rc;
    gen_fwd_b_kernel<T><<<sgrid, kThreads, smem, st>>>(sp);
    if (L.end("gen_fwd_b")) return L.status;
  }

  fork.join();
  if (S.on()) {
    // merge this rank's per-CTA partials into one un-normalised partial for the all-gather
    L.begin();
    Combine2Params cp;
    memset(&cp, 0, sizeof(cp));
    cp.part_acc = w.part_acc; cp.part_max = w.part_max; cp.part_sum = w.part_sum; cp.nchunk = nchunk_b;
    cp.m = p.m; cp.D = p.D;
    cp.acc_bh_stride = (int64_t)nchunk_b * p.m * p.D; cp.acc_chunk_stride = (int64_t)p.m * p.D;
    cp.vec_bh_stride = (int64_t)nchunk_b * p.m; cp.vec_chunk_stride = p.m;
    cp.partial_only = 1; cp.out_acc = S.xfer; cp.out_max = S.xfer + md_all; cp.out_sum = S.xfer + md_all + m_all;
    if (int rc = set_smem(combine_kern, 16, max_smem, "combine_local")) return rc;
    combine_kern<<<(unsigned)p.BH, kThreads, 16, st>>>(cp);
    if (L.end("combine_local")) return L.status;
  }
  }  // stage 1
  if (S.stage == 1) return 0;

  L.begin();
  {
    Combine2Params cp;
    memset(&cp, 0, sizeof(cp));
    if (S.on()) {
      // gathered layout: world x [BH*m*D acc | BH*m max | BH*m sum]
      const int64_t per_rank = (int64_t)(md_all + 2 * m_all);
      cp.part_acc = S.xfer; cp.part_max = S.xfer + md_all; cp.part_sum = S.xfer + md_all + m_all;
      cp.nchunk = S.world;
      cp.acc_bh_stride = (int64_t)p.m * p.D; cp.acc_chunk_stride = per_rank;
      cp.vec_bh_stride = p.m; cp.vec_chunk_stride = per_rank;
    } else {
      cp.part_acc = w.part_acc; cp.part_max = w.part_max; cp.part_sum = w.part_sum; cp.nchunk = nchunk_b;
      cp.acc_bh_stride = (int64_t)nchunk_b * p.m * p.D; cp.acc_chunk_stride = (int64_t)p.m * p.D;
      cp.vec_bh_stride = (int64_t)nchunk_b * p.m; cp.vec_chunk_stride = p.m;
    }
    if (use_tc && p.D % 16 == 0) {
      // the tensor-core output pass packs its own operand copies: merge + step2 only, spread over
      // D / 16 CTAs per slice
      CombineSlabParams sp2;
      sp2.part_acc = cp.part_acc; sp2.part_max = cp.part_max; sp2.part_sum = cp.part_sum; sp2.nchunk = cp.nchunk;
      sp2.acc_bh_stride = cp.acc_bh_stride; sp2.acc_chunk_stride = cp.acc_chunk_stride;
      sp2.vec_bh_stride = cp.vec_bh_stride; sp2.vec_chunk_stride = cp.vec_chunk_stride;
      sp2.k2inv = a.k2_inv; sp2.bmat = a.bmat; sp2.lse3 = a.lse3; sp2.step2 = a.step2; sp2.m = p.m; sp2.D = p.D;
      const size_t csm = combine_slab_smem(p.m);
      if (int rc = set_smem(combine_slab_kernel, csm, max_smem, "combine")) return rc;
      launch_pdl(combine_slab_kernel, dim3((unsigned)p.BH, (unsigned)(p.D / 16)), dim3(kThreads), csm, st, sp2);
    } else {
      cp.k2inv = a.k2_inv; cp.k_landmarks = a.k_landmarks; cp.bmat = a.bmat; cp.lse3 = a.lse3;
      cp.step2 = a.step2; cp.m = p.m; cp.D = p.D;
      cp.dtype = 0; cp.MP = MP; cp.kt16 = w.kt16; cp.st16T = w.st16;
      cp.st_scale = w.st_scale; cp.kt_mul = scale * tc::kLog2e;
      size_t smem = sizeof(float) * (size_t)p.m * p.D;
      if (int rc = set_smem(combine_kern, smem, max_smem, "combine")) return rc;
      combine_kern<<<(unsigned)p.BH, kThreads, smem, st>>>(cp);
    }
  }
  if (L.end("combine")) return L.status;

  if constexpr (k16) {
    if (use_tc) {
      return dispatch_tc(p.D, MP, [&](auto dtag, auto mtag) -> int {
        constexpr int D = decltype(dtag)::value, MPc = decltype(mtag)::value;
        CUtensorMap tm_q, tm_o;
        if (!tc::make_map_big(&tm_q, a.q, a.shape.dtype, big, tc::kTile) ||
            !tc::make_map_big(&tm_o, a.out, a.shape.dtype, big, tc::kTile))
          return fail(FNB_ERR_CUDA, "cuTensorMapEncodeTiled failed for the forward output pass");
        L.begin();
        auto kern = tc::tc_fwd_c_kernel<T, D, MPc>;
        size_t smem = tc::FwdCSmem<D, MPc>::kBytes;
        if (int rc2 = set_smem(kern, smem, max_smem, "tc_fwd_c")) return rc2;
        launch_pdl(kern, dim3((unsigned)(p.BH * sch.nchunk)), dim3(tc::kTcThreads), smem, st, tm_q, tm_o, a.k_landmarks,
                   a.step2, a.lse1, sch_fc, p.m, scale, a.device_status);
        return L.end("tc_fwd_c");
      });
    }
  }
  L.begin();
  {
    size_t smem = fwd_c_smem(p.mpad, p.D);
    if (int rc = set_smem(gen_fwd_c_kernel<T>, smem, max_smem, "gen_fwd_c")) return rc;
    gen_fwd_c_kernel<T><<<sgrid, kThreads, smem, st>>>(sp);
  }
  if (L.end("gen_fwd_c")) return L.status;
  return 0;
}

// ------------------------------------------------------------------------------------------
// Backward: softmax-1 row pass (partials) -> landmark-sized middle (dO3, dK2inv, pseudoinverse
// backward) -> softmax-3 column pass (dK, dV, dQt partials) -> dQ row pass.
template <class T>
static int backward_impl(const fnb_bwd_args& a, const Plan& p, const BwdWs& w, int max_smem, int sms,
                         cudaStream_t st, bool allow_inner_fork, const SpCtx& S = SpCtx()) {
  Launcher L(st, a.device);
  const float scale = powf((float)p.D, -0.25f);
  constexpr bool k16 = !std::is_same<T, float>::value;
  tc::TcSched sch = tc::make_sched(p.BH, p.N, tc_ctas_per_sm(p.D) * sms);   // one wave
  const int64_t seg_N = S.on() ? S.N_global : p.N, row_offset = S.on() ? (int64_t)S.rank * p.N : 0;
  const tc::BigLayout big{a.shape.batch, a.shape.heads, p.N, p.D, a.shape.layout};
  sch.seg_N = seg_N; sch.row_offset = row_offset; sch.H = big.map_h();
  const bool use_tc = k16 && tc::tc_supported(a.shape.dtype, p.D, p.m, a.shape.flags) && sch.nchunk <= p.nchunk;
  if (a.shape.layout != FNB_LAYOUT_BHND && !use_tc)
    return fail(FNB_ERR_INVALID_ARGUMENT, "the (B,N,H,D) layout needs the tensor-core path (16-bit dtype, head_dim 64 with "
                "num_landmarks <= 64 or head_dim 128 with num_landmarks <= 128)");
  const int MP = p.m <= 64 ? 64 : 128;
  const bool smem_ns = p.m <= ns::kN;
  // With head_dim 64 on the tensor-core path the reduction of the pass-A partials and the two
  // products that follow run inside the Newton-Schulz backward kernel.
  const bool fused_mid = smem_ns && use_tc && p.D == 64 && p.J >= 1 && ns_on_tensor_cores(a.shape.flags);
  // The column pass does not need the pseudoinverse backward (it leaves dS3' tiles for the in-place
  // pass, which is the first consumer of the landmark gradients), so the two run side by side:
  // the Newton-Schulz kernel on a side stream with one SM per slice, the column pass on the rest.
  // Off while profiling (kernels are timed one by one).
  const bool side_ns = fused_mid && !L.prof && allow_inner_fork && p.BH * 4 <= sms;
  tc::TcSched sch_b = sch;
  if (side_ns) {
    sch_b = tc::make_sched(p.BH, p.N, 2 * (sms - (int)p.BH));
    sch_b.seg_N = seg_N; sch_b.row_offset = row_offset; sch_b.H = big.map_h();
  }
  int kshift = 0;
  while ((int64_t(2) << kshift) <= seg_N && kshift < 14) ++kshift;   // floor(log2 N), at most 14
  if (a.shape.dtype == FNB_BF16) kshift = 0;   // bf16 has the FP32 exponent range: no shift, nothing to clamp
  const int l2 = l2_mode();
  const int ef = (l2 & 2) ? 1 : 0, el = (l2 & 16) ? 2 : 0;
  const int strided = (l2 & 1) ? tc::kOrderStrided : 0;
  tc::TcSched sch_a = sch, sch_c = sch;
  sch_a.order = strided ? (strided | tc::kOrderDescending) : 0;   // starts on the end of Q the output pass left in L2
  sch_a.hint = hint_bits(ef, ef, el, 0);                          // Q, dO die here; the parked dS1 tiles are read back
  sch_b.order = strided;
  sch_b.hint = hint_bits(ef, ef, el, ef);                         // K, V die here, dV is final; parked dS3' tiles are read back

  StreamParams sp;
  memset(&sp, 0, sizeof(sp));
  sp.q = a.q; sp.k = a.k; sp.v = a.v; sp.dO = a.d_out;
  sp.dq = a.dq; sp.dk = a.dk; sp.dv = a.dv;
  sp.lse1 = const_cast<float*>(a.lse1);
  sp.qt = a.q_landmarks; sp.kt = a.k_landmarks; sp.step2 = a.step2;
  sp.lse3 = a.lse3; sp.dO3 = w.dO3; sp.D3 = w.D3;
  sp.dqt_tot = w.dqt_tot; sp.dkt_tot = w.dkt_tot;
  sp.partA = w.partA; sp.partB = w.partB;
  sp.N = p.N; sp.rows_per_chunk = p.rows_per_chunk; sp.D = p.D; sp.m = p.m; sp.mpad = p.mpad;
  sp.nchunk = p.nchunk; sp.scale = scale; sp.seg_N = seg_N; sp.row_offset = row_offset;
  const unsigned sgrid = (unsigned)(p.BH * p.nchunk);
  const unsigned tgrid = (unsigned)(p.BH * sch.nchunk);
  const size_t gsmem = bwd_ac_smem(p.mpad, p.D);
  const int nchunk_used = use_tc ? sch.nchunk : p.nchunk;        // pass A partials
  const int nchunk_colpass = use_tc ? sch_b.nchunk : p.nchunk;   // column pass partials

  void* qt16 = w.op16[3]; void* do3n = w.op16[5];
  CUtensorMap tm_q, tm_g, tm_dq, tm_dk;
  if (use_tc) {
    if (!tc::make_map_big(&tm_q, a.q, a.shape.dtype, big, tc::kTile) ||
        !tc::make_map_big(&tm_g, a.d_out, a.shape.dtype, big, tc::kTile) ||
        !tc::make_map_big(&tm_dq, a.dq, a.shape.dtype, big, tc::kTile) ||
        !tc::make_map_big(&tm_dk, a.dk, a.shape.dtype, big, tc::kTile))
      return fail(FNB_ERR_CUDA, "cuTensorMapEncodeTiled failed for the backward row passes");
  }
  auto reduce_chunks = [&](const float* in, int nchunk, int elems, float* out) {
    dim3 grid((unsigned)((elems / 4 + 63) / 64), (unsigned)p.BH);
    launch_pdl(reduce_chunks_kernel, dim3(grid), dim3(kThreads), 0, st, in, nchunk, elems, out);
  };

  // ---- pass A ---------------------------------------------------------------------------------
  if (S.run(0)) {
  if constexpr (k16) {
    if (use_tc) {
      int rc = dispatch_tc(p.D, MP, [&](auto dtag, auto mtag) -> int {
        constexpr int D = decltype(dtag)::value, MPc = decltype(mtag)::value;
        L.begin();
        auto kern = tc::tc_bwd_a_kernel<T, D, MPc>;
        size_t sm = tc::BwdASmem<D, MPc>::kBytes;
        if (int rc2 = set_smem(kern, sm, max_smem, "tc_bwd_a")) return rc2;
        launch_pdl(kern, dim3(tgrid), dim3(tc::kTcThreads), sm, st, tm_q, tm_g, tm_dq, a.k_landmarks, a.step2, a.lse1,
                   w.partA, w.st_scale, sch_a, p.m, scale, a.device_status);
        return L.end("tc_bwd_a");
      });
      if (rc) return rc;
    }
  }
  if (!use_tc) {
    L.begin();
    if (int rc = set_smem(gen_bwd_a_kernel<T>, gsmem, max_smem, "gen_bwd_a")) return rc;
    gen_bwd_a_kernel<T><<<sgrid, kThreads, gsmem, st>>>(sp);
    if (L.end("gen_bwd_a")) return L.status;
  }
  if (S.on()) {
    L.begin();
    reduce_chunks(w.partA, nchunk_used, 2 * p.m * p.D, S.xfer);
    if (L.end("reduce_partA")) return L.status;
  }
  }  // stage 0
  if (S.stage == 0) return 0;
  const float* partA_src = S.on() ? S.xfer : w.partA;
  const int partA_chunks = S.on() ? 1 : nchunk_used;

  // ---- landmark-sized middle ------------------------------------------------------------------
  if (S.run(1)) {
  Fork fork(st, a.device, side_ns);
  if (smem_ns) {
    if (!fused_mid) {
    L.begin();
    {
      BwdMid1Params mp;
      mp.partA = partA_src; mp.nchunk = partA_chunks; mp.k2inv = a.k2_inv; mp.bmat = a.bmat;
      mp.q_landmarks = a.q_landmarks; mp.dkt_a = w.dkt_a; mp.dO3 = w.dO3; mp.D3 = w.D3; mp.G = w.G;
      mp.m = p.m; mp.D = p.D; mp.dtype = use_tc ? a.shape.dtype : 0; mp.MP = MP;
      mp.qt16 = qt16; mp.qtT16 = nullptr; mp.do3n = do3n; mp.do3T = nullptr; mp.do3_scale = w.do3_scale;
      mp.qt_mul = scale * tc::kLog2e; mp.qtT_mul = scale;
      size_t sm = bwd_mid1_smem(p.m, p.D);
      auto kern = p.D == 16 ? bwd_mid1_kernel<1> : p.D == 32 ? bwd_mid1_kernel<2> : p.D == 64 ? bwd_mid1_kernel<4>
                                                                                            : bwd_mid1_kernel<8>;
      if (int rc = set_smem(kern, sm, max_smem, "bwd_mid1")) return rc;
      kern<<<(unsigned)p.BH, kThreads, sm, st>>>(mp);
    }
    if (L.end("bwd_mid1")) return L.status;
    }
    // One SM per slice is slow at summing many chunk partials (L2 -> SM bandwidth): a wide
    // reduction first, then the fused stage reads a single chunk.
    const float* fused_pa = partA_src;
    int fused_pa_chunks = partA_chunks;
    if (fused_mid && partA_chunks > (side_ns ? 1 : 4)) {
      L.begin();
      reduce_chunks(partA_src, partA_chunks, 2 * p.m * p.D, w.partA_red);
      if (L.end("reduce_partA")) return L.status;
      fused_pa = w.partA_red;
      fused_pa_chunks = 1;
    }
    cudaStream_t ns_stream = fork.begin();   // the caller's stream unless side_ns
    L.begin();
    {
      ns::NsBwdParams np;
      np.k2 = a.k2; np.iterates = a.ns_iterates; np.G = w.G; np.qt = a.q_landmarks; np.kt = a.k_landmarks;
      np.dkt_a = w.dkt_a; np.dqt_ns = w.dqt_ns; np.dkt_tot = w.dkt_tot; np.spill = w.dK2;
      np.m = p.m; np.D = p.D; np.J = p.J; np.kappa = a.shape.kappa_star;
      np.rows_k = use_tc ? w.rows_k : nullptr; np.N = seg_N; np.scale = scale;
      if (p.J >= 1 && ns_on_tensor_cores(a.shape.flags)) {
        auto ns_kern = p.D == 128 ? nstc::ns_bwd_tc_kernel<2> : nstc::ns_bwd_tc_kernel<1>;
        if (int rc = set_smem(ns_kern, nstc::kBwdSmem, max_smem, "ns_bwd")) return rc;
        nstc::BwdHeadParams hp{};
        if (fused_mid) {
          hp.partA = fused_pa; hp.nchunk = fused_pa_chunks; hp.k2inv = a.k2_inv; hp.bmat = a.bmat;
          hp.dkt_a = w.dkt_a; hp.D3 = side_ns ? nullptr : w.D3; hp.do3n = do3n; hp.do3_scale = w.do3_scale;
          hp.qt16 = qt16; hp.qt_mul = scale * tc::kLog2e; hp.dtype = a.shape.dtype; hp.MP = MP;
        }
        if (side_ns)
          ns_kern<<<(unsigned)p.BH, nstc::kNsTcThreads, nstc::kBwdSmem, ns_stream>>>(np, hp, a.device_status);
        else
          launch_pdl(ns_kern, dim3((unsigned)p.BH), dim3(nstc::kNsTcThreads), nstc::kBwdSmem, st, np, hp, a.device_status);
      } else {
        if (int rc = set_smem(ns::ns_bwd_kernel, ns::kBwdSmem, max_smem, "ns_bwd")) return rc;
        ns::ns_bwd_kernel<<<(unsigned)p.BH, kThreads, ns::kBwdSmem, st>>>(np);
      }
    }
    if (L.end("ns_bwd")) return L.status;
    fork.end();
    if (side_ns) {
      // what the column pass needs from the middle stage (dO3 -> D3, its 16-bit copy and scale, the
      // 16-bit Qt operand), on the caller's stream; the Newton-Schulz kernel, enqueued first, is
      // resident on its SMs by the time the column pass starts
      ColpassOperandParams cp;
      cp.dstep2 = fused_pa; cp.bh_stride = 2 * (int64_t)p.m * p.D; cp.k2inv = a.k2_inv; cp.bmat = a.bmat;
      cp.q_landmarks = a.q_landmarks; cp.D3 = w.D3; cp.do3n = do3n; cp.do3_scale = w.do3_scale; cp.qt16 = qt16;
      cp.qt_mul = scale * tc::kLog2e; cp.m = p.m; cp.dtype = a.shape.dtype;
      if (int rc = set_smem(colpass_operands_kernel, (size_t)kColpassOperandSmem, max_smem, "colpass_operands")) return rc;
      launch_pdl(colpass_operands_kernel, dim3((unsigned)p.BH), dim3(kThreads), (size_t)kColpassOperandSmem, st, cp);
    }
  } else {
    L.begin();
    {
      MidBwdParams mp;
      mp.partA = partA_src; mp.nchunk = partA_chunks;
      mp.qt = a.q_landmarks; mp.kt = a.k_landmarks; mp.k2 = a.k2; mp.iterates = a.ns_iterates;
      mp.k2inv = a.k2_inv; mp.bmat = a.bmat;
      mp.dstep2 = w.dstep2; mp.dkt_a = w.dkt_a; mp.dO3 = w.dO3; mp.D3 = w.D3;
      mp.dqt_ns = w.dqt_ns; mp.dkt_tot = w.dkt_tot; mp.G = w.G; mp.dK2 = w.dK2; mp.scratch = w.pinv;
      mp.m = p.m; mp.D = p.D; mp.J = p.J; mp.kappa = a.shape.kappa_star; mp.first_half_only = 0;
      mp.use_tc = (a.shape.flags & FNB_FLAG_FORCE_GENERIC) ? 0 : 1;
      mp.status = a.device_status;
      const size_t mid_smem = mp.use_tc ? kTcGemmSmem : 0;
      if (mp.use_tc)
        if (int rc = set_smem(mid_bwd_kernel, mid_smem, max_smem, "mid_bwd")) return rc;
      if (mp.use_tc && !mp.first_half_only) {
        const int cs = mid_cluster_size(mid_bwd_kernel, p.BH, a.device);
        FNB_CUDA(launch_cluster(mid_bwd_kernel, dim3((unsigned)(p.BH * cs)), dim3(kMidTcThreads), mid_smem, st, cs, mp));
      } else {
        mid_bwd_kernel<<<(unsigned)p.BH, kThreads, mid_smem, st>>>(mp);
      }
    }
    if (L.end("mid_bwd")) return L.status;
    if (use_tc) {
      // what the tensor-core column pass and the in-place pass need from the middle stage
      L.begin();
      MidPackParams pp;
      pp.dO3 = w.dO3; pp.q_landmarks = a.q_landmarks; pp.dkt_tot = w.dkt_tot; pp.do3n = do3n; pp.do3_scale = w.do3_scale;
      pp.qt16 = qt16; pp.rows_k = w.rows_k; pp.m = p.m; pp.D = p.D; pp.MP = MP; pp.dtype = a.shape.dtype;
      pp.qt_mul = scale * tc::kLog2e; pp.scale = scale; pp.N = seg_N;
      mid_pack_kernel<<<dim3((unsigned)p.BH, kMidPackSplit), kThreads, 0, st>>>(pp);
      if (L.end("mid_pack")) return L.status;
    }
  }

  // ---- pass B ---------------------------------------------------------------------------------
  if constexpr (k16) {
    if (use_tc) {
      int rc = dispatch_tc(p.D, MP, [&](auto dtag, auto mtag) -> int {
        constexpr int D = decltype(dtag)::value, MPc = decltype(mtag)::value;
        CUtensorMap tm_k, tm_v, tm_qt, tm_do3, tm_dv;
        if (!tc::make_map_big(&tm_k, a.k, a.shape.dtype, big, tc::kTile) ||
            !tc::make_map_big(&tm_v, a.v, a.shape.dtype, big, tc::kTile) ||
            !tc::make_map_big(&tm_dv, a.dv, a.shape.dtype, big, tc::kTile) ||
            !tc::make_map_2d(&tm_qt, qt16, a.shape.dtype, p.BH * MPc, D, MPc) ||
            !tc::make_map_2d(&tm_do3, do3n, a.shape.dtype, p.BH * MPc, D, MPc))
          return fail(FNB_ERR_CUDA, "cuTensorMapEncodeTiled failed for the backward column pass");
        L.begin();
        auto kern = tc::tc_bwd_b_kernel<T, D, MPc>;
        size_t sm = tc::BwdBSmem<D, MPc>::kBytes;
        if (int rc2 = set_smem(kern, sm, max_smem, "tc_bwd_b")) return rc2;
        const dim3 bgrid((unsigned)(p.BH * sch_b.nchunk));
        if (side_ns)   // an ordinary launch: it must not claim SMs before the Newton-Schulz kernel has its own
          kern<<<bgrid, tc::kTcThreads, sm, st>>>(tm_k, tm_v, tm_qt, tm_do3, tm_dk, tm_dv, a.lse3, w.D3, w.do3_scale, w.partB,
                                                  w.tile_scale, sch_b, p.m, scale, kshift, a.device_status);
        else
          launch_pdl(kern, bgrid, dim3(tc::kTcThreads), sm, st, tm_k, tm_v, tm_qt, tm_do3, tm_dk, tm_dv, a.lse3, w.D3, w.do3_scale,
                     w.partB, w.tile_scale, sch_b, p.m, scale, kshift, a.device_status);
        return L.end("tc_bwd_b");
      });
      if (rc) return rc;
    }
  }
  if (!use_tc) {
    L.begin();
    if (int rc = set_smem(gen_bwd_b_kernel<T>, gsmem, max_smem, "gen_bwd_b")) return rc;
    gen_bwd_b_kernel<T><<<sgrid, kThreads, gsmem, st>>>(sp);
    if (L.end("gen_bwd_b")) return L.status;
  }
  if (S.on()) {
    // the Newton-Schulz kernel on the side stream reads its (dstep2, dKt) input from the transfer
    // buffer that the reduction below overwrites: wait for it first
    fork.join();
    L.begin();
    reduce_chunks(w.partB, nchunk_colpass, p.m * p.D, S.xfer);
    if (L.end("reduce_partB")) return L.status;
  }
  fork.join();
  }  // stage 1
  if (S.stage == 1) return 0;
  const float* partB_src = S.on() ? S.xfer : w.partB;
  const int partB_chunks = S.on() ? 1 : nchunk_colpass;

  // ---- pass C ---------------------------------------------------------------------------------
  if constexpr (k16) {
    if (use_tc) {
      return dispatch_tc(p.D, MP, [&](auto dtag, auto mtag) -> int {
      constexpr int D = decltype(dtag)::value, MPc = decltype(mtag)::value;
      L.begin();
      auto kern = tc::tc_rows_inplace_kernel<T, D, MPc>;
      size_t sm = tc::RowsSmem<D, MPc>::kBytes;
      if (int rc2 = set_smem(kern, sm, max_smem, "tc_bwd_c")) return rc2;
      // dQ from the dS1 tiles pass A left in dq, dK from the dS3' tiles the column pass left in dk.
      // Every CTA first sums the column-pass partials of the landmark rows its own tiles touch
      // (rows_q = s (dQt_ns + sum of partials) / len), so no separate reduction kernel runs.
      // The dQ side keeps contiguous runs of tiles (a CTA sums the partials of the landmarks its own
      // run touches); the dK side follows the column pass backwards.
      tc::RowsSide side_q{a.k_landmarks, w.rows_q, w.st_scale, tc::kLn2, partB_src, w.dqt_ns, partB_chunks, scale, 0, nullptr};
      tc::RowsSide side_k{a.q_landmarks, w.rows_k, nullptr, exp2f(-(float)kshift) * tc::kLn2, nullptr, nullptr, 0, 0.f,
                          ((l2 & 4) ? tc::kOrderDescending : 0) | (((l2 & 4) && strided) ? tc::kOrderStrided : 0),
                          w.tile_scale};
      sch_c.hint = hint_bits(ef, ef, ef, ef);   // parked tiles are dead once read, dQ / dK are final
      // (after the join with the side stream the event wait stays a full dependency; only the
      // dependency on the column pass is the programmatic one, as for the combine step of the forward)
      if (l2 & 4)
        launch_pdl(kern, dim3(tgrid), dim3(tc::RowsSmem<D, MPc>::kThreads), sm, st, tm_dk, tm_dq, side_k, side_q, 2, scale * tc::kLog2e, sch_c,
                   p.m, a.device_status);
      else
        launch_pdl(kern, dim3(tgrid), dim3(tc::RowsSmem<D, MPc>::kThreads), sm, st, tm_dq, tm_dk, side_q, side_k, 2, scale * tc::kLog2e, sch_c,
                   p.m, a.device_status);
      return L.end("tc_bwd_c");
      });
    }
  }
  L.begin();
  {
    const int md = p.m * p.D;
    dim3 grid((unsigned)((md / 4 + 63) / 64), (unsigned)p.BH);
    dqt_reduce2_kernel<<<grid, kThreads, 0, st>>>(partB_src, partB_chunks, w.dqt_ns, w.dqt_tot, nullptr, p.m, p.D,
                                                 seg_N, scale);
  }
  if (L.end("dqt_reduce")) return L.status;
  L.begin();
  if (int rc = set_smem(gen_bwd_c_kernel<T>, gsmem, max_smem, "gen_bwd_c")) return rc;
  gen_bwd_c_kernel<T><<<sgrid, kThreads, gsmem, st>>>(sp);
  if (L.end("gen_bwd_c")) return L.status;
  return 0;
}


static size_t fwd_ws_total(const fnb_shape& s) { return carve_fwd(plan_of(s), nullptr).bytes; }
static size_t bwd_ws_total(const fnb_shape& s) { return carve_bwd(plan_of(s), nullptr).bytes; }

}  // namespace fnb

using namespace fnb;

extern "C" {

const char* fnb_last_error(void) { return g_err; }
int fnb_version(void) { return FNB_ABI_VERSION; }

int fnb_capabilities(int device, fnb_caps* caps) {
  if (!caps) return fail(FNB_ERR_INVALID_ARGUMENT, "caps is NULL");
  memset(caps, 0, sizeof(*caps));
  caps->abi_version = FNB_ABI_VERSION;
  cudaDeviceProp prop;
  FNB_CUDA(cudaGetDeviceProperties(&prop, device));
  caps->cc_major = prop.major; caps->cc_minor = prop.minor;
  caps->sm_count = prop.multiProcessorCount;
  caps->max_smem_per_block = (int)prop.sharedMemPerBlockOptin;
  caps->l2_bytes = prop.l2CacheSize;
  caps->total_mem_bytes = (int64_t)prop.totalGlobalMem;
  if (prop.major != 10)
    return fail(FNB_ERR_UNSUPPORTED_DEVICE,
                "device %d (%s) has compute capability %d.%d; this library is built for sm_100a only",
                device, prop.name, prop.major, prop.minor);
  return 0;
}

int fnb_check_shape(const fnb_shape* shape) { return check_shape(shape); }

size_t fnb_fwd_workspace_bytes(const fnb_shape* shape) {
  if (check_shape(shape)) return 0;
  return fwd_ws_total(*shape);
}
size_t fnb_bwd_workspace_bytes(const fnb_shape* shape) {
  if (check_shape(shape)) return 0;
  return bwd_ws_total(*shape);
}

static int check_fwd_pointers(const fnb_fwd_args* a) {
  const void* big[] = {a->q, a->k, a->v, a->out};
  for (const void* ptr : big)
    if (!ptr || !aligned16(ptr))
      return fail(FNB_ERR_INVALID_ARGUMENT, "q, k, v, out must be non-NULL and 16-byte aligned");
  const void* small[] = {a->lse1, a->q_landmarks, a->k_landmarks, a->k2, a->lse2, a->ns_iterates,
                         a->k2_inv, a->bmat, a->lse3, a->step2};
  for (const void* ptr : small)
    if (!ptr) return fail(FNB_ERR_INVALID_ARGUMENT, "a saved-tensor output pointer is NULL");
  return 0;
}
static int check_bwd_pointers(const fnb_bwd_args* a) {
  const void* big[] = {a->q, a->k, a->v, a->d_out, a->dq, a->dk, a->dv};
  for (const void* ptr : big)
    if (!ptr || !aligned16(ptr))
      return fail(FNB_ERR_INVALID_ARGUMENT, "q, k, v, d_out, dq, dk, dv must be non-NULL and 16-byte aligned");
  const void* small[] = {a->lse1, a->q_landmarks, a->k_landmarks, a->k2, a->ns_iterates, a->k2_inv,
                         a->bmat, a->lse3, a->step2};
  for (const void* ptr : small)
    if (!ptr) return fail(FNB_ERR_INVALID_ARGUMENT, "a saved-tensor input pointer is NULL");
  return 0;
}

int fnb_forward(const fnb_fwd_args* a) {
  if (!a) return fail(FNB_ERR_INVALID_ARGUMENT, "args is NULL");
  if (int rc = check_shape(&a->shape)) return rc;
  if (int rc = check_fwd_pointers(a)) return rc;
  const size_t need = fwd_ws_total(a->shape);
  if (!a->workspace || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 255u))
    return fail(FNB_ERR_WORKSPACE, "forward workspace must be 256-byte aligned and >= %zu bytes (got %zu)",
                need, a->workspace_bytes);
  DeviceGuard g(a->device);
  if (!g.ok) return fail(FNB_ERR_CUDA, "cannot select CUDA device %d", a->device);
  int max_smem = 0, cc = 0, sms = 0;
  if (int rc = device_limits(a->device, &max_smem, &cc, &sms)) return rc;
  cudaStream_t st = (cudaStream_t)a->stream;
  Plan p = plan_of(a->shape);
  FwdWs w = carve_fwd(p, a->workspace);
  switch (a->shape.dtype) {
    case FNB_F32: return forward_impl<float>(*a, p, w, max_smem, sms, st, true);
    case FNB_F16: return forward_impl<__half>(*a, p, w, max_smem, sms, st, true);
    default: return forward_impl<__nv_bfloat16>(*a, p, w, max_smem, sms, st, true);
  }
}

int fnb_backward(const fnb_bwd_args* a) {
  if (!a) return fail(FNB_ERR_INVALID_ARGUMENT, "args is NULL");
  if (int rc = check_shape(&a->shape)) return rc;
  if (int rc = check_bwd_pointers(a)) return rc;
  const size_t need = bwd_ws_total(a->shape);
  if (!a->workspace || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 255u))
    return fail(FNB_ERR_WORKSPACE, "backward workspace must be 256-byte aligned and >= %zu bytes (got %zu)",
                need, a->workspace_bytes);
  DeviceGuard g(a->device);
  if (!g.ok) return fail(FNB_ERR_CUDA, "cannot select CUDA device %d", a->device);
  int max_smem = 0, cc = 0, sms = 0;
  if (int rc = device_limits(a->device, &max_smem, &cc, &sms)) return rc;
  cudaStream_t st = (cudaStream_t)a->stream;
  Plan p = plan_of(a->shape);
  BwdWs w = carve_bwd(p, a->workspace);
  switch (a->shape.dtype) {
    case FNB_F32: return backward_impl<float>(*a, p, w, max_smem, sms, st, true);
    case FNB_F16: return backward_impl<__half>(*a, p, w, max_smem, sms, st, true);
    default: return backward_impl<__nv_bfloat16>(*a, p, w, max_smem, sms, st, true);
  }
}

static int check_sp(const fnb_shape& s, const fnb_sp_info* sp, int is_backward) {
  if (!sp) return fail(FNB_ERR_INVALID_ARGUMENT, "sp is NULL");
  if (sp->world < 1 || sp->rank < 0 || sp->rank >= sp->world)
    return fail(FNB_ERR_INVALID_ARGUMENT, "sequence parallel: rank %d / world %d out of range", sp->rank, sp->world);
  if (sp->stage < 0 || sp->stage > 2) return fail(FNB_ERR_INVALID_ARGUMENT, "sequence parallel: stage must be 0, 1 or 2");
  if (s.layout != FNB_LAYOUT_BHND) return fail(FNB_ERR_INVALID_ARGUMENT, "sequence parallel: only the contiguous (B,H,N,D) layout");
  if (sp->seq_len_global != (int64_t)sp->world * s.seq_len)
    return fail(FNB_ERR_INVALID_ARGUMENT, "sequence parallel: seq_len_global (%lld) must equal world (%d) x local seq_len (%lld)",
                (long long)sp->seq_len_global, sp->world, (long long)s.seq_len);
  if (s.num_landmarks % sp->world != 0 || sp->seq_len_global % s.num_landmarks != 0)
    return fail(FNB_ERR_INVALID_ARGUMENT,
                "sequence parallel: num_landmarks (%d) must be a multiple of world (%d) and divide seq_len_global (%lld)",
                s.num_landmarks, sp->world, (long long)sp->seq_len_global);
  const size_t need = fnb_sp_xfer_floats(&s, sp->world, is_backward, sp->stage);
  if (!sp->xfer || sp->xfer_floats < need)
    return fail(FNB_ERR_WORKSPACE, "sequence parallel: xfer must hold %zu floats (got %zu)", need, sp->xfer_floats);
  return 0;
}

size_t fnb_sp_xfer_floats(const fnb_shape* s, int world, int is_backward, int stage) {
  if (check_shape(s) || world < 1) return 0;
  const size_t md = (size_t)s->batch * s->heads * s->num_landmarks * s->head_dim;
  const size_t mv = (size_t)s->batch * s->heads * s->num_landmarks;
  if (is_backward) return stage == 0 ? 2 * md : md;
  if (stage == 0) return 2 * md;
  if (stage == 1) return md + 2 * mv;
  return (size_t)world * (md + 2 * mv);
}

int fnb_sp_forward(const fnb_fwd_args* a, const fnb_sp_info* sp) {
  if (!a) return fail(FNB_ERR_INVALID_ARGUMENT, "args is NULL");
  if (int rc = check_shape(&a->shape)) return rc;
  if (int rc = check_sp(a->shape, sp, 0)) return rc;
  if (int rc = check_fwd_pointers(a)) return rc;
  const size_t need = fwd_ws_total(a->shape);
  if (!a->workspace || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 255u))
    return fail(FNB_ERR_WORKSPACE, "forward workspace must be 256-byte aligned and >= %zu bytes (got %zu)", need,
                a->workspace_bytes);
  DeviceGuard g(a->device);
  if (!g.ok) return fail(FNB_ERR_CUDA, "cannot select CUDA device %d", a->device);
  int max_smem = 0, cc = 0, sms = 0;
  if (int rc = device_limits(a->device, &max_smem, &cc, &sms)) return rc;
  cudaStream_t st = (cudaStream_t)a->stream;
  Plan p = plan_of(a->shape);
  FwdWs w = carve_fwd(p, a->workspace);
  SpCtx S;
  S.stage = sp->stage; S.rank = sp->rank; S.world = sp->world; S.N_global = sp->seq_len_global; S.xfer = sp->xfer;
  switch (a->shape.dtype) {
    case FNB_F32: return forward_impl<float>(*a, p, w, max_smem, sms, st, true, S);
    case FNB_F16: return forward_impl<__half>(*a, p, w, max_smem, sms, st, true, S);
    default: return forward_impl<__nv_bfloat16>(*a, p, w, max_smem, sms, st, true, S);
  }
}

int fnb_sp_backward(const fnb_bwd_args* a, const fnb_sp_info* sp) {
  if (!a) return fail(FNB_ERR_INVALID_ARGUMENT, "args is NULL");
  if (int rc = check_shape(&a->shape)) return rc;
  if (int rc = check_sp(a->shape, sp, 1)) return rc;
  if (int rc = check_bwd_pointers(a)) return rc;
  const size_t need = bwd_ws_total(a->shape);
  if (!a->workspace || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 255u))
    return fail(FNB_ERR_WORKSPACE, "backward workspace must be 256-byte aligned and >= %zu bytes (got %zu)", need,
                a->workspace_bytes);
  DeviceGuard g(a->device);
  if (!g.ok) return fail(FNB_ERR_CUDA, "cannot select CUDA device %d", a->device);
  int max_smem = 0, cc = 0, sms = 0;
  if (int rc = device_limits(a->device, &max_smem, &cc, &sms)) return rc;
  cudaStream_t st = (cudaStream_t)a->stream;
  Plan p = plan_of(a->shape);
  BwdWs w = carve_bwd(p, a->workspace);
  SpCtx S;
  S.stage = sp->stage; S.rank = sp->rank; S.world = sp->world; S.N_global = sp->seq_len_global; S.xfer = sp->xfer;
  switch (a->shape.dtype) {
    case FNB_F32: return backward_impl<float>(*a, p, w, max_smem, sms, st, true, S);
    case FNB_F16: return backward_impl<__half>(*a, p, w, max_smem, sms, st, true, S);
    default: return backward_impl<__nv_bfloat16>(*a, p, w, max_smem, sms, st, true, S);
  }
}

size_t fnb_debug_pinv_workspace_bytes(int64_t bh, int32_t m) {
  if (bh <= 0 || m < 1 || m > kMaxM) return 0;
  return align256((size_t)bh * kPinvBwdBufs * m * m * sizeof(float));
}

static int check_pinv_args(int64_t bh, int32_t m, int32_t J, float kappa, const void* ws,
                           size_t ws_bytes) {
  if (bh <= 0 || bh > ((int64_t)1 << 24)) return fail(FNB_ERR_INVALID_ARGUMENT, "bh out of range");
  if (m < 1 || m > kMaxM) return fail(FNB_ERR_INVALID_ARGUMENT, "num_landmarks must be in [1, %d], got %d", kMaxM, m);
  if (J < 1 || J > 20) return fail(FNB_ERR_INVALID_ARGUMENT, "newton_iter must be in [1, 20], got %d", J);
  if (!std::isfinite(kappa) || kappa < 0.f) return fail(FNB_ERR_INVALID_ARGUMENT, "kappa_star must be finite and >= 0");
  if (!ws || ws_bytes < fnb_debug_pinv_workspace_bytes(bh, m))
    return fail(FNB_ERR_WORKSPACE, "pinv workspace too small: need %zu bytes", fnb_debug_pinv_workspace_bytes(bh, m));
  return 0;
}

int fnb_debug_pinv_forward(int64_t bh, int32_t m, int32_t J, float kappa, const float* k2,
                           float* ns_iterates, float* k2_inv, void* workspace, size_t workspace_bytes,
                           int32_t device, void* stream) {
  if (int rc = check_pinv_args(bh, m, J, kappa, workspace, workspace_bytes)) return rc;
  if (!k2 || !ns_iterates || !k2_inv) return fail(FNB_ERR_INVALID_ARGUMENT, "NULL tensor pointer");
  DeviceGuard g(device);
  if (!g.ok) return fail(FNB_ERR_CUDA, "cannot select CUDA device %d", device);
  if (m <= ns::kN && ns_on_tensor_cores(0)) {
    FNB_CUDA(cudaFuncSetAttribute(nstc::ns_pinv_fwd_tc_debug_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)nstc::kFwdSmem));
    nstc::ns_pinv_fwd_tc_debug_kernel<<<(unsigned)bh, nstc::kNsTcThreads, nstc::kFwdSmem, (cudaStream_t)stream>>>(
        k2, ns_iterates, k2_inv, m, J, kappa, nullptr);
  } else if (m <= ns::kN) {
    FNB_CUDA(cudaFuncSetAttribute(ns::ns_pinv_fwd_debug_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)ns::kFwdSmem));
    ns::ns_pinv_fwd_debug_kernel<<<(unsigned)bh, kThreads, ns::kFwdSmem, (cudaStream_t)stream>>>(
        k2, ns_iterates, k2_inv, m, J, kappa);
  } else {
    const int use_tc = ns_on_tensor_cores(0) ? 1 : 0;
    if (use_tc)
      FNB_CUDA(cudaFuncSetAttribute(pinv_fwd_debug_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcGemmSmem));
    const int cs = use_tc ? mid_cluster_size(pinv_fwd_debug_kernel, bh, device) : 1;
    FNB_CUDA(launch_cluster(pinv_fwd_debug_kernel, dim3((unsigned)(bh * cs)), dim3(use_tc ? kMidTcThreads : kThreads),
                            use_tc ? kTcGemmSmem : 0, (cudaStream_t)stream, cs, k2, ns_iterates, k2_inv, (float*)workspace, m,
                            J, kappa, use_tc));
  }
  FNB_CUDA(cudaPeekAtLastError());
  return 0;
}

int fnb_debug_pinv_backward(int64_t bh, int32_t m, int32_t J, float kappa, const float* k2,
                            const float* ns_iterates, const float* d_k2_inv, float* d_k2,
                            void* workspace, size_t workspace_bytes, int32_t device, void* stream) {
  if (int rc = check_pinv_args(bh, m, J, kappa, workspace, workspace_bytes)) return rc;
  if (!k2 || !ns_iterates || !d_k2_inv || !d_k2) return fail(FNB_ERR_INVALID_ARGUMENT, "NULL tensor pointer");
  DeviceGuard g(device);
  if (!g.ok) return fail(FNB_ERR_CUDA, "cannot select CUDA device %d", device);
  if (m <= ns::kN && ns_on_tensor_cores(0)) {
    FNB_CUDA(cudaFuncSetAttribute(nstc::ns_pinv_bwd_tc_debug_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)nstc::kBwdSmem));
    nstc::ns_pinv_bwd_tc_debug_kernel<<<(unsigned)bh, nstc::kNsTcThreads, nstc::kBwdSmem, (cudaStream_t)stream>>>(
        k2, ns_iterates, d_k2_inv, d_k2, (float*)workspace, m, J, kappa, nullptr, nullptr, nullptr);
  } else if (m <= ns::kN) {
    FNB_CUDA(cudaFuncSetAttribute(ns::ns_pinv_bwd_debug_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)ns::kBwdSmem));
    ns::ns_pinv_bwd_debug_kernel<<<(unsigned)bh, kThreads, ns::kBwdSmem, (cudaStream_t)stream>>>(
        k2, ns_iterates, d_k2_inv, d_k2, (float*)workspace, m, J, kappa);
  } else {
    const int use_tc = ns_on_tensor_cores(0) ? 1 : 0;
    if (use_tc)
      FNB_CUDA(cudaFuncSetAttribute(pinv_bwd_debug_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcGemmSmem));
    const int cs = use_tc ? mid_cluster_size(pinv_bwd_debug_kernel, bh, device) : 1;
    FNB_CUDA(launch_cluster(pinv_bwd_debug_kernel, dim3((unsigned)(bh * cs)), dim3(use_tc ? kMidTcThreads : kThreads),
                            use_tc ? kTcGemmSmem : 0, (cudaStream_t)stream, cs, k2, ns_iterates, d_k2_inv, d_k2,
                            (float*)workspace, m, J, kappa, use_tc));
  }
  FNB_CUDA(cudaPeekAtLastError());
  return 0;
}

// Device address of g_noalloc_scratch on `device`.  In host code the array's name is only a
// stand-in; the address a kernel can use comes from cudaGetSymbolAddress, asked once per device
// while that device is current.
static int noalloc_scratch(int device, float** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static float* table[kMaxDevices] = {};
  if (device < 0 || device >= kMaxDevices) return fail(FNB_ERR_INVALID_ARGUMENT, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(mu);
  if (!table[device]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);   // the caller made `device` current
    if (e != cudaSuccess || !ptr)
      return fail(FNB_ERR_CUDA, "cudaGetSymbolAddress(scratch) failed on device %d: %s", device, cudaGetErrorString(e));
    table[device] = static_cast<float*>(ptr);
  }
  *out = table[device];
  return 0;
}

int fnb_pinv_backward_noalloc(int64_t bh, int32_t m, int32_t J, float kappa, const float* k2,
                              const float* ns_iterates, const float* d_k2_inv, float* d_k2, int32_t device,
                              void* stream) {
  if (bh < 1 || bh > kNoAllocMaxSlices)
    return fail(FNB_ERR_INVALID_ARGUMENT, "fnb_pinv_backward_noalloc handles 1..%d slices per call, got %lld",
                kNoAllocMaxSlices, (long long)bh);
  if (m < 1 || m > kNoAllocMaxM)
    return fail(FNB_ERR_INVALID_ARGUMENT, "fnb_pinv_backward_noalloc handles num_landmarks in [1, %d], got %d",
                kNoAllocMaxM, m);
  if (J < 1 || J > 20) return fail(FNB_ERR_INVALID_ARGUMENT, "newton_iter must be in [1, 20], got %d", J);
  if (!std::isfinite(kappa) || kappa < 0.f) return fail(FNB_ERR_INVALID_ARGUMENT, "kappa_star must be finite and >= 0");
  if (!k2 || !ns_iterates || !d_k2_inv || !d_k2) return fail(FNB_ERR_INVALID_ARGUMENT, "NULL tensor pointer");
  DeviceGuard g(device);
  if (!g.ok) return fail(FNB_ERR_CUDA, "cannot select CUDA device %d", device);
  int max_smem = 0, cc = 0, sms = 0;
  if (int rc = device_limits(device, &max_smem, &cc, &sms)) return rc;
  float* scratch = nullptr;
  if (int rc = noalloc_scratch(device, &scratch)) return rc;
  if (int rc = set_smem(ns::ns_pinv_bwd_debug_kernel, ns::kBwdSmem, max_smem, "ns_pinv_bwd")) return rc;
  // Nothing in the scratch has to start at zero: with the ridge each slice's (m x m) block is
  // fully written (G^T Z_J) before it is read back; without the ridge it is not touched.
  ns::ns_pinv_bwd_debug_kernel<<<(unsigned)bh, kThreads, ns::kBwdSmem, (cudaStream_t)stream>>>(
      k2, ns_iterates, d_k2_inv, d_k2, scratch, m, J, kappa);
  FNB_CUDA(cudaPeekAtLastError());
  return 0;
}

#ifdef FNB_TC_TRACE
// profiling builds only: the per-tile timestamps of the traced CTA of the last tc_fwd_b launch
__attribute__((visibility("default"))) int fnb_debug_tc_trace(long long* out, int cta) {
  if (cta >= 0) { cudaMemcpyToSymbol(tc::g_tc_trace_cta, &cta, sizeof(int)); return 0; }
  return cudaMemcpyFromSymbol(out, tc::g_tc_trace, sizeof(long long) * 8 * 256) == cudaSuccess ? 0 : -1;
}
__attribute__((visibility("default"))) int fnb_debug_gemm_cycles(unsigned long long* out, int reset) {
  if (reset) { unsigned long long z[8] = {}; return cudaMemcpyToSymbol(g_gemm_cycles, z, sizeof(z)) == cudaSuccess ? 0 : -1; }
  return cudaMemcpyFromSymbol(out, g_gemm_cycles, sizeof(unsigned long long) * 8) == cudaSuccess ? 0 : -1;
}
__attribute__((visibility("default"))) int fnb_debug_tc_span(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, tc::g_tc_span, sizeof(unsigned long long) * 6 * 1024) == cudaSuccess ? 0 : -1;
}
#endif

int fnb_debug_ns_bwd_step(int64_t bh, int32_t m, const float* k2, const float* z_j, const float* d_z_next,
                          float* d_z_out, float* d_k2_acc, int32_t device, void* stream) {
  if (bh <= 0 || bh > ((int64_t)1 << 24)) return fail(FNB_ERR_INVALID_ARGUMENT, "bh out of range");
  if (m < 1 || m > ns::kN)
    return fail(FNB_ERR_INVALID_ARGUMENT, "fnb_debug_ns_bwd_step handles num_landmarks in [1, %d], got %d", ns::kN, m);
  if (!k2 || !z_j || !d_z_next || !d_z_out || !d_k2_acc) return fail(FNB_ERR_INVALID_ARGUMENT, "NULL tensor pointer");
  DeviceGuard g(device);
  if (!g.ok) return fail(FNB_ERR_CUDA, "cannot select CUDA device %d", device);
  int max_smem = 0, cc = 0, sms = 0;
  if (int rc = device_limits(device, &max_smem, &cc, &sms)) return rc;
  if (int rc = set_smem(nstc::ns_pinv_bwd_tc_debug_kernel, nstc::kBwdSmem, max_smem, "ns_pinv_bwd")) return rc;
  // one iteration of the product kernel's loop (J = 1, no ridge), stopped in front of the Z0 tail
  nstc::ns_pinv_bwd_tc_debug_kernel<<<(unsigned)bh, nstc::kNsTcThreads, nstc::kBwdSmem, (cudaStream_t)stream>>>(
      k2, z_j, d_z_next, nullptr, nullptr, m, 1, 0.f, nullptr, d_z_out, d_k2_acc);
  FNB_CUDA(cudaPeekAtLastError());
  return 0;
}

int fnb_debug_ns_bwd_final(int64_t bh, int32_t m, int32_t D, const float* q_landmarks, const float* k_landmarks,
                           const float* k2, const float* d_z0, const float* d_k2_in, const float* zeros_md,
                           float* d_q_landmarks, float* d_k_landmarks, float* d_k2_out, int32_t device, void* stream) {
  if (bh <= 0 || bh > ((int64_t)1 << 24)) return fail(FNB_ERR_INVALID_ARGUMENT, "bh out of range");
  if (m < 1 || m > ns::kN)
    return fail(FNB_ERR_INVALID_ARGUMENT, "fnb_debug_ns_bwd_final handles num_landmarks in [1, %d], got %d", ns::kN, m);
  if (!(D == 16 || D == 32 || D == 64 || D == 128)) return fail(FNB_ERR_INVALID_ARGUMENT, "head_dim must be 16, 32, 64 or 128");
  if (!q_landmarks || !k_landmarks || !k2 || !d_z0 || !d_k2_in || !zeros_md || !d_q_landmarks || !d_k_landmarks || !d_k2_out)
    return fail(FNB_ERR_INVALID_ARGUMENT, "NULL tensor pointer");
  DeviceGuard g(device);
  if (!g.ok) return fail(FNB_ERR_CUDA, "cannot select CUDA device %d", device);
  int max_smem = 0, cc = 0, sms = 0;
  if (int rc = device_limits(device, &max_smem, &cc, &sms)) return rc;
  if (int rc = set_smem(ns::ns_bwd_final_debug_kernel, ns::kBwdSmem, max_smem, "ns_bwd_final")) return rc;
  ns::ns_bwd_final_debug_kernel<<<(unsigned)bh, kThreads, ns::kBwdSmem, (cudaStream_t)stream>>>(
      q_landmarks, k_landmarks, k2, d_z0, d_k2_in, zeros_md, d_q_landmarks, d_k_landmarks, d_k2_out, m, D);
  FNB_CUDA(cudaPeekAtLastError());
  return 0;
}

namespace {
struct KernelEntry { const char* name; const void* fn; int threads; size_t dyn_smem; };
}
int fnb_kernel_report(int device, fnb_kernel_info* out, int cap) {
  if (!out || cap <= 0) return 0;
  DeviceGuard g(device);
  if (!g.ok) return 0;
  using H = __half;
  const KernelEntry ks[] = {
      {"landmark_partial<half>", (const void*)landmark_partial_kernel<H, true>, kThreads, 0},
      {"ns_fwd_tc", (const void*)nstc::ns_fwd_tc_kernel, nstc::kNsTcThreads, nstc::kFwdSmem},
      {"conv_residual<half>", (const void*)conv_residual_kernel<H>, kThreads, conv_smem_bytes(64, 3)},
      {"conv_dw_partial<half,2>", (const void*)conv_dw_partial_kernel<H, 2>, kThreads, conv_smem_bytes(64, 3)},
      {"tc_fwd_b<half,64,64>", (const void*)tc::tc_fwd_b_kernel<H, 64, 64>, tc::kTcThreads, tc::FwdBSmem<64, 64>::kBytes},
      {"combine_slab", (const void*)combine_slab_kernel, kThreads, combine_slab_smem(64)},
      {"tc_fwd_c<half,64,64>", (const void*)tc::tc_fwd_c_kernel<H, 64, 64>, tc::kTcThreads, tc::FwdCSmem<64, 64>::kBytes},
      {"tc_bwd_a<half,64,64>", (const void*)tc::tc_bwd_a_kernel<H, 64, 64>, tc::kTcThreads, tc::BwdASmem<64, 64>::kBytes},
      {"reduce_chunks", (const void*)reduce_chunks_kernel, kThreads, 0},
      {"ns_bwd_tc", (const void*)nstc::ns_bwd_tc_kernel<1>, nstc::kNsTcThreads, nstc::kBwdSmem},
      {"ns_bwd_tc_d128", (const void*)nstc::ns_bwd_tc_kernel<2>, nstc::kNsTcThreads, nstc::kBwdSmem},
      {"colpass_operands", (const void*)colpass_operands_kernel, kThreads, (size_t)kColpassOperandSmem},
      {"tc_bwd_b<half,64,64>", (const void*)tc::tc_bwd_b_kernel<H, 64, 64>, tc::kTcThreads, tc::BwdBSmem<64, 64>::kBytes},
      {"tc_rows_inplace<half,64,64>", (const void*)tc::tc_rows_inplace_kernel<H, 64, 64>, tc::kTcThreads, tc::RowsSmem<64, 64>::kBytes},
      {"tc_fwd_b<half,128,64>", (const void*)tc::tc_fwd_b_kernel<H, 128, 64>, tc::kTcThreads, tc::FwdBSmem<128, 64>::kBytes},
      {"tc_fwd_c<half,128,64>", (const void*)tc::tc_fwd_c_kernel<H, 128, 64>, tc::kTcThreads, tc::FwdCSmem<128, 64>::kBytes},
      {"tc_bwd_a<half,128,64>", (const void*)tc::tc_bwd_a_kernel<H, 128, 64>, tc::kTcThreads, tc::BwdASmem<128, 64>::kBytes},
      {"tc_bwd_b<half,128,64>", (const void*)tc::tc_bwd_b_kernel<H, 128, 64>, tc::kTcThreads, tc::BwdBSmem<128, 64>::kBytes},
      {"tc_rows_inplace<half,128,64>", (const void*)tc::tc_rows_inplace_kernel<H, 128, 64>, tc::RowsSmem<128, 64>::kThreads, tc::RowsSmem<128, 64>::kBytes},
  };
  int n = 0;
  for (const KernelEntry& k : ks) {
    if (n >= cap) break;
    cudaFuncAttributes at;
    if (cudaFuncGetAttributes(&at, k.fn) != cudaSuccess) { cudaGetLastError(); continue; }
    fnb_kernel_info& o = out[n];
    memset(&o, 0, sizeof(o));
    strncpy(o.name, k.name, sizeof(o.name) - 1);
    o.registers = at.numRegs;
    o.static_smem_bytes = (int)at.sharedSizeBytes;
    o.dynamic_smem_bytes = (int)k.dyn_smem;
    o.local_bytes_per_thread = (int)at.localSizeBytes;
    o.threads = k.threads;
    int nb = 0;
    // the same attributes the launches set (set_smem): opt-in dynamic size, largest shared-memory carveout
    if (k.dyn_smem > 0 && raise_smem(k.fn, k.dyn_smem) != cudaSuccess) cudaGetLastError();
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, k.fn, k.threads, k.dyn_smem) != cudaSuccess) { cudaGetLastError(); nb = -1; }
    o.blocks_per_sm = nb;
    ++n;
  }
  return n;
}

// ---- depthwise convolution residual --------------------------------------------------------
static int check_conv_shape(int64_t B, int64_t H, int64_t N, int D, int ks, int dtype, int layout) {
  if (B <= 0 || H <= 0 || N <= 0)
    return fail(FNB_ERR_INVALID_ARGUMENT, "batch, heads and seq_len must be positive (got %lld, %lld, %lld)",
                (long long)B, (long long)H, (long long)N);
  if (B * H > 65535) return fail(FNB_ERR_INVALID_ARGUMENT, "batch * heads (%lld) exceeds 65535", (long long)(B * H));
  if (!(D == 16 || D == 32 || D == 64 || D == 128))
    return fail(FNB_ERR_INVALID_ARGUMENT, "head_dim must be 16, 32, 64 or 128, got %d", D);
  if (ks < 1 || ks > kConvMaxTaps || (ks & 1) == 0)
    return fail(FNB_ERR_INVALID_ARGUMENT, "conv kernel_size must be odd and in [1, %d], got %d", kConvMaxTaps, ks);
  if (dtype != FNB_F32 && dtype != FNB_F16 && dtype != FNB_BF16)
    return fail(FNB_ERR_INVALID_ARGUMENT, "Supported dtypes: float32, float16, bfloat16 (got code %d)", dtype);
  if (layout != FNB_LAYOUT_BHND && layout != FNB_LAYOUT_BNHD)
    return fail(FNB_ERR_INVALID_ARGUMENT, "layout must be FNB_LAYOUT_BHND (0) or FNB_LAYOUT_BNHD (1), got %d", layout);
  return 0;
}

int fnb_conv_residual(const fnb_conv_args* a) {
  if (!a) return fail(FNB_ERR_INVALID_ARGUMENT, "args is NULL");
  if (int rc = check_conv_shape(a->batch, a->heads, a->seq_len, a->head_dim, a->kernel_size, a->dtype, a->layout)) return rc;
  if (!a->v || !a->result || !a->weight) return fail(FNB_ERR_INVALID_ARGUMENT, "v, result and weight must not be NULL");
  if (!aligned16(a->v) || !aligned16(a->result) || (a->base && !aligned16(a->base)))
    return fail(FNB_ERR_INVALID_ARGUMENT, "v, base and result must be 16-byte aligned");
  if (a->v == a->result) return fail(FNB_ERR_INVALID_ARGUMENT, "result must not alias v");
  DeviceGuard g(a->device);
  if (!g.ok) return fail(FNB_ERR_CUDA, "cannot select CUDA device %d", a->device);
  int max_smem = 0, cc = 0, sms = 0;
  if (int rc = device_limits(a->device, &max_smem, &cc, &sms)) return rc;
  tc::BigLayout big{a->batch, a->heads, a->seq_len, a->head_dim, a->layout};
  ConvParams p;
  p.v = a->v; p.base = a->base; p.result = a->result; p.w = a->weight; p.N = a->seq_len;
  p.H = (int)a->heads; p.D = a->head_dim; p.ks = a->kernel_size; p.flip = a->transposed ? 1 : 0;
  p.row_stride = big.row_stride(); p.head_stride = big.head_stride(); p.batch_stride = big.batch_stride();
  const size_t smem = conv_smem_bytes(p.D, p.ks);
  const dim3 grid((unsigned)((a->seq_len + kConvRows - 1) / kConvRows), (unsigned)(a->batch * a->heads));
  cudaStream_t st = (cudaStream_t)a->stream;
  auto launch = [&](auto kern) -> int {
    if (int rc = set_smem(kern, smem, max_smem, "conv_residual")) return rc;
    kern<<<grid, kThreads, smem, st>>>(p);
    FNB_CUDA(cudaPeekAtLastError());
    return 0;
  };
  switch (a->dtype) {
    case FNB_F32: return launch(conv_residual_kernel<float>);
    case FNB_F16: return launch(conv_residual_kernel<__half>);
    default: return launch(conv_residual_kernel<__nv_bfloat16>);
  }
}

size_t fnb_conv_dweight_workspace_bytes(int64_t batch, int64_t heads, int64_t seq_len, int32_t kernel_size) {
  if (batch <= 0 || heads <= 0 || seq_len <= 0 || kernel_size < 1 || kernel_size > kConvMaxTaps) return 0;
  const int64_t tiles = (seq_len + kConvRows - 1) / kConvRows;
  return align256(sizeof(float) * (size_t)(batch * heads * tiles * kernel_size));
}

int fnb_conv_residual_dweight(const fnb_conv_dw_args* a) {
  if (!a) return fail(FNB_ERR_INVALID_ARGUMENT, "args is NULL");
  if (int rc = check_conv_shape(a->batch, a->heads, a->seq_len, a->head_dim, a->kernel_size, a->dtype, a->layout)) return rc;
  if (!a->v || !a->d_out || !a->d_weight) return fail(FNB_ERR_INVALID_ARGUMENT, "v, d_out and d_weight must not be NULL");
  if (!aligned16(a->v) || !aligned16(a->d_out)) return fail(FNB_ERR_INVALID_ARGUMENT, "v and d_out must be 16-byte aligned");
  const size_t need = fnb_conv_dweight_workspace_bytes(a->batch, a->heads, a->seq_len, a->kernel_size);
  if (!a->workspace || a->workspace_bytes < need || !aligned16(a->workspace))
    return fail(FNB_ERR_WORKSPACE, "conv weight-gradient workspace must be 16-byte aligned and >= %zu bytes (got %zu)",
                need, a->workspace_bytes);
  DeviceGuard g(a->device);
  if (!g.ok) return fail(FNB_ERR_CUDA, "cannot select CUDA device %d", a->device);
  int max_smem = 0, cc = 0, sms = 0;
  if (int rc = device_limits(a->device, &max_smem, &cc, &sms)) return rc;
  tc::BigLayout big{a->batch, a->heads, a->seq_len, a->head_dim, a->layout};
  ConvDwParams p;
  p.v = a->v; p.g = a->d_out; p.part = (float*)a->workspace; p.N = a->seq_len;
  p.H = (int)a->heads; p.D = a->head_dim; p.ks = a->kernel_size;
  p.row_stride = big.row_stride(); p.head_stride = big.head_stride(); p.batch_stride = big.batch_stride();
  const size_t smem = conv_smem_bytes(p.D, p.ks);
  const int tiles = (int)((a->seq_len + kConvRows - 1) / kConvRows);
  const dim3 grid((unsigned)tiles, (unsigned)(a->batch * a->heads));
  cudaStream_t st = (cudaStream_t)a->stream;
  auto launch = [&](auto kern) -> int {
    if (int rc = set_smem(kern, smem, max_smem, "conv_dweight")) return rc;
    kern<<<grid, kThreads, smem, st>>>(p);
    FNB_CUDA(cudaPeekAtLastError());
    return 0;
  };
  // rows of a 64-row tile per thread: 64 * (16-byte chunks per row) / 256
  const int nr = std::max(1, kConvRows * (a->head_dim / (a->dtype == FNB_F32 ? 4 : 8)) / kThreads);
  auto by_rows = [&](auto tag) -> int {
    using T = decltype(tag);
    switch (nr) {
      case 1: return launch(conv_dw_partial_kernel<T, 1>);
      case 2: return launch(conv_dw_partial_kernel<T, 2>);
      case 4: return launch(conv_dw_partial_kernel<T, 4>);
      default: return launch(conv_dw_partial_kernel<T, 8>);
    }
  };
  int rc;
  switch (a->dtype) {
    case FNB_F32: rc = by_rows(float{}); break;
    case FNB_F16: rc = by_rows(__half{}); break;
    default: rc = by_rows(__nv_bfloat16{}); break;
  }
  if (rc) return rc;
  const int warps = (int)a->heads * a->kernel_size;
  conv_dw_reduce_kernel<<<(unsigned)((warps * 32 + kThreads - 1) / kThreads), kThreads, 0, st>>>(
      p.part, a->d_weight, (int)a->batch, (int)a->heads, tiles, a->kernel_size);
  FNB_CUDA(cudaPeekAtLastError());
  return 0;
}

int fnb_debug_set_wait_limit_ms(int device, int ms) {
  if (ms < 1 || ms > 10000) return fail(FNB_ERR_INVALID_ARGUMENT, "wait limit must be 1..10000 ms, got %d", ms);
  DeviceGuard g(device);
  if (!g.ok) return fail(FNB_ERR_CUDA, "cannot select CUDA device %d", device);
  const unsigned long long ns = (unsigned long long)ms * 1000000ull;
  FNB_CUDA(cudaMemcpyToSymbol(tc::g_wait_limit_ns, &ns, sizeof(ns)));
  return 0;
}

int fnb_set_profiling(int mode) {
  int prev = g_profile;
  g_profile = mode ? 1 : 0;
  return prev;
}

int fnb_last_profile(fnb_kernel_time* out, int cap) {
  int n = 0;
  if (!out || cap <= 0) return 0;
  for (size_t i = 0; i < g_prof.names.size() && 2 * i + 1 < g_prof.used; ++i) {
    if (n >= cap) break;
    cudaEvent_t e0 = g_prof.pool[2 * i], e1 = g_prof.pool[2 * i + 1];
    float ms = 0.f;
    if (cudaEventSynchronize(e1) != cudaSuccess || cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) {
      cudaGetLastError();
      ms = -1.f;
    }
    strncpy(out[n].name, g_prof.names[i].c_str(), sizeof(out[n].name) - 1);
    out[n].name[sizeof(out[n].name) - 1] = 0;
    out[n].ms = ms;
    ++n;
  }
  return n;
}

}  // extern "C"
