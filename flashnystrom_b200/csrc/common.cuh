// Shared device/host helpers for the flashnystrom_b200 library.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <math.h>

namespace fnb {

constexpr int kThreads = 256;   // every CUDA-core kernel in this library uses 256-thread CTAs
constexpr int kTileRows = 32;   // rows of Q/K/V/dO staged per step by the CUDA-core kernels
constexpr int kMaxM = 128;
constexpr int kMaxD = 128;

// ---- dtype conversion -------------------------------------------------------------------
template <class T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) {
  return __bfloat162float(x);
}
template <class T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

template <class T> struct Vec16 { static constexpr int n = 16 / sizeof(T); };

// 16-byte global load of Vec16<T>::n elements, converted to float.
template <class T>
__device__ __forceinline__ void load16(const T* p, float* out) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec16<T>::n; ++i) out[i] = to_f<T>(e[i]);
}

// ---- segment geometry (floor-division segments, last one takes the remainder) ------------
struct Segments {
  int64_t N;
  int m;
  int64_t seg;
  __host__ __device__ Segments(int64_t N_, int m_) : N(N_), m(m_), seg(N_ / m_) {}
  __host__ __device__ int64_t start(int l) const { return seg * l; }
  __host__ __device__ int64_t end(int l) const { return l == m - 1 ? N : seg * (l + 1); }
  __host__ __device__ int64_t len(int l) const { return end(l) - start(l); }
  __host__ __device__ int landmark_of(int64_t n) const {
    int64_t l = n / seg;
    return l > m - 1 ? m - 1 : (int)l;
  }
};

// ---- launch plan shared by host sizing code and kernels ---------------------------------
struct Plan {
  int64_t BH, N;
  int D, m, J;
  int mpad;           // m rounded up to a multiple of 16
  int lm_chunks;      // CTAs per landmark segment in the pooling pass
  int nchunk;         // CTAs along N per (b,h) in the streaming passes
  int64_t rows_per_chunk;
};

// SM count of the current device (148 when it cannot be asked): workspace sizes and the grids of
// the CUDA-core kernels follow it, so size a workspace with the device current that will run the call.
inline int current_sm_count() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
    cudaGetLastError();
    return 148;
  }
  return sms;
}

inline Plan make_plan(int64_t BH, int64_t N, int D, int m, int J) {
  Plan p;
  p.BH = BH; p.N = N; p.D = D; p.m = m; p.J = J;
  p.mpad = (m + 15) / 16 * 16;
  const int64_t target = 4 * (int64_t)current_sm_count();  // 4 CTAs per SM
  int64_t seg = N / m;
  // pooling pass: a persistent grid of 4 CTAs per SM walks (tensor, slice, landmark, chunk) items;
  // about six items per CTA keep the last round of the walk short
  int64_t c = (6 * target + 2 * BH * m - 1) / (2 * BH * m);
  int64_t cmax = (seg + 63) / 64;
  if (c > cmax) c = cmax;
  if (c < 1) c = 1;
  p.lm_chunks = (int)c;
  int64_t want = (target + BH - 1) / BH;
  int64_t tiles = (N + kTileRows - 1) / kTileRows;
  if (want > tiles) want = tiles;
  if (want < 1) want = 1;
  int64_t tiles_per_chunk = (tiles + want - 1) / want;
  p.rows_per_chunk = tiles_per_chunk * kTileRows;
  p.nchunk = (int)((N + p.rows_per_chunk - 1) / p.rows_per_chunk);
  return p;
}

// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may
// start while its predecessor in the stream is still running.  pdl_trigger() lets the successor of
// this kernel be scheduled early; pdl_wait() returns once the predecessor grid has completed and
// its writes are visible, so it must precede every access to global memory that another kernel
// of the stream writes or reads.  Both are no-ops for a kernel launched the ordinary way.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

#ifdef __CUDACC__
// Scaled landmark row from the raw segment sums of the pooling pass.
//   land: [2][BH][m][C][D] partial sums (which = 0: Q, 1: K), head_dim D = 64.
// Thread t returns columns 16 (t & 3) .. +15 of landmark row t >> 2 (zeros for rows >= m):
// scale * sum / len(row), len from the floor-division segments of a length-seg_N sequence.
__device__ __forceinline__ void pooled_row16(const float* land, int which, int64_t BH, int64_t bh, int m, int C,
                                             int64_t seg_N, float scale, float* v) {
  const int r = (threadIdx.x >> 2) & 63, c0 = (threadIdx.x & 3) * 16;
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = 0.f;
  if (r >= m) return;
  const float* src = land + ((((size_t)which * BH + bh) * m + r) * C) * 64 + c0;
  for (int c = 0; c < C; ++c) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 x = *reinterpret_cast<const float4*>(src + (size_t)c * 64 + 4 * q);
      v[4 * q] += x.x; v[4 * q + 1] += x.y; v[4 * q + 2] += x.z; v[4 * q + 3] += x.w;
    }
  }
  const float f = scale / (float)Segments(seg_N, m).len(r);
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] *= f;
}
#endif

inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

}  // namespace fnb
