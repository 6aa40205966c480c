// Depthwise convolution residual of the attention module: every head has one 1-D kernel of odd
// length ks that is applied along the sequence to each of its D channels (zero padding, ks / 2 on
// either side), and the result is added to the attention output:
//     result[b,h,n,:] = base[b,h,n,:] + sum_j w[h][j] v[b,h,n + j - ks/2,:]
// The reference forms it with two transposing copies around a grouped F.conv1d and a separate add
// (flash_nystrom/flash_nystrom.py:19-55 and the `out + ...` that follows the kernel call): nine
// passes over N x D-sized data.  Here it is one streaming kernel in the tensors' own layout (plain
// (B,H,N,D) or the head-split view of (B,N,H*D)): a CTA stages 64 rows of V plus the halo in shared
// memory once (converted to FP32, so a tap costs two 16-byte shared loads and eight FMAs) and every
// tap reads it from there, so V, the base and the result cross HBM once each.  The backward is the same kernel with the taps reversed (dV) and a two-stage, fixed-order
// reduction for the ks x H weight gradients.  CUDA cores: the work is a few FMAs per byte.
#pragma once
#include "common.cuh"

namespace fnb {

constexpr int kConvRows = 64;        // output rows per CTA
constexpr int kConvMaxTaps = 127;    // halo of at most 63 rows on either side

struct ConvParams {
  const void* v;            // input whose rows are convolved
  const void* base;         // or null: added to the result
  void* result;
  const float* w;           // [H][ks]
  int64_t N;
  int H, D, ks, flip;       // flip: taps reversed (the transposed operator, for dV)
  int64_t row_stride, head_stride, batch_stride;   // in elements, the same for v, base and result
};

__host__ __device__ inline size_t conv_smem_bytes(int D, int ks) {
  return sizeof(float) * ((size_t)(kConvRows + ks - 1) * D + kConvMaxTaps);
}

// rows [r0 - pad, r0 + kConvRows + pad) of one slice -> shared memory as FP32 (zero outside [0, N)).
// A 16-byte chunk of a 16-bit row becomes two float4: they go to two planes (elements 0..3 of every
// chunk in the first, 4..7 in the second), so that a warp's 16-byte shared loads of one plane cover
// consecutive addresses (rows of 128 bytes for head_dim 64) instead of every other 16 bytes.
//   address of (plane, row, chunk) = plane * rows * cpr * 4 + row * cpr * 4 + chunk * 4   [floats]
template <class T>
__device__ __forceinline__ void conv_stage(float* tile, const T* slice, int64_t r0, int pad, int64_t N, int D,
                                           int64_t row_stride) {
  constexpr int V = Vec16<T>::n;
  const int cpr = D / V, rows = kConvRows + 2 * pad;
  for (int idx = threadIdx.x; idx < rows * cpr; idx += kThreads) {
    const int r = idx / cpr, c = idx - r * cpr;
    const int64_t n = r0 - pad + r;
    float x[V];
#pragma unroll
    for (int e = 0; e < V; ++e) x[e] = 0.f;
    if (n >= 0 && n < N) load16<T>(slice + n * row_stride + c * V, x);
#pragma unroll
    for (int e = 0; e < V; e += 4)
      *reinterpret_cast<float4*>(tile + ((size_t)(e >> 2) * rows + r) * (cpr * 4) + c * 4) =
          make_float4(x[e], x[e + 1], x[e + 2], x[e + 3]);
  }
}

template <class T>
__global__ void __launch_bounds__(kThreads) conv_residual_kernel(ConvParams p) {
  constexpr int V = Vec16<T>::n;
  extern __shared__ __align__(16) uint8_t conv_smem[];
  const int D = p.D, ks = p.ks, pad = ks / 2;
  float* tile = reinterpret_cast<float*>(conv_smem);
  float* ws = tile + (size_t)(kConvRows + ks - 1) * D;
  const int64_t bh = blockIdx.y, b = bh / p.H, h = bh - b * p.H;
  const int64_t off = b * p.batch_stride + h * p.head_stride;
  const int64_t r0 = (int64_t)blockIdx.x * kConvRows;
  if (threadIdx.x < ks) ws[threadIdx.x] = p.w[h * ks + (p.flip ? ks - 1 - threadIdx.x : threadIdx.x)];
  conv_stage<T>(tile, reinterpret_cast<const T*>(p.v) + off, r0, pad, p.N, D, p.row_stride);
  __syncthreads();
  const int cpr = D / V, rpp = kThreads / cpr;
  const int c = threadIdx.x % cpr, rg = threadIdx.x / cpr;
  const T* base = p.base ? reinterpret_cast<const T*>(p.base) + off : nullptr;
  T* result = reinterpret_cast<T*>(p.result) + off;
  for (int r = rg; r < kConvRows; r += rpp) {
    const int64_t n = r0 + r;
    if (n >= p.N) break;
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; ++e) acc[e] = 0.f;
    const int trows = kConvRows + 2 * pad;
    for (int j = 0; j < ks; ++j) {
      const float wj = ws[j];
#pragma unroll
      for (int e = 0; e < V; e += 4) {
        const float4 y = *reinterpret_cast<const float4*>(tile + ((size_t)(e >> 2) * trows + r + j) * (cpr * 4) + c * 4);
        acc[e] = fmaf(wj, y.x, acc[e]); acc[e + 1] = fmaf(wj, y.y, acc[e + 1]);
        acc[e + 2] = fmaf(wj, y.z, acc[e + 2]); acc[e + 3] = fmaf(wj, y.w, acc[e + 3]);
      }
    }
    if (base) {
      float y[V];
      load16<T>(base + n * p.row_stride + c * V, y);
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] += y[e];
    }
    uint4 out;
    T* o = reinterpret_cast<T*>(&out);
#pragma unroll
    for (int e = 0; e < V; ++e) o[e] = from_f<T>(acc[e]);
    *reinterpret_cast<uint4*>(result + n * p.row_stride + c * V) = out;
  }
}

// Weight gradient, stage 1: part[bh][tile][j] = sum over the tile's rows n and all d of
// g[n][d] v[n + j - pad][d].  A thread keeps its rows of g in registers and walks the taps; every
// tap is folded over the warp with shuffles and over the eight warps through shared memory.
struct ConvDwParams {
  const void* v; const void* g;
  float* part;              // [B*H][tiles][ks]
  int64_t N;
  int H, D, ks;
  int64_t row_stride, head_stride, batch_stride;
};

// NR: rows of the tile per thread = max(1, kConvRows * (D / V) / kThreads), V elements per 16 bytes
template <class T, int NR>
__global__ void __launch_bounds__(kThreads) conv_dw_partial_kernel(ConvDwParams p) {
  constexpr int V = Vec16<T>::n;
  constexpr int kMaxRows = NR;
  extern __shared__ __align__(16) uint8_t conv_smem[];
  __shared__ float red[kThreads / 32][kConvMaxTaps + 1];
  const int D = p.D, ks = p.ks, pad = ks / 2;
  float* tile = reinterpret_cast<float*>(conv_smem);
  const int64_t bh = blockIdx.y, b = bh / p.H, h = bh - b * p.H;
  const int64_t off = b * p.batch_stride + h * p.head_stride;
  const int64_t r0 = (int64_t)blockIdx.x * kConvRows;
  conv_stage<T>(tile, reinterpret_cast<const T*>(p.v) + off, r0, pad, p.N, D, p.row_stride);
  const int cpr = D / V, rpp = kThreads / cpr;
  const int c = threadIdx.x % cpr, rg = threadIdx.x / cpr;
  const T* g = reinterpret_cast<const T*>(p.g) + off;
  float gv[kMaxRows][V];
#pragma unroll
  for (int i = 0; i < kMaxRows; ++i) {
    const int rr = rg + i * rpp;          // row of the tile this thread holds in slot i
    const int64_t n = r0 + rr;
#pragma unroll
    for (int e = 0; e < V; ++e) gv[i][e] = 0.f;
    if (rr < kConvRows && n < p.N) load16<T>(g + n * p.row_stride + c * V, gv[i]);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int j = 0; j < ks; ++j) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxRows; ++i) {
      if (rg + i * rpp < kConvRows) {
#pragma unroll
        for (int e = 0; e < V; e += 4) {
          const float4 y = *reinterpret_cast<const float4*>(
              tile + ((size_t)(e >> 2) * (kConvRows + 2 * pad) + rg + i * rpp + j) * (cpr * 4) + c * 4);
          s = fmaf(gv[i][e], y.x, s); s = fmaf(gv[i][e + 1], y.y, s);
          s = fmaf(gv[i][e + 2], y.z, s); s = fmaf(gv[i][e + 3], y.w, s);
        }
      }
    }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) red[warp][j] = s;
  }
  __syncthreads();
  if (threadIdx.x < ks) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) s += red[w][threadIdx.x];
    p.part[(bh * gridDim.x + blockIdx.x) * ks + threadIdx.x] = s;
  }
}

// Weight gradient, stage 2: dw[h][j] = sum over batches and tiles, in a fixed order (one warp per
// (h, j): lane l takes partials l, l + 32, ..., then the lanes are folded).
__global__ void __launch_bounds__(kThreads)
conv_dw_reduce_kernel(const float* part, float* dw, int B, int H, int tiles, int ks) {
  const int warp = (blockIdx.x * kThreads + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= H * ks) return;
  const int h = warp / ks, j = warp - h * ks;
  float s = 0.f;
  for (int i = lane; i < B * tiles; i += 32) {
    const int b = i / tiles, t = i - b * tiles;
    s += part[(((int64_t)b * H + h) * tiles + t) * ks + j];
  }
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) dw[h * ks + j] = s;
}

}  // namespace fnb
