// CUDA-core FP32 streaming kernels: the passes over the N-sized tensors for every dtype,
// head size and landmark count the library accepts (fp32 / fp16 / bf16, D in {16,32,64,128},
// 1 <= m <= 128).  They are the verification path and the path for shapes the tensor-core
// kernels do not cover, like the reference's FP32 scalar twins
// (csrc/kernels/kernel1_scalar.cuh:18-92, kernel3_scalar.cuh:13-114).
//
// Each CTA (256 threads viewed as 16 x 16) owns a contiguous chunk of rows of one (b,h) slice
// and walks it in tiles of 32 rows.  All products are register-tiled FP32 FMAs on operands in
// shared memory: thread (ty,tx) owns output rows ty+16i and columns tx+16j.
#pragma once
#include "common.cuh"

namespace fnb {

// acc[i][j] += sum_k fa(i,k) * fb(k,j)
template <int I, int J, class FA, class FB>
__device__ __forceinline__ void bgemm(float (&acc)[I][J], int ilim, int jlim, int K, FA fa, FB fb) {
#pragma unroll 2
  for (int k = 0; k < K; ++k) {
    float a[I], b[J];
#pragma unroll
    for (int i = 0; i < I; ++i) a[i] = (i < ilim) ? fa(i, k) : 0.f;
#pragma unroll
    for (int j = 0; j < J; ++j) b[j] = (j < jlim) ? fb(k, j) : 0.f;
#pragma unroll
    for (int i = 0; i < I; ++i) {
      if (i < ilim) {
#pragma unroll
        for (int j = 0; j < J; ++j)
          if (j < jlim) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
    }
  }
}

template <int I, int J>
__device__ __forceinline__ void zero(float (&acc)[I][J]) {
#pragma unroll
  for (int i = 0; i < I; ++i)
#pragma unroll
    for (int j = 0; j < J; ++j) acc[i][j] = 0.f;
}

// Stage rows [r0, r0+32) of a (N x D) slice into shared memory as scale * float; rows >= rend
// become zero.  dst row stride = ld.
template <class T>
__device__ __forceinline__ void load_tile(float* dst, int ld, const T* slice, int64_t r0,
                                          int64_t rend, int D, float scale) {
  constexpr int V = Vec16<T>::n;
  const int vpr = D / V;
  for (int v = threadIdx.x; v < kTileRows * vpr; v += kThreads) {
    int r = v / vpr, cv = v - r * vpr;
    float x[V];
    if (r0 + r < rend) {
      load16<T>(slice + (r0 + r) * D + cv * V, x);
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) x[e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < V; ++e) dst[r * ld + cv * V + e] = x[e] * scale;
  }
}

// Stage an (m x D) FP32 matrix from global memory into shared memory with row stride ld,
// zero-filling rows m..mpad-1.
__device__ __forceinline__ void load_small(float* dst, int ld, const float* src, int m, int mpad, int D) {
  for (int idx = threadIdx.x; idx < mpad * D; idx += kThreads) {
    int r = idx / D, c = idx - r * D;
    dst[r * ld + c] = (r < m) ? src[r * D + c] : 0.f;
  }
}

// ------------------------------------------------------------------------------------------
// Pass 1: raw segment sums of Q and K (landmark pooling).
// Work items (which, bh, landmark, chunk) are walked by a grid-stride loop, so the grid can be
// sized to the machine.  out[which][bh][l][c][D].  kContig: the slices are contiguous (row stride D,
// slice bh at bh * N * D); the addressing of the streaming loop is then 32-bit and free of the
// run-time strides, which this kernel is sensitive to (59 against 92 us with them at B=1, H=16,
// N=65536, D=64).
template <class T, bool kContig>
__global__ void __launch_bounds__(kThreads, 4)
landmark_partial_kernel(const T* __restrict__ q, const T* __restrict__ k, float* __restrict__ out,
                        int64_t BH, int64_t N, int D, int m, int C, int64_t seg_N, int64_t row_offset,
                        int H, int64_t row_stride, int64_t head_stride, int64_t batch_stride) {
  constexpr int V = Vec16<T>::n;
  __shared__ float red[kThreads * 8];
  pdl_trigger();
  pdl_wait();
  const int64_t per_which = BH * m * C, items = 2 * per_which;
  const int vpr = D / V, rows_per_iter = kThreads / vpr;
  const int cv = threadIdx.x % vpr, ro = threadIdx.x / vpr;
  // lanes that hold the same columns are vpr apart: fold them with shuffles when that tiles a warp
  const bool warp_fold = vpr <= 32 && (vpr & (vpr - 1)) == 0;
  Segments sg(seg_N, m);
  for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
    const int which = (int)(item / per_which);
    const int64_t rest = item - which * per_which;
    const int64_t bh = rest / (m * C);
    const int lc = (int)(rest - bh * (m * C));
    const int l = lc / C, c = lc - l * C;
    // slice (bh % H, bh / H); its rows are row_stride elements apart (D for the contiguous layout)
    const T* slice = (which ? k : q) + (kContig ? bh * N * D : (bh / H) * batch_stride + (bh % H) * head_stride);
    // segment l in global rows, clipped to the rows this rank holds, in local row numbers
    int64_t start = sg.start(l) - row_offset, end = sg.end(l) - row_offset;
    if (start < 0) start = 0;
    if (end > N) end = N;
    const int64_t len = end > start ? end - start : 0;
    const int64_t per = (len + C - 1) / C;
    const int64_t r0 = start + c * per;
    int64_t r1 = r0 + per;
    if (r1 > start + len) r1 = start + len;
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; ++e) acc[e] = 0.f;
    // eight independent 16-byte loads in flight per thread
    int64_t r = r0 + ro;
    if constexpr (kContig) {
      for (; r + 7 * rows_per_iter < r1; r += 8 * rows_per_iter) {
        uint4 raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          raw[u] = __ldcs(reinterpret_cast<const uint4*>(slice + (r + u * rows_per_iter) * D + cv * V));
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const T* e16 = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
          for (int e = 0; e < V; ++e) acc[e] += to_f<T>(e16[e]);
        }
      }
      for (; r < r1; r += rows_per_iter) {
        float x[V];
        load16<T>(slice + r * D + cv * V, x);
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] += x[e];
      }
    } else {
      // strided rows: one running pointer, advanced by additions only
      const T* ptr = slice + r * row_stride + cv * V;
      const int64_t step = (int64_t)rows_per_iter * row_stride;
      for (; r + 7 * rows_per_iter < r1; r += 8 * rows_per_iter) {
        uint4 raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          raw[u] = __ldcs(reinterpret_cast<const uint4*>(ptr));
          ptr += step;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const T* e16 = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
          for (int e = 0; e < V; ++e) acc[e] += to_f<T>(e16[e]);
        }
      }
      for (; r < r1; r += rows_per_iter, ptr += step) {
        float x[V];
        load16<T>(ptr, x);
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] += x[e];
      }
    }
    float* dst = out + ((((size_t)which * BH + bh) * m + l) * C + c) * D;
    if (warp_fold) {
      for (int o = vpr; o < 32; o <<= 1)
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
      const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
      if (lane < vpr)
#pragma unroll
        for (int e = 0; e < V; ++e) red[w * D + lane * V + e] = acc[e];
      __syncthreads();
      if (threadIdx.x < D) {
        float s = 0.f;
#pragma unroll
        for (int ww = 0; ww < kThreads / 32; ++ww) s += red[ww * D + threadIdx.x];
        dst[threadIdx.x] = s;
      }
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) red[ro * D + cv * V + e] = acc[e];
      __syncthreads();
      if (threadIdx.x < D) {
        float s = 0.f;
        for (int rr = 0; rr < rows_per_iter; ++rr) s += red[rr * D + threadIdx.x];
        dst[threadIdx.x] = s;
      }
    }
    __syncthreads();   // red is reused by the next item
  }
}

// ------------------------------------------------------------------------------------------
struct StreamParams {
  const void* q; const void* k; const void* v; const void* dO;
  void* out; void* dq; void* dk; void* dv;
  float* lse1;                 // written by fwd_c, read by bwd_a / bwd_c
  const float* qt; const float* kt; const float* step2;
  const float* lse3; const float* dO3; const float* D3;
  const float* dqt_tot; const float* dkt_tot;
  float* part_acc; float* part_max; float* part_sum;   // softmax-3 partials
  float* partA;                // [BH][nchunk][2][m][D]
  float* partB;                // [BH][nchunk][m][D]
  int64_t N, rows_per_chunk;
  int D, m, mpad, nchunk;
  float scale;
  int64_t seg_N, row_offset;   // landmark-segment geometry (global length, first global row)
};

__host__ __device__ inline size_t fwd_b_smem(int mpad, int D) {
  return sizeof(float) * ((size_t)mpad * (D + 1) + 2 * kTileRows * D + kTileRows * (mpad + 1) + 3 * kMaxM);
}
__host__ __device__ inline size_t fwd_c_smem(int mpad, int D) {
  return sizeof(float) * ((size_t)mpad * (D + 1) + (size_t)mpad * D + kTileRows * D + kTileRows * (mpad + 1));
}
__host__ __device__ inline size_t bwd_ac_smem(int mpad, int D) {
  return sizeof(float) * (2 * (size_t)mpad * (D + 1) + 2 * kTileRows * D + 2 * kTileRows * (mpad + 1));
}
__host__ __device__ inline size_t bwd_b_smem(int mpad, int D) { return bwd_ac_smem(mpad, D); }

// ------------------------------------------------------------------------------------------
// Pass 2: partial Bmat = softmax(Qt (sK)^T) V over this CTA's rows, with running max / sum.
template <class T>
__global__ void __launch_bounds__(kThreads, 1) gen_fwd_b_kernel(StreamParams p) {
  extern __shared__ float smem[];
  const int D = p.D, m = p.m, mpad = p.mpad, t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const int mj = mpad >> 4, dj = D >> 4;
  const int ldq = D + 1, ldp = mpad + 1;
  float* Qt = smem;
  float* Ks = Qt + mpad * ldq;
  float* Vs = Ks + kTileRows * D;
  float* Ps = Vs + kTileRows * D;
  float* rmax = Ps + kTileRows * ldp;
  float* rsum = rmax + kMaxM;
  float* alpha = rsum + kMaxM;
  const int64_t bh = blockIdx.x / p.nchunk, N = p.N;
  const int chunk = (int)(blockIdx.x - bh * p.nchunk);
  const int64_t rb = chunk * p.rows_per_chunk;
  const int64_t re = min(N, rb + p.rows_per_chunk);
  const T* kk = (const T*)p.k + bh * N * D;
  const T* vv = (const T*)p.v + bh * N * D;
  load_small(Qt, ldq, p.qt + bh * m * D, m, mpad, D);
  if (t < kMaxM) { rmax[t] = -INFINITY; rsum[t] = 0.f; alpha[t] = 0.f; }
  float acc[8][8];
  zero(acc);
  __syncthreads();
  for (int64_t r0 = rb; r0 < re; r0 += kTileRows) {
    load_tile<T>(Ks, D, kk, r0, re, D, p.scale);
    load_tile<T>(Vs, D, vv, r0, re, D, 1.f);
    __syncthreads();
    float s[2][8];
    zero(s);
    bgemm<2, 8>(s, 2, mj, D,
                [&](int i, int k) { return Ks[(ty + 16 * i) * D + k]; },
                [&](int k, int j) { return Qt[(tx + 16 * j) * ldq + k]; });
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < mj) Ps[(ty + 16 * i) * ldp + tx + 16 * j] = (r0 + ty + 16 * i < re) ? s[i][j] : -INFINITY;
    __syncthreads();
    if (t < m) {
      float mx = rmax[t], tm = -INFINITY;
      for (int n = 0; n < kTileRows; ++n) tm = fmaxf(tm, Ps[n * ldp + t]);
      float nm = fmaxf(mx, tm);
      float a = expf(mx - nm);
      float sum = rsum[t] * a;
      for (int n = 0; n < kTileRows; ++n) {
        float e = expf(Ps[n * ldp + t] - nm);
        Ps[n * ldp + t] = e;
        sum += e;
      }
      rmax[t] = nm; rsum[t] = sum; alpha[t] = a;
    } else if (t < mpad) {
      for (int n = 0; n < kTileRows; ++n) Ps[n * ldp + t] = 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (i < mj) {
        float a = alpha[ty + 16 * i];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] *= a;
      }
    }
    bgemm<8, 8>(acc, mj, dj, kTileRows,
                [&](int i, int k) { return Ps[k * ldp + ty + 16 * i]; },
                [&](int k, int j) { return Vs[k * D + tx + 16 * j]; });
    __syncthreads();
  }
  const size_t slot = (size_t)bh * p.nchunk + chunk;
  float* pa = p.part_acc + slot * m * D;
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int l = ty + 16 * i, d = tx + 16 * j;
      if (i < mj && j < dj && l < m) pa[l * D + d] = acc[i][j];
    }
  if (t < m) { p.part_max[slot * m + t] = rmax[t]; p.part_sum[slot * m + t] = rsum[t]; }
}

// ------------------------------------------------------------------------------------------
// Pass 3: O = softmax(sQ Kt^T) step2 and lse1, one 32-row tile at a time.
template <class T>
__global__ void __launch_bounds__(kThreads, 1) gen_fwd_c_kernel(StreamParams p) {
  extern __shared__ float smem[];
  const int D = p.D, m = p.m, mpad = p.mpad, t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const int mj = mpad >> 4, dj = D >> 4;
  const int ldk = D + 1, ldp = mpad + 1;
  float* Kt = smem;
  float* St = Kt + mpad * ldk;
  float* Xs = St + mpad * D;
  float* Ps = Xs + kTileRows * D;
  const int64_t bh = blockIdx.x / p.nchunk, N = p.N;
  const int chunk = (int)(blockIdx.x - bh * p.nchunk);
  const int64_t rb = chunk * p.rows_per_chunk;
  const int64_t re = min(N, rb + p.rows_per_chunk);
  const T* qq = (const T*)p.q + bh * N * D;
  T* oo = (T*)p.out + bh * N * D;
  float* lse1 = p.lse1 + bh * N;
  load_small(Kt, ldk, p.kt + bh * m * D, m, mpad, D);
  load_small(St, D, p.step2 + bh * m * D, m, mpad, D);
  __syncthreads();
  for (int64_t r0 = rb; r0 < re; r0 += kTileRows) {
    load_tile<T>(Xs, D, qq, r0, re, D, p.scale);
    __syncthreads();
    float s[2][8];
    zero(s);
    bgemm<2, 8>(s, 2, mj, D,
                [&](int i, int k) { return Xs[(ty + 16 * i) * D + k]; },
                [&](int k, int j) { return Kt[(tx + 16 * j) * ldk + k]; });
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < mj && tx + 16 * j < m) mx = fmaxf(mx, s[i][j]);
      for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float e = (j < mj && tx + 16 * j < m) ? expf(s[i][j] - mx) : 0.f;
        s[i][j] = e;
        sum += e;
      }
      for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      float inv = 1.f / sum;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < mj) Ps[(ty + 16 * i) * ldp + tx + 16 * j] = s[i][j] * inv;
      int64_t row = r0 + ty + 16 * i;
      if (tx == 0 && row < re) lse1[row] = mx + logf(sum);
    }
    __syncthreads();
    float o[2][8];
    zero(o);
    bgemm<2, 8>(o, 2, dj, m,
                [&](int i, int k) { return Ps[(ty + 16 * i) * ldp + k]; },
                [&](int k, int j) { return St[k * D + tx + 16 * j]; });
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      int64_t row = r0 + ty + 16 * i;
      if (row < re) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < dj) oo[row * D + tx + 16 * j] = from_f<T>(o[i][j]);
      }
    }
    __syncthreads();
  }
}

// Shared front half of the two softmax-1 backward passes: for the staged tile compute
// P1 = exp(S1 - lse1), dP1 = dO step2^T, D1 = rowsum(P1 o dP1), dS1 = P1 o (dP1 - D1)
// and leave P1 / dS1 in shared memory (rows past the end are zero).
__device__ __forceinline__ void softmax1_bwd_tile(const float* Xs, const float* Gs, const float* Kt,
                                                  const float* St, float* Ps, float* dSs,
                                                  const float* lse1, int64_t r0, int64_t re, int D,
                                                  int m, int mj, int ldk, int ldp, bool want_p) {
  const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
  float s[2][8], g[2][8];
  zero(s);
  zero(g);
  bgemm<2, 8>(s, 2, mj, D,
              [&](int i, int k) { return Xs[(ty + 16 * i) * D + k]; },
              [&](int k, int j) { return Kt[(tx + 16 * j) * ldk + k]; });
  bgemm<2, 8>(g, 2, mj, D,
              [&](int i, int k) { return Gs[(ty + 16 * i) * D + k]; },
              [&](int k, int j) { return St[(tx + 16 * j) * ldk + k]; });
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    int64_t row = r0 + ty + 16 * i;
    bool ok = row < re;
    float l = ok ? lse1[row] : 0.f;
    float d1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float pv = (ok && j < mj && tx + 16 * j < m) ? expf(s[i][j] - l) : 0.f;
      s[i][j] = pv;
      d1 += pv * g[i][j];
    }
    for (int o = 8; o > 0; o >>= 1) d1 += __shfl_xor_sync(0xffffffffu, d1, o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < mj) {
        if (want_p) Ps[(ty + 16 * i) * ldp + tx + 16 * j] = s[i][j];
        dSs[(ty + 16 * i) * ldp + tx + 16 * j] = s[i][j] * (g[i][j] - d1);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Backward pass A: per-chunk partials of dstep2 = P1^T dO and dKt = dS1^T (sQ).
template <class T>
__global__ void __launch_bounds__(kThreads, 1) gen_bwd_a_kernel(StreamParams p) {
  extern __shared__ float smem[];
  const int D = p.D, m = p.m, mpad = p.mpad, t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const int mj = mpad >> 4, dj = D >> 4;
  const int ldk = D + 1, ldp = mpad + 1;
  float* Kt = smem;
  float* St = Kt + mpad * ldk;
  float* Xs = St + mpad * ldk;
  float* Gs = Xs + kTileRows * D;
  float* Ps = Gs + kTileRows * D;
  float* dSs = Ps + kTileRows * ldp;
  const int64_t bh = blockIdx.x / p.nchunk, N = p.N;
  const int chunk = (int)(blockIdx.x - bh * p.nchunk);
  const int64_t rb = chunk * p.rows_per_chunk;
  const int64_t re = min(N, rb + p.rows_per_chunk);
  const T* qq = (const T*)p.q + bh * N * D;
  const T* gg = (const T*)p.dO + bh * N * D;
  const float* lse1 = p.lse1 + bh * N;
  load_small(Kt, ldk, p.kt + bh * m * D, m, mpad, D);
  load_small(St, ldk, p.step2 + bh * m * D, m, mpad, D);
  float accA[8][8], accB[8][8];
  zero(accA);
  zero(accB);
  __syncthreads();
  for (int64_t r0 = rb; r0 < re; r0 += kTileRows) {
    load_tile<T>(Xs, D, qq, r0, re, D, p.scale);
    load_tile<T>(Gs, D, gg, r0, re, D, 1.f);
    __syncthreads();
    softmax1_bwd_tile(Xs, Gs, Kt, St, Ps, dSs, lse1, r0, re, D, m, mj, ldk, ldp, true);
    __syncthreads();
    bgemm<8, 8>(accA, mj, dj, kTileRows,
                [&](int i, int k) { return Ps[k * ldp + ty + 16 * i]; },
                [&](int k, int j) { return Gs[k * D + tx + 16 * j]; });
    bgemm<8, 8>(accB, mj, dj, kTileRows,
                [&](int i, int k) { return dSs[k * ldp + ty + 16 * i]; },
                [&](int k, int j) { return Xs[k * D + tx + 16 * j]; });
    __syncthreads();
  }
  float* pa = p.partA + ((size_t)bh * p.nchunk + chunk) * 2 * m * D;
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int l = ty + 16 * i, d = tx + 16 * j;
      if (i < mj && j < dj && l < m) {
        pa[l * D + d] = accA[i][j];
        pa[m * D + l * D + d] = accB[i][j];
      }
    }
}

// ------------------------------------------------------------------------------------------
// Backward pass C: dQ = s (dS1 Kt + dQt_tot[l(n)] / len_l), written once.
template <class T>
__global__ void __launch_bounds__(kThreads, 1) gen_bwd_c_kernel(StreamParams p) {
  extern __shared__ float smem[];
  const int D = p.D, m = p.m, mpad = p.mpad, t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const int mj = mpad >> 4, dj = D >> 4;
  const int ldk = D + 1, ldp = mpad + 1;
  float* Kt = smem;
  float* St = Kt + mpad * ldk;
  float* Xs = St + mpad * ldk;
  float* Gs = Xs + kTileRows * D;
  float* Ps = Gs + kTileRows * D;
  float* dSs = Ps + kTileRows * ldp;
  const int64_t bh = blockIdx.x / p.nchunk, N = p.N;
  const int chunk = (int)(blockIdx.x - bh * p.nchunk);
  const int64_t rb = chunk * p.rows_per_chunk;
  const int64_t re = min(N, rb + p.rows_per_chunk);
  const T* qq = (const T*)p.q + bh * N * D;
  const T* gg = (const T*)p.dO + bh * N * D;
  T* dq = (T*)p.dq + bh * N * D;
  const float* lse1 = p.lse1 + bh * N;
  const float* dqt = p.dqt_tot + bh * m * D;
  Segments sg(p.seg_N, m);
  load_small(Kt, ldk, p.kt + bh * m * D, m, mpad, D);
  load_small(St, ldk, p.step2 + bh * m * D, m, mpad, D);
  __syncthreads();
  for (int64_t r0 = rb; r0 < re; r0 += kTileRows) {
    load_tile<T>(Xs, D, qq, r0, re, D, p.scale);
    load_tile<T>(Gs, D, gg, r0, re, D, 1.f);
    __syncthreads();
    softmax1_bwd_tile(Xs, Gs, Kt, St, Ps, dSs, lse1, r0, re, D, m, mj, ldk, ldp, false);
    __syncthreads();
    float o[2][8];
    zero(o);
    bgemm<2, 8>(o, 2, dj, m,
                [&](int i, int k) { return dSs[(ty + 16 * i) * ldp + k]; },
                [&](int k, int j) { return Kt[k * ldk + tx + 16 * j]; });
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      int64_t row = r0 + ty + 16 * i;
      if (row < re) {
        int l = sg.landmark_of(p.row_offset + row);
        float inv = 1.f / (float)sg.len(l);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < dj) {
            int d = tx + 16 * j;
            dq[row * D + d] = from_f<T>(p.scale * (o[i][j] + dqt[l * D + d] * inv));
          }
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------
// Backward pass B: dV = P3^T dO3, dK = s (dS3^T Qt + dKt_tot[l(n)] / len_l), both written
// once, and per-chunk partials of dQt = dS3 (sK).
template <class T>
__global__ void __launch_bounds__(kThreads, 1) gen_bwd_b_kernel(StreamParams p) {
  extern __shared__ float smem[];
  const int D = p.D, m = p.m, mpad = p.mpad, t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const int mj = mpad >> 4, dj = D >> 4;
  const int ldk = D + 1, ldp = mpad + 1;
  float* Qt = smem;
  float* Gt = Qt + mpad * ldk;
  float* Ks = Gt + mpad * ldk;
  float* Vs = Ks + kTileRows * D;
  float* Ps = Vs + kTileRows * D;
  float* dSs = Ps + kTileRows * ldp;
  const int64_t bh = blockIdx.x / p.nchunk, N = p.N;
  const int chunk = (int)(blockIdx.x - bh * p.nchunk);
  const int64_t rb = chunk * p.rows_per_chunk;
  const int64_t re = min(N, rb + p.rows_per_chunk);
  const T* kk = (const T*)p.k + bh * N * D;
  const T* vv = (const T*)p.v + bh * N * D;
  T* dk = (T*)p.dk + bh * N * D;
  T* dv = (T*)p.dv + bh * N * D;
  const float* dkt = p.dkt_tot + bh * m * D;
  Segments sg(p.seg_N, m);
  load_small(Qt, ldk, p.qt + bh * m * D, m, mpad, D);
  load_small(Gt, ldk, p.dO3 + bh * m * D, m, mpad, D);
  float lse3[8], d3[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int l = tx + 16 * j;
    lse3[j] = (l < m) ? p.lse3[bh * m + l] : 0.f;
    d3[j] = (l < m) ? p.D3[bh * m + l] : 0.f;
  }
  float acc[8][8];
  zero(acc);
  __syncthreads();
  for (int64_t r0 = rb; r0 < re; r0 += kTileRows) {
    load_tile<T>(Ks, D, kk, r0, re, D, p.scale);
    load_tile<T>(Vs, D, vv, r0, re, D, 1.f);
    __syncthreads();
    {
      float s[2][8], g[2][8];
      zero(s);
      zero(g);
      bgemm<2, 8>(s, 2, mj, D,
                  [&](int i, int k) { return Ks[(ty + 16 * i) * D + k]; },
                  [&](int k, int j) { return Qt[(tx + 16 * j) * ldk + k]; });
      bgemm<2, 8>(g, 2, mj, D,
                  [&](int i, int k) { return Vs[(ty + 16 * i) * D + k]; },
                  [&](int k, int j) { return Gt[(tx + 16 * j) * ldk + k]; });
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        bool ok = r0 + ty + 16 * i < re;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j < mj) {
            float pv = (ok && tx + 16 * j < m) ? expf(s[i][j] - lse3[j]) : 0.f;
            Ps[(ty + 16 * i) * ldp + tx + 16 * j] = pv;
            dSs[(ty + 16 * i) * ldp + tx + 16 * j] = pv * (g[i][j] - d3[j]);
          }
        }
      }
    }
    __syncthreads();
    {
      float o[2][8];
      zero(o);
      bgemm<2, 8>(o, 2, dj, m,
                  [&](int i, int k) { return Ps[(ty + 16 * i) * ldp + k]; },
                  [&](int k, int j) { return Gt[k * ldk + tx + 16 * j]; });
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        int64_t row = r0 + ty + 16 * i;
        if (row < re) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < dj) dv[row * D + tx + 16 * j] = from_f<T>(o[i][j]);
        }
      }
      zero(o);
      bgemm<2, 8>(o, 2, dj, m,
                  [&](int i, int k) { return dSs[(ty + 16 * i) * ldp + k]; },
                  [&](int k, int j) { return Qt[k * ldk + tx + 16 * j]; });
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        int64_t row = r0 + ty + 16 * i;
        if (row < re) {
          int l = sg.landmark_of(p.row_offset + row);
          float inv = 1.f / (float)sg.len(l);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < dj) {
              int d = tx + 16 * j;
              dk[row * D + d] = from_f<T>(p.scale * (o[i][j] + dkt[l * D + d] * inv));
            }
        }
      }
    }
    bgemm<8, 8>(acc, mj, dj, kTileRows,
                [&](int i, int k) { return dSs[k * ldp + ty + 16 * i]; },
                [&](int k, int j) { return Ks[k * D + tx + 16 * j]; });
    __syncthreads();
  }
  float* pb = p.partB + ((size_t)bh * p.nchunk + chunk) * m * D;
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int l = ty + 16 * i, d = tx + 16 * j;
      if (i < mj && j < dj && l < m) pb[l * D + d] = acc[i][j];
    }
}

}  // namespace fnb
