// The landmark-sized ("middle") stages: everything that works on (m x m) and (m x D) FP32
// matrices per (b,h) slice.  One CTA of 256 threads per slice; operands live in global
// memory (they are a few hundred KB per slice and stay in L2) and are staged through shared
// memory k-slab by k-slab, so the same code serves every m <= 128.
//
//   mid_fwd_kernel     : landmark finalisation, softmax-2, optional Tikhonov ridge,
//                        Z0 and the J Newton-Schulz iterations (all iterates saved)
//   combine_kernel     : merges the per-chunk softmax-3 partials, then step2 = K2inv * Bmat
//   mid_bwd_kernel     : reduces the softmax-1 side partials, dO3 / dK2inv / D3, the exact
//                        backward through every Newton-Schulz iterate, the Z0 norms, the ridge
//                        wrap and the softmax-2 Jacobian
//   dqt_reduce_kernel  : final landmark gradient of Q
#pragma once
#include "common.cuh"
#include "small_kernels.cuh"

namespace fnb {

constexpr int kGemmKT = 16;            // k-slab depth
constexpr int kGemmLd = kMaxM + 4;     // shared row stride of a slab
constexpr int kGemmSmemFloats = 2 * kGemmKT * kGemmLd;

// C(MxN) = alpha * op(A) * op(B) + beta * C + diag * I,  M, N <= 128, any K.
//   TA == false: A is (M x K) row-major with leading dimension lda;  TA == true: A is (K x M).
//   TB == false: B is (K x N) row-major with leading dimension ldb;  TB == true: B is (N x K).
// C may alias A or B.  All 256 threads must call; ends with a barrier.
// Pointers are deliberately not __restrict__: operands are produced by this same CTA and must
// be read through the coherent path.
template <bool TA, bool TB>
__device__ __noinline__ void cta_gemm(float* C, int ldc, const float* A, int lda, const float* B, int ldb,
                         int M, int N, int K, float alpha, float beta, float diag, float* sm) {
  float* As = sm;
  float* Bs = sm + kGemmKT * kGemmLd;
  const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const int MI = (M + 15) >> 4, NJ = (N + 15) >> 4;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kGemmKT) {
    // stage A slab: As[kk][r] = op(A)(r, k0+kk)
    for (int idx = t; idx < kGemmKT * 16 * MI; idx += kThreads) {
      int kk, r;
      if (TA) { r = idx % (16 * MI); kk = idx / (16 * MI); }
      else    { kk = idx % kGemmKT;  r = idx / kGemmKT; }
      float x = 0.f;
      if (r < M && k0 + kk < K) x = TA ? A[(size_t)(k0 + kk) * lda + r] : A[(size_t)r * lda + k0 + kk];
      As[kk * kGemmLd + r] = x;
    }
    for (int idx = t; idx < kGemmKT * 16 * NJ; idx += kThreads) {
      int kk, c;
      if (TB) { kk = idx % kGemmKT;  c = idx / kGemmKT; }
      else    { c = idx % (16 * NJ); kk = idx / (16 * NJ); }
      float x = 0.f;
      if (c < N && k0 + kk < K) x = TB ? B[(size_t)c * ldb + k0 + kk] : B[(size_t)(k0 + kk) * ldb + c];
      Bs[kk * kGemmLd + c] = x;
    }
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < kGemmKT; ++kk) {
      float a[8], b[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = (i < MI) ? As[kk * kGemmLd + ty + 16 * i] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) b[j] = (j < NJ) ? Bs[kk * kGemmLd + tx + 16 * j] : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (i < MI) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < NJ) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int r = ty + 16 * i, c = tx + 16 * j;
      if (i < MI && j < NJ && r < M && c < N) {
        float val = alpha * acc[i][j];
        if (beta != 0.f) val += beta * C[(size_t)r * ldc + c];
        if (r == c) val += diag;
        C[(size_t)r * ldc + c] = val;
      }
    }
  }
  __syncthreads();
}

// ||A||_1 (max column abs-sum), ||A||_inf (max row abs-sum) and their first-occurrence
// argmax positions, for an (m x m) matrix in global memory.  red: >= 2*m floats of smem.
// Results are broadcast through red[0..3] and returned in registers by every thread.
struct Norms { float n1, ninf; int jc, ir; };
__device__ inline Norms cta_norms(const float* A, int m, float* red) {
  const int t = threadIdx.x;
  if (t < m) {
    float cs = 0.f;
    for (int i = 0; i < m; ++i) cs += fabsf(A[i * m + t]);
    red[t] = cs;
  } else if (t >= 128 && t - 128 < m) {
    int i = t - 128;
    float rs = 0.f;
    for (int j = 0; j < m; ++j) rs += fabsf(A[i * m + j]);
    red[kMaxM + i] = rs;
  }
  __syncthreads();
  __shared__ float out_n1, out_ninf;
  __shared__ int out_jc, out_ir;
  if (t == 0) {
    float best = red[0]; int bi = 0;
    for (int j = 1; j < m; ++j) if (red[j] > best) { best = red[j]; bi = j; }
    out_n1 = best; out_jc = bi;
  } else if (t == 32) {
    float best = red[kMaxM]; int bi = 0;
    for (int i = 1; i < m; ++i) if (red[kMaxM + i] > best) { best = red[kMaxM + i]; bi = i; }
    out_ninf = best; out_ir = bi;
  }
  __syncthreads();
  Norms r{out_n1, out_ninf, out_jc, out_ir};
  __syncthreads();
  return r;
}

// dst = a*X + diag*I   (m x m, elementwise)
__device__ inline void cta_affine(float* dst, const float* X, float a, float diag, int m) {
  for (int idx = threadIdx.x; idx < m * m; idx += kThreads) {
    int r = idx / m, c = idx - r * m;
    dst[idx] = a * X[idx] + (r == c ? diag : 0.f);
  }
  __syncthreads();
}

// Scratch layout (floats) for the pseudoinverse forward: 4 (m x m) buffers.
constexpr int kPinvFwdBufs = 4;
// Newton-Schulz pseudoinverse of the softmax matrix k2 (optionally ridge-regularised through
// the normal equations).  Every iterate Z_0..Z_J is stored; k2inv = Z_J or Z_J * k2^T.
__device__ inline void pinv_forward(const float* k2, float* iterates, float* k2inv,
                                    float* scratch, int m, int J, float kappa, float* sm) {
  const int mm = m * m;
  float* Ab = scratch;            // ridge matrix (only with kappa > 0)
  float* Mb = scratch + mm;
  float* Ub = scratch + 2 * mm;
  float* Vb = scratch + 3 * mm;
  float* red = sm;                // norms use the first 2*kMaxM floats of the gemm staging area
  const float* A = k2;
  if (kappa > 0.f) {
    Norms nk = cta_norms(k2, m, red);
    float lam = nk.n1 * nk.ninf / kappa;
    cta_gemm<true, false>(Ab, m, k2, m, k2, m, m, m, m, 1.f, 0.f, lam, sm);
    A = Ab;
  }
  Norms na = cta_norms(A, m, red);
  const float c = fmaxf(na.n1 * na.ninf, 1e-12f);
  for (int idx = threadIdx.x; idx < mm; idx += kThreads) {
    int r = idx / m, cc = idx - r * m;
    iterates[idx] = A[cc * m + r] / c;
  }
  __syncthreads();
  for (int j = 0; j < J; ++j) {
    const float* Z = iterates + (size_t)j * mm;
    float* Zn = iterates + (size_t)(j + 1) * mm;
    cta_gemm<false, false>(Mb, m, A, m, Z, m, m, m, m, 1.f, 0.f, 0.f, sm);        // M = A Z
    cta_affine(Ub, Mb, -1.f, 7.f, m);                                             // U = 7I - M
    cta_gemm<false, false>(Vb, m, Mb, m, Ub, m, m, m, m, -1.f, 0.f, 15.f, sm);    // V = 15I - M U
    cta_gemm<false, false>(Ub, m, Mb, m, Vb, m, m, m, m, -1.f, 0.f, 13.f, sm);    // T = 13I - M V
    cta_gemm<false, false>(Zn, m, Z, m, Ub, m, m, m, m, 0.25f, 0.f, 0.f, sm);     // Z' = Z T / 4
  }
  const float* ZJ = iterates + (size_t)J * mm;
  if (kappa > 0.f) {
    cta_gemm<false, true>(k2inv, m, ZJ, m, k2, m, m, m, m, 1.f, 0.f, 0.f, sm);
  } else {
    for (int idx = threadIdx.x; idx < mm; idx += kThreads) k2inv[idx] = ZJ[idx];
    __syncthreads();
  }
}

// Scratch layout for the pseudoinverse backward: 12 (m x m) buffers.
constexpr int kPinvBwdBufs = 12;
// Gradient of the pseudoinverse w.r.t. the softmax matrix k2 (lambda detached).
//   G = dL/d k2inv  ->  dK2 = dL/d k2.
__device__ inline void pinv_backward(const float* k2, const float* iterates, const float* G,
                                     float* dK2, float* scratch, int m, int J, float kappa,
                                     float* sm) {
  const int mm = m * m;
  float* Ab = scratch;
  float* Mb = scratch + 1 * mm;
  float* Ub = scratch + 2 * mm;
  float* Vb = scratch + 3 * mm;
  float* Tb = scratch + 4 * mm;
  float* dZ = scratch + 5 * mm;
  float* dZo = scratch + 6 * mm;
  float* dT = scratch + 7 * mm;
  float* dV = scratch + 8 * mm;
  float* dM = scratch + 9 * mm;
  float* dA = scratch + 10 * mm;
  float* dK2a = scratch + 11 * mm;
  float* red = sm;
  const float* A = k2;
  const float* ZJ = iterates + (size_t)J * mm;
  if (kappa > 0.f) {
    Norms nk = cta_norms(k2, m, red);
    float lam = nk.n1 * nk.ninf / kappa;
    cta_gemm<true, false>(Ab, m, k2, m, k2, m, m, m, m, 1.f, 0.f, lam, sm);
    A = Ab;
    cta_gemm<true, false>(dK2a, m, G, m, ZJ, m, m, m, m, 1.f, 0.f, 0.f, sm);   // G^T Z_J
    cta_gemm<false, false>(dZ, m, G, m, k2, m, m, m, m, 1.f, 0.f, 0.f, sm);    // G K2
  } else {
    for (int idx = threadIdx.x; idx < mm; idx += kThreads) dZ[idx] = G[idx];
  }
  for (int idx = threadIdx.x; idx < mm; idx += kThreads) dA[idx] = 0.f;
  __syncthreads();

  for (int j = J - 1; j >= 0; --j) {
    const float* Z = iterates + (size_t)j * mm;
    cta_gemm<false, false>(Mb, m, A, m, Z, m, m, m, m, 1.f, 0.f, 0.f, sm);
    cta_affine(Ub, Mb, -1.f, 7.f, m);
    cta_gemm<false, false>(Vb, m, Mb, m, Ub, m, m, m, m, -1.f, 0.f, 15.f, sm);
    cta_gemm<false, false>(Tb, m, Mb, m, Vb, m, m, m, m, -1.f, 0.f, 13.f, sm);
    cta_gemm<true, false>(dT, m, Z, m, dZ, m, m, m, m, 0.25f, 0.f, 0.f, sm);    // dT = Z^T dZ / 4
    cta_gemm<false, true>(dZo, m, dZ, m, Tb, m, m, m, m, 0.25f, 0.f, 0.f, sm);  // dZ T^T / 4
    cta_gemm<false, true>(dM, m, dT, m, Vb, m, m, m, m, -1.f, 0.f, 0.f, sm);    // -dT V^T
    cta_gemm<true, false>(dV, m, Mb, m, dT, m, m, m, m, -1.f, 0.f, 0.f, sm);    // dV = -M^T dT
    cta_gemm<false, true>(dM, m, dV, m, Ub, m, m, m, m, -1.f, 1.f, 0.f, sm);    // -= dV U^T
    cta_gemm<true, false>(dM, m, Mb, m, dV, m, m, m, m, 1.f, 1.f, 0.f, sm);     // += M^T dV
    cta_gemm<false, true>(dA, m, dM, m, Z, m, m, m, m, 1.f, 1.f, 0.f, sm);      // dA += dM Z^T
    cta_gemm<true, false>(dZ, m, A, m, dM, m, m, m, m, 1.f, 0.f, 0.f, sm);      // A^T dM
    for (int idx = threadIdx.x; idx < mm; idx += kThreads) dZ[idx] += dZo[idx];
    __syncthreads();
  }
  // Z0 = A^T / c with c = ||A||_1 ||A||_inf
  Norms na = cta_norms(A, m, red);
  const float craw = na.n1 * na.ninf;
  const float c = fmaxf(craw, 1e-12f);
  // S = sum_{a,b} dZ0[a,b] A[b,a]
  float part = 0.f;
  for (int idx = threadIdx.x; idx < mm; idx += kThreads) {
    int a = idx / m, b = idx - a * m;
    part += dZ[idx] * A[b * m + a];
  }
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
  __syncthreads();
  float S = 0.f;
  for (int w = 0; w < kThreads / 32; ++w) S += red[w];
  __syncthreads();
  const bool clamped = !(craw > 1e-12f);
  const float col_term = clamped ? 0.f : -S * na.ninf / (c * c);
  const float row_term = clamped ? 0.f : -S * na.n1 / (c * c);
  for (int idx = threadIdx.x; idx < mm; idx += kThreads) {
    int r = idx / m, cc = idx - r * m;
    float a = A[idx];
    float sg = a > 0.f ? 1.f : (a < 0.f ? -1.f : 0.f);
    float g = dA[idx] + dZ[cc * m + r] / c;
    if (cc == na.jc) g += sg * col_term;
    if (r == na.ir) g += sg * row_term;
    dA[idx] = g;
  }
  __syncthreads();
  if (kappa > 0.f) {
    // dK2 = dK2a + K2 (dA + dA^T)
    for (int idx = threadIdx.x; idx < mm; idx += kThreads) {
      int r = idx / m, cc = idx - r * m;
      dM[idx] = dA[idx] + dA[cc * m + r];
    }
    __syncthreads();
    cta_gemm<false, false>(dK2a, m, k2, m, dM, m, m, m, m, 1.f, 1.f, 0.f, sm);
    for (int idx = threadIdx.x; idx < mm; idx += kThreads) dK2[idx] = dK2a[idx];
  } else {
    for (int idx = threadIdx.x; idx < mm; idx += kThreads) dK2[idx] = dA[idx];
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------
struct MidFwdParams {
  const float* land_partial;  // [2][BH][m][C][D] raw segment sums (not scaled)
  int C;
  float* qt; float* kt;       // [BH][m][D]
  float* k2; float* lse2; float* iterates; float* k2inv;
  float* scratch;             // [BH][kPinvFwdBufs][m][m]
  int64_t BH, N;
  int m, D, J;
  float kappa, scale;
  int landmarks_only;         // 1: stop after writing qt / kt (the shared-memory NS kernel follows)
  void* qt16;                 // optional [BH][MP][D] 16-bit copy of qt16_mul * qt (tensor-core path)
  int dtype, MP;
  float qt16_mul;
};

__global__ void __launch_bounds__(kThreads) mid_fwd_kernel(MidFwdParams p) {
  __shared__ float sm[kGemmSmemFloats];
  const int64_t bh = blockIdx.x;
  const int m = p.m, D = p.D, t = threadIdx.x;
  Segments sg(p.N, m);
  float* qt = p.qt + bh * m * D;
  float* kt = p.kt + bh * m * D;
  for (int idx = t; idx < 2 * m * D; idx += kThreads) {
    int which = idx / (m * D), rem = idx - which * m * D;
    int l = rem / D, d = rem - l * D;
    const float* src = p.land_partial + ((((size_t)which * p.BH + bh) * m + l) * p.C) * D + d;
    float s = 0.f;
    for (int c = 0; c < p.C; ++c) s += src[(size_t)c * D];
    float val = s * (p.scale / (float)sg.len(l));
    (which ? kt : qt)[rem] = val;
  }
  __syncthreads();
  if (p.qt16)
    pack_pair(qt, reinterpret_cast<char*>(p.qt16) + (size_t)bh * p.MP * D * 2, nullptr, p.dtype, m, D, p.MP,
              p.qt16_mul);
  if (p.landmarks_only) return;
  float* k2 = p.k2 + bh * m * m;
  cta_gemm<false, true>(k2, m, qt, D, kt, D, m, m, D, 1.f, 0.f, 0.f, sm);
  // row softmax, one warp per row
  const int w = t >> 5, lane = t & 31;
  for (int r = w; r < m; r += kThreads / 32) {
    float mx = -INFINITY;
    for (int c = lane; c < m; c += 32) mx = fmaxf(mx, k2[r * m + c]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int c = lane; c < m; c += 32) sum += expf(k2[r * m + c] - mx);
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    for (int c = lane; c < m; c += 32) k2[r * m + c] = expf(k2[r * m + c] - mx) / sum;
    if (lane == 0) p.lse2[bh * m + r] = mx + logf(sum);
  }
  __syncthreads();
  pinv_forward(k2, p.iterates + bh * (size_t)(p.J + 1) * m * m, p.k2inv + bh * m * m,
               p.scratch + bh * (size_t)kPinvFwdBufs * m * m, m, p.J, p.kappa, sm);
}

__global__ void __launch_bounds__(kThreads)
pinv_fwd_debug_kernel(const float* k2, float* iterates, float* k2inv, float* scratch, int m,
                      int J, float kappa) {
  __shared__ float sm[kGemmSmemFloats];
  const int64_t bh = blockIdx.x;
  pinv_forward(k2 + bh * m * m, iterates + bh * (size_t)(J + 1) * m * m, k2inv + bh * m * m,
               scratch + bh * (size_t)kPinvFwdBufs * m * m, m, J, kappa, sm);
}

__global__ void __launch_bounds__(kThreads)
pinv_bwd_debug_kernel(const float* k2, const float* iterates, const float* G, float* dK2,
                      float* scratch, int m, int J, float kappa) {
  __shared__ float sm[kGemmSmemFloats];
  const int64_t bh = blockIdx.x;
  pinv_backward(k2 + bh * m * m, iterates + bh * (size_t)(J + 1) * m * m, G + bh * m * m,
                dK2 + bh * m * m, scratch + bh * (size_t)kPinvBwdBufs * m * m, m, J, kappa, sm);
}

// ------------------------------------------------------------------------------------------
// Softmax-3 partials: per (bh, chunk) an un-normalised accumulator acc[m][D] with its running
// maximum and running sum per landmark row.
struct CombineParams {
  const float* part_acc;   // [BH][nchunk][m][D]
  const float* part_max;   // [BH][nchunk][m]
  const float* part_sum;   // [BH][nchunk][m]
  int nchunk;
  const float* k2inv;      // [BH][m][m]
  float* bmat; float* lse3; float* step2;
  int m, D;
};

__global__ void __launch_bounds__(kThreads) combine_kernel(CombineParams p) {
  __shared__ float sm[kGemmSmemFloats];
  __shared__ float gmax[kMaxM], gsum[kMaxM];
  constexpr int kBatch = 16;
  __shared__ float wts[kBatch][kMaxM];
  const int64_t bh = blockIdx.x;
  const int m = p.m, D = p.D, t = threadIdx.x, nc = p.nchunk;
  const float* pmax = p.part_max + bh * nc * m;
  const float* psum = p.part_sum + bh * nc * m;
  const float* pacc = p.part_acc + bh * (size_t)nc * m * D;
  if (t < m) {
    float M = -INFINITY;
    for (int c = 0; c < nc; ++c) M = fmaxf(M, pmax[c * m + t]);
    float L = 0.f;
    for (int c = 0; c < nc; ++c) L += expf(pmax[c * m + t] - M) * psum[c * m + t];
    gmax[t] = M; gsum[t] = L;
    p.lse3[bh * m + t] = M + logf(L);
  }
  __syncthreads();
  // each thread owns elements idx = t + 256*e of the (m x D) result
  constexpr int kMaxPer = kMaxM * kMaxD / kThreads;  // 64
  float acc[kMaxPer];
#pragma unroll
  for (int e = 0; e < kMaxPer; ++e) acc[e] = 0.f;
  const int total = m * D;
  for (int c0 = 0; c0 < nc; c0 += kBatch) {
    for (int idx = t; idx < kBatch * m; idx += kThreads) {
      int cc = idx / m, l = idx - cc * m;
      wts[cc][l] = (c0 + cc < nc) ? expf(pmax[(c0 + cc) * m + l] - gmax[l]) : 0.f;
    }
    __syncthreads();
    int cend = min(kBatch, nc - c0);
    for (int cc = 0; cc < cend; ++cc) {
      const float* src = pacc + (size_t)(c0 + cc) * total;
#pragma unroll
      for (int e = 0; e < kMaxPer; ++e) {
        int idx = t + e * kThreads;
        if (idx < total) acc[e] = fmaf(wts[cc][idx / D], src[idx], acc[e]);
      }
    }
    __syncthreads();
  }
  float* bmat = p.bmat + bh * (size_t)total;
#pragma unroll
  for (int e = 0; e < kMaxPer; ++e) {
    int idx = t + e * kThreads;
    if (idx < total) bmat[idx] = acc[e] / gsum[idx / D];
  }
  __syncthreads();
  cta_gemm<false, false>(p.step2 + bh * (size_t)total, D, p.k2inv + bh * m * m, m, bmat, D, m, D, m,
                         1.f, 0.f, 0.f, sm);
}

// ------------------------------------------------------------------------------------------
struct MidBwdParams {
  const float* partA;        // [BH][nchunk][2][m][D]: dstep2 and dKt partials of the row pass
  int nchunk;
  const float* qt; const float* kt; const float* k2; const float* iterates;
  const float* k2inv; const float* bmat;
  float* dstep2;             // [BH][m][D] scratch
  float* dkt_a;              // [BH][m][D] scratch
  float* dO3;                // [BH][m][D] out
  float* D3;                 // [BH][m]    out
  float* dqt_ns;             // [BH][m][D] out
  float* dkt_tot;            // [BH][m][D] out
  float* G;                  // [BH][m][m] scratch (dK2inv)
  float* dK2;                // [BH][m][m] scratch
  float* scratch;            // [BH][kPinvBwdBufs][m][m]
  int m, D, J;
  float kappa;
  int first_half_only;       // 1: stop after dO3 / dK2inv / D3 (the shared-memory NS kernel follows)
};

__global__ void __launch_bounds__(kThreads) mid_bwd_kernel(MidBwdParams p) {
  __shared__ float sm[kGemmSmemFloats];
  const int64_t bh = blockIdx.x;
  const int m = p.m, D = p.D, t = threadIdx.x, mm = m * m, md = m * D;
  float* dstep2 = p.dstep2 + bh * md;
  float* dkt_a = p.dkt_a + bh * md;
  const float* partA = p.partA + bh * (size_t)p.nchunk * 2 * md;
  for (int idx = t; idx < 2 * md; idx += kThreads) {
    float s = 0.f;
    for (int c = 0; c < p.nchunk; ++c) s += partA[(size_t)c * 2 * md + idx];
    if (idx < md) dstep2[idx] = s; else dkt_a[idx - md] = s;
  }
  __syncthreads();
  const float* k2inv = p.k2inv + bh * mm;
  const float* bmat = p.bmat + bh * md;
  const float* k2 = p.k2 + bh * mm;
  const float* qt = p.qt + bh * md;
  const float* kt = p.kt + bh * md;
  float* dO3 = p.dO3 + bh * md;
  float* G = p.G + bh * mm;
  float* dK2 = p.dK2 + bh * mm;
  cta_gemm<true, false>(dO3, D, k2inv, m, dstep2, D, m, D, m, 1.f, 0.f, 0.f, sm);   // K2inv^T dstep2
  cta_gemm<false, true>(G, m, dstep2, D, bmat, D, m, m, D, 1.f, 0.f, 0.f, sm);      // dstep2 Bmat^T
  {
    const int w = t >> 5, lane = t & 31;
    for (int l = w; l < m; l += kThreads / 32) {
      float s = 0.f;
      for (int d = lane; d < D; d += 32) s += bmat[l * D + d] * dO3[l * D + d];
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) p.D3[bh * m + l] = s;
    }
  }
  if (p.first_half_only) return;
  pinv_backward(k2, p.iterates + bh * (size_t)(p.J + 1) * mm, G, dK2,
                p.scratch + bh * (size_t)kPinvBwdBufs * mm, m, p.J, p.kappa, sm);
  // softmax-2 Jacobian, in place: dS2 = K2 o (dK2 - rowsum(dK2 o K2))
  {
    const int w = t >> 5, lane = t & 31;
    for (int r = w; r < m; r += kThreads / 32) {
      float s = 0.f;
      for (int c = lane; c < m; c += 32) s += dK2[r * m + c] * k2[r * m + c];
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      for (int c = lane; c < m; c += 32) dK2[r * m + c] = k2[r * m + c] * (dK2[r * m + c] - s);
    }
  }
  __syncthreads();
  float* dqt_ns = p.dqt_ns + bh * md;
  float* dkt_tot = p.dkt_tot + bh * md;
  cta_gemm<false, false>(dqt_ns, D, dK2, m, kt, D, m, D, m, 1.f, 0.f, 0.f, sm);      // dS2 Kt
  for (int idx = t; idx < md; idx += kThreads) dkt_tot[idx] = dkt_a[idx];
  __syncthreads();
  cta_gemm<true, false>(dkt_tot, D, dK2, m, qt, D, m, D, m, 1.f, 1.f, 0.f, sm);      // += dS2^T Qt
}

// dqt_tot = dqt_ns + sum over chunks of the column-pass partials
__global__ void __launch_bounds__(kThreads)
dqt_reduce_kernel(const float* partB, int nchunk, const float* dqt_ns, float* dqt_tot, int md) {
  const int64_t bh = blockIdx.x;
  for (int idx = threadIdx.x; idx < md; idx += kThreads) {
    const float* src = partB + bh * (size_t)nchunk * md + idx;
    float s = dqt_ns[bh * md + idx];
    for (int c = 0; c < nchunk; ++c) s += src[(size_t)c * md];
    dqt_tot[bh * md + idx] = s;
  }
}

}  // namespace fnb
