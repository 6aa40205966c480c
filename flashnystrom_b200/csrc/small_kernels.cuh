// Landmark-sized glue between the streaming passes, one CTA of 256 threads per (b,h) slice,
// row-parallel: 4 threads share one landmark row and each owns D/4 consecutive columns, so the
// reductions over per-CTA partials are coalesced float4 streams and need no index division.
//
//   combine2_kernel  : merge softmax-3 partials -> Bmat, lse3; step2 = K2inv Bmat; 16-bit operand
//                      copies for the forward output pass
//   bwd_mid1_kernel  : reduce softmax-1 side partials -> dstep2, dKt_a; dO3 = K2inv^T dstep2;
//                      dK2inv = dstep2 Bmat^T; D3; 16-bit operand copies for the column pass
//   pack_bwd_ac_kernel : 16-bit operand copies for the backward row passes
#pragma once
#include "common.cuh"

namespace fnb {

__device__ __forceinline__ void store16(void* p, int dtype, size_t idx, float v) {
  if (dtype == 1) reinterpret_cast<__half*>(p)[idx] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(p)[idx] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ uint32_t pack2x16(int dtype, float a, float b) {
  if (dtype == 1) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// max over the CTA; red: 8 floats of shared scratch.  Ends with a barrier.
__device__ __forceinline__ float cta_max(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
  for (int w = 1; w < kThreads / 32; ++w) r = fmaxf(r, red[w]);
  return r;
}
// power of two >= amax (exact scale), 1 for a zero / non-finite matrix
__device__ __forceinline__ float pow2_scale(float amax) {
  int e = 0;
  if (amax > 0.f && isfinite(amax)) frexpf(amax, &e);
  e = max(-100, min(100, e));
  return ldexpf(1.f, e);
}

// 16-bit copies of an FP32 (m x D) global matrix: out_n[MP][D] and / or out_t[D][MP], times mul.
__device__ __forceinline__ void pack_pair(const float* src, void* out_n, void* out_t, int dtype, int m, int D,
                                          int MP, float mul) {
  if (out_n)   // four consecutive columns per step (D is a multiple of 16, the matrices are 16-byte aligned)
    for (int g = threadIdx.x; g < MP * D / 4; g += (int)blockDim.x) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if ((g * 4) / D < m) x = reinterpret_cast<const float4*>(src)[g];
      reinterpret_cast<uint2*>(out_n)[g] = make_uint2(pack2x16(dtype, x.x * mul, x.y * mul), pack2x16(dtype, x.z * mul, x.w * mul));
    }
  if (out_t)
    for (int idx = threadIdx.x; idx < D * MP; idx += kThreads) {
      int d = idx / MP, l = idx - d * MP;
      store16(out_t, dtype, idx, l < m ? src[l * D + d] * mul : 0.f);
    }
}

struct Combine2Params {
  const float* part_acc; const float* part_max; const float* part_sum;  // [BH][nchunk][m][D], [..][m]
  int nchunk;
  const float* k2inv;         // [BH][m][m]
  const float* k_landmarks;   // [BH][m][D]
  float* bmat; float* lse3; float* step2;
  int m, D;
  // operand copies (skipped when dtype == 0)
  int dtype, MP;
  void* kt16;                 // [BH][MP][D]  = kt_mul * Kt
  void* st16T;                // [BH][D][MP]  = step2^T / st_scale
  float* st_scale;            // [BH]
  float kt_mul;
  // element strides between slices and between chunks of the partial arrays (acc_*: the m x D
  // accumulators, vec_*: the per-landmark max / sum vectors); lets the kernel read partials gathered from ranks
  int64_t acc_bh_stride, acc_chunk_stride, vec_bh_stride, vec_chunk_stride;
  // partial_only: write the merged, still un-normalised partial (acc, max, sum) of this rank
  // into out_acc [BH][m][D], out_max / out_sum [BH][m] and stop
  int partial_only;
  float* out_acc; float* out_max; float* out_sum;
};

template <int NV>
__global__ void __launch_bounds__(kThreads) combine2_kernel(Combine2Params p) {
  extern __shared__ float sm[];            // bmat then step2: [m][D]
  __shared__ float red[8];
  const int64_t bh = blockIdx.x;
  const int m = p.m, D = p.D, t = threadIdx.x, nc = p.nchunk;
  constexpr int nv = NV;                      // float4 per thread per row: D = 16 * NV
  constexpr int CB = NV <= 2 ? 8 : (NV == 4 ? 4 : 2);   // chunks whose loads are in flight together
  const int q = t & 3, dpt = D >> 2, d0 = q * dpt;
  const int64_t cs = p.acc_chunk_stride, csv = p.vec_chunk_stride;
  const float* pmax = p.part_max + bh * p.vec_bh_stride;
  const float* psum = p.part_sum + bh * p.vec_bh_stride;
  const float* pacc = p.part_acc + bh * p.acc_bh_stride;
  for (int l = t >> 2; l < m; l += kThreads / 4) {
    float M = -INFINITY;
    for (int c0 = 0; c0 < nc; c0 += 8) {
      float pm[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) pm[i] = (c0 + i < nc) ? pmax[(c0 + i) * csv + l] : -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) M = fmaxf(M, pm[i]);
    }
    float Lsum = 0.f;
    float4 acc[8];
#pragma unroll
    for (int v = 0; v < 8; ++v) acc[v] = make_float4(0, 0, 0, 0);
    for (int c0 = 0; c0 < nc; c0 += CB) {
      float pm[CB], ps[CB];
      float4 x[CB][NV];
#pragma unroll
      for (int i = 0; i < CB; ++i) {
        const int c = min(c0 + i, nc - 1);
        pm[i] = pmax[c * csv + l];
        ps[i] = psum[c * csv + l];
        const float4* src = reinterpret_cast<const float4*>(pacc + (size_t)c * cs + (size_t)l * D + d0);
#pragma unroll
        for (int v = 0; v < NV; ++v) x[i][v] = src[v];
      }
#pragma unroll
      for (int i = 0; i < CB; ++i) {
        const float w = (c0 + i < nc) ? expf(pm[i] - M) : 0.f;
        Lsum = fmaf(w, ps[i], Lsum);
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          acc[v].x = fmaf(w, x[i][v].x, acc[v].x); acc[v].y = fmaf(w, x[i][v].y, acc[v].y);
          acc[v].z = fmaf(w, x[i][v].z, acc[v].z); acc[v].w = fmaf(w, x[i][v].w, acc[v].w);
        }
      }
    }
    if (p.partial_only) {
      float4* dst = reinterpret_cast<float4*>(p.out_acc + (bh * m + l) * D + d0);
#pragma unroll
      for (int v = 0; v < 8; ++v) if (v < nv) dst[v] = acc[v];
      if (q == 0) { p.out_max[bh * m + l] = M; p.out_sum[bh * m + l] = Lsum; }
      continue;
    }
    const float inv = 1.f / Lsum;
    float4* dst_s = reinterpret_cast<float4*>(sm + l * D + d0);
    float4* dst_g = reinterpret_cast<float4*>(p.bmat + (bh * m + l) * D + d0);
#pragma unroll
    for (int v = 0; v < 8; ++v)
      if (v < nv) {
        const float4 x = make_float4(acc[v].x * inv, acc[v].y * inv, acc[v].z * inv, acc[v].w * inv);
        dst_s[v] = x;
        dst_g[v] = x;
      }
    if (q == 0) p.lse3[bh * m + l] = M + logf(Lsum);
  }
  if (p.partial_only) return;
  __syncthreads();
  // step2 = K2inv Bmat
  const float* k2inv = p.k2inv + bh * m * m;
  float amax = 0.f;
  float4 keep[2][8];   // step2 values of this thread's (up to two) rows, for the packed copy
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int l = (t >> 2) + pass * (kThreads / 4);
    float4 acc[8];
#pragma unroll
    for (int v = 0; v < 8; ++v) acc[v] = make_float4(0, 0, 0, 0);
    if (l < m) {
#pragma unroll 4
      for (int k = 0; k < m; ++k) {
        const float a = k2inv[l * m + k];
        const float4* b = reinterpret_cast<const float4*>(sm + k * D + d0);
#pragma unroll
        for (int v = 0; v < 8; ++v)
          if (v < nv) {
            const float4 x = b[v];
            acc[v].x = fmaf(a, x.x, acc[v].x); acc[v].y = fmaf(a, x.y, acc[v].y);
            acc[v].z = fmaf(a, x.z, acc[v].z); acc[v].w = fmaf(a, x.w, acc[v].w);
          }
      }
      float4* dst_g = reinterpret_cast<float4*>(p.step2 + (bh * m + l) * D + d0);
#pragma unroll
      for (int v = 0; v < 8; ++v)
        if (v < nv) {
          dst_g[v] = acc[v];
          amax = fmaxf(amax, fmaxf(fmaxf(fabsf(acc[v].x), fabsf(acc[v].y)), fmaxf(fabsf(acc[v].z), fabsf(acc[v].w))));
        }
    }
#pragma unroll
    for (int v = 0; v < 8; ++v) keep[pass][v] = acc[v];
  }
  if (p.dtype == 0) return;
  const float sc = pow2_scale(cta_max(amax, red));
  if (t == 0) p.st_scale[bh] = sc;
  const float inv_sc = 1.f / sc;
  const int MP = p.MP;
  void* st16T = reinterpret_cast<char*>(p.st16T) + (size_t)bh * D * MP * 2;
  void* kt16 = reinterpret_cast<char*>(p.kt16) + (size_t)bh * MP * D * 2;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int l = (t >> 2) + pass * (kThreads / 4);
    if (l < m) {
#pragma unroll
      for (int v = 0; v < 8; ++v)
        if (v < nv) {
          const int d = d0 + 4 * v;
          store16(st16T, p.dtype, (size_t)(d + 0) * MP + l, keep[pass][v].x * inv_sc);
          store16(st16T, p.dtype, (size_t)(d + 1) * MP + l, keep[pass][v].y * inv_sc);
          store16(st16T, p.dtype, (size_t)(d + 2) * MP + l, keep[pass][v].z * inv_sc);
          store16(st16T, p.dtype, (size_t)(d + 3) * MP + l, keep[pass][v].w * inv_sc);
        }
    }
  }
  for (int idx = t; idx < D * (MP - m); idx += kThreads) {
    const int d = idx / (MP - m), l = m + idx - d * (MP - m);
    store16(st16T, p.dtype, (size_t)d * MP + l, 0.f);
  }
  pack_pair(p.k_landmarks + bh * (int64_t)m * D, kt16, nullptr, p.dtype, m, D, MP, p.kt_mul);
}

// ------------------------------------------------------------------------------------------
struct BwdMid1Params {
  const float* partA;         // [BH][nchunk][2][m][D]
  int nchunk;
  const float* k2inv; const float* bmat; const float* q_landmarks;
  float* dkt_a;               // [BH][m][D]    (null: not written)
  float* dO3;                 // [BH][m][D]    (null: not written)
  float* D3;                  // [BH][m]
  float* G;                   // [BH][m][m]  dK2inv  (null: not computed)
  int m, D;
  int dtype, MP;
  void* qt16;                 // [BH][MP][D] = qt_mul * Qt
  void* qtT16;                // [BH][D][MP] = qtT_mul * Qt^T
  void* do3n;                 // [BH][MP][D] = dO3 / do3_scale
  void* do3T;                 // [BH][D][MP]
  float* do3_scale;           // [BH]
  float qt_mul, qtT_mul;
};

__host__ __device__ inline size_t bwd_mid1_smem(int m, int D) {
  return sizeof(float) * (2 * (size_t)m * (D + 4) + (size_t)m * D + (size_t)m * (m + 1));
}

template <int NV>
__global__ void __launch_bounds__(kThreads) bwd_mid1_kernel(BwdMid1Params p) {
  // NV = D / 16.  Shared memory (bwd_mid1_smem): dstep2 [m][D+4], Bmat [m][D+4], dO3 [m][D],
  // K2inv [m][m+1].  Both products are register-tiled (thread (ty, tx) of a 16 x 16 grid owns rows
  // ty + 16 i and columns tx + 16 j), with padded rows so that a warp's shared loads spread over
  // the banks.
  extern __shared__ float sm[];
  __shared__ float red[8];
  const int64_t bh = blockIdx.x;
  const int m = p.m, D = p.D, t = threadIdx.x, nc = p.nchunk, md = m * D, ldb = D + 4, ldk = m + 1;
  constexpr int CB = NV <= 2 ? 8 : (NV == 4 ? 4 : 2);
  const int q = t & 3;
  float* ds = sm;                    // dstep2 [m][ldb]
  float* bm = ds + m * ldb;          // Bmat   [m][ldb]
  float* do3 = bm + m * ldb;         // dO3    [m][D]
  float* sK = do3 + md;              // K2inv  [m][ldk]
  const float* partA = p.partA + bh * (int64_t)nc * 2 * md;
  const float* bmat = p.bmat + bh * (int64_t)md;
  const float* k2inv = p.k2inv + bh * m * m;
  for (int idx = t; idx < m * m; idx += kThreads) sK[(idx / m) * ldk + idx % m] = k2inv[idx];
  // chunk sums of (dstep2, dKt): thread = (row l, interleaved float4 columns 4 q + 16 v)
  for (int l = t >> 2; l < m; l += kThreads / 4) {
    float4 a0[NV], a1[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) { a0[v] = make_float4(0, 0, 0, 0); a1[v] = make_float4(0, 0, 0, 0); }
    for (int c0 = 0; c0 < nc; c0 += CB) {
      float4 x[CB][NV], y[CB][NV];
#pragma unroll
      for (int i = 0; i < CB; ++i) {
        const int c = min(c0 + i, nc - 1);
        const float* s0 = partA + (size_t)c * 2 * md + l * D + 4 * q;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          x[i][v] = *reinterpret_cast<const float4*>(s0 + 16 * v);
          y[i][v] = *reinterpret_cast<const float4*>(s0 + md + 16 * v);
        }
      }
#pragma unroll
      for (int i = 0; i < CB; ++i) {
        if (c0 + i < nc) {
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            a0[v].x += x[i][v].x; a0[v].y += x[i][v].y; a0[v].z += x[i][v].z; a0[v].w += x[i][v].w;
            a1[v].x += y[i][v].x; a1[v].y += y[i][v].y; a1[v].z += y[i][v].z; a1[v].w += y[i][v].w;
          }
        }
      }
    }
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int d = 4 * q + 16 * v;
      *reinterpret_cast<float4*>(ds + l * ldb + d) = a0[v];
      *reinterpret_cast<float4*>(bm + l * ldb + d) = *reinterpret_cast<const float4*>(bmat + l * D + d);
      if (p.dkt_a) *reinterpret_cast<float4*>(p.dkt_a + bh * md + l * D + d) = a1[v];
    }
  }
  __syncthreads();
  const int tx = t & 15, ty = t >> 4;
  const int MI = (m + 15) >> 4;
  float amax = 0.f;
  {
    // dO3[l][d] = sum_k K2inv[k][l] dstep2[k][d]:  rows l = ty + 16 i, columns d = tx + 16 j
    float acc[4][NV];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < NV; ++j) acc[i][j] = 0.f;
#pragma unroll 2
    for (int k = 0; k < m; ++k) {
      float a[4], b[NV];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = (i < MI && ty + 16 * i < m) ? sK[k * ldk + ty + 16 * i] : 0.f;
#pragma unroll
      for (int j = 0; j < NV; ++j) b[j] = ds[k * ldb + tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < NV; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int l = ty + 16 * i;
      if (l < m) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const int d = tx + 16 * j;
          do3[l * D + d] = acc[i][j];
          if (p.dO3) p.dO3[bh * md + l * D + d] = acc[i][j];
          amax = fmaxf(amax, fabsf(acc[i][j]));
        }
      }
    }
  }
  if (p.G) {
    // G[l][j] = sum_d dstep2[l][d] Bmat[j][d]:  rows l = ty + 16 i, columns j = tx + 16 jj
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 2
    for (int d = 0; d < D; d += 4) {
      float4 a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        a[i] = (ty + 16 * i < m) ? *reinterpret_cast<const float4*>(ds + (ty + 16 * i) * ldb + d) : make_float4(0, 0, 0, 0);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        b[j] = (tx + 16 * j < m) ? *reinterpret_cast<const float4*>(bm + (tx + 16 * j) * ldb + d) : make_float4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[i][j] += (a[i].x * b[j].x + a[i].y * b[j].y) + (a[i].z * b[j].z + a[i].w * b[j].w);
    }
    float* G = p.G + bh * m * m;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (ty + 16 * i < m && tx + 16 * j < m) G[(ty + 16 * i) * m + tx + 16 * j] = acc[i][j];
  }
  __syncthreads();   // dO3 is complete in shared memory
  // D3[l] = sum_d dO3[l][d] Bmat[l][d]: four threads per row
  for (int l0 = 0; l0 < m; l0 += kThreads / 4) {
    const bool act = l0 + (t >> 2) < m;
    const int l = act ? l0 + (t >> 2) : m - 1;
    float d3 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int d = 4 * q + 16 * v;
      const float4 x = *reinterpret_cast<const float4*>(do3 + l * D + d);
      const float4 y = *reinterpret_cast<const float4*>(bm + l * ldb + d);
      d3 += (x.x * y.x + x.y * y.y) + (x.z * y.z + x.w * y.w);
    }
    d3 += __shfl_xor_sync(0xffffffffu, d3, 1);
    d3 += __shfl_xor_sync(0xffffffffu, d3, 2);
    if (q == 0 && act) p.D3[bh * m + l] = d3;
  }
  if (p.dtype == 0) return;
  const float sc = pow2_scale(cta_max(amax, red));   // barrier inside: do3 is complete
  if (t == 0) p.do3_scale[bh] = sc;
  const float inv_sc = 1.f / sc;
  const int MP = p.MP;
  const size_t ob = (size_t)bh * MP * D * 2;
  const float* qt = p.q_landmarks + bh * (int64_t)md;
  // 16-bit copies, eight elements (one 16-byte store) at a time: dO3 / scale and qt_mul * Qt, rows >= m zero
  auto pack8 = [&](const float* x, float mul) {
    uint4 w;
    uint32_t* u = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a = x ? x[2 * e] * mul : 0.f, b = x ? x[2 * e + 1] * mul : 0.f;
      if (p.dtype == 1) { __half2 h = __floats2half2_rn(a, b); u[e] = *reinterpret_cast<uint32_t*>(&h); }
      else { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); u[e] = *reinterpret_cast<uint32_t*>(&h); }
    }
    return w;
  };
  for (int idx = t; idx < MP * D / 8; idx += kThreads) {
    const int r = (idx * 8) / D, c = idx * 8 - r * D;
    reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.do3n) + ob)[idx] = pack8(r < m ? do3 + r * D + c : nullptr, inv_sc);
    float qv[8];
    if (r < m) {
      const float4 x = *reinterpret_cast<const float4*>(qt + r * D + c), y = *reinterpret_cast<const float4*>(qt + r * D + c + 4);
      qv[0] = x.x; qv[1] = x.y; qv[2] = x.z; qv[3] = x.w; qv[4] = y.x; qv[5] = y.y; qv[6] = y.z; qv[7] = y.w;
    }
    reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.qt16) + ob)[idx] = pack8(r < m ? qv : nullptr, p.qt_mul);
  }
  if (p.do3T)
    for (int idx = t; idx < D * MP; idx += kThreads) {
      int d = idx / MP, l = idx - d * MP;
      store16(reinterpret_cast<char*>(p.do3T) + ob, p.dtype, idx, l < m ? do3[l * D + d] * inv_sc : 0.f);
    }
  if (p.qtT16) pack_pair(qt, nullptr, reinterpret_cast<char*>(p.qtT16) + ob, p.dtype, m, D, MP, p.qtT_mul);
}

// ------------------------------------------------------------------------------------------
// Column-slab version of the combine step for head_dim a multiple of 16 and num_landmarks <= 64:
// grid (BH, D / 16).  A CTA merges the softmax-3 partials of its 16 head-dim columns for every
// landmark (thread = landmark row x 4 columns, all chunk loads in flight at once), writes those
// columns of Bmat (and lse3 from slab 0), then forms the same columns of step2 = K2inv Bmat from
// shared memory.  No operand copies: the output pass packs its own.
struct CombineSlabParams {
  const float* part_acc; const float* part_max; const float* part_sum;
  int nchunk;
  int64_t acc_bh_stride, acc_chunk_stride, vec_bh_stride, vec_chunk_stride;
  const float* k2inv;
  float* bmat; float* lse3; float* step2;
  int m, D;
};

constexpr int kSlabMaxChunks = 20;   // chunks merged with every load in flight; more run in rounds

// Dynamic shared memory: K2inv with padded rows, m (m + 1) floats (combine_slab_smem).
__host__ __device__ inline size_t combine_slab_smem(int m) { return sizeof(float) * (size_t)m * (m + 1); }

__global__ void __launch_bounds__(kThreads) combine_slab_kernel(CombineSlabParams p) {
  extern __shared__ float sK[];                        // [m][m + 1]
  __shared__ __align__(16) float sB[kMaxM * 16];
  pdl_trigger();
  pdl_wait();
  const int64_t bh = blockIdx.x;
  const int slab = blockIdx.y, t = threadIdx.x, q = t & 3;
  const int m = p.m, D = p.D, nc = p.nchunk, d0 = 16 * slab + 4 * q, ms = m + 1;
  const float* k2inv = p.k2inv + bh * m * m;
  for (int idx = t; idx < m * m; idx += kThreads) sK[(idx / m) * ms + idx % m] = k2inv[idx];
  // thread t merges landmark rows t >> 2 and, with more than 64 landmarks, (t >> 2) + 64
  for (int l = t >> 2; l < kMaxM; l += 64) {
    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (l < m) {
      const float* pacc = p.part_acc + bh * p.acc_bh_stride + (size_t)l * D + d0;
      const float* pmax = p.part_max + bh * p.vec_bh_stride + l;
      const float* psum = p.part_sum + bh * p.vec_bh_stride + l;
      // with at most kSlabMaxChunks chunks (the usual case) the maxima come out of the one batch of
      // loads below; otherwise a first sweep finds them
      float M = -INFINITY;
      if (nc > kSlabMaxChunks)
        for (int c = 0; c < nc; ++c) M = fmaxf(M, pmax[c * p.vec_chunk_stride]);
      float Lsum = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int c0 = 0; c0 < nc; c0 += kSlabMaxChunks) {
        float4 x[kSlabMaxChunks];
        float wgt[kSlabMaxChunks], ps[kSlabMaxChunks];
#pragma unroll
        for (int i = 0; i < kSlabMaxChunks; ++i) {
          const int c = min(c0 + i, nc - 1);
          x[i] = *reinterpret_cast<const float4*>(pacc + (size_t)c * p.acc_chunk_stride);
          wgt[i] = pmax[c * p.vec_chunk_stride];
          ps[i] = psum[c * p.vec_chunk_stride];
        }
        if (nc <= kSlabMaxChunks) {
#pragma unroll
          for (int i = 0; i < kSlabMaxChunks; ++i) M = fmaxf(M, wgt[i]);   // entries past nc repeat the last chunk
        }
#pragma unroll
        for (int i = 0; i < kSlabMaxChunks; ++i) {
          const float w = (c0 + i < nc) ? expf(wgt[i] - M) : 0.f;
          Lsum = fmaf(w, ps[i], Lsum);
          acc.x = fmaf(w, x[i].x, acc.x); acc.y = fmaf(w, x[i].y, acc.y);
          acc.z = fmaf(w, x[i].z, acc.z); acc.w = fmaf(w, x[i].w, acc.w);
        }
      }
      const float inv = 1.f / Lsum;
      b = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
      *reinterpret_cast<float4*>(p.bmat + (bh * m + l) * D + d0) = b;
      if (slab == 0 && q == 0) p.lse3[bh * m + l] = M + logf(Lsum);
    }
    *reinterpret_cast<float4*>(sB + l * 16 + 4 * q) = b;
  }
  __syncthreads();
  for (int l = t >> 2; l < m; l += 64) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int k = 0; k < m; ++k) {
      const float a = sK[l * ms + k];
      const float4 x = *reinterpret_cast<const float4*>(sB + k * 16 + 4 * q);
      acc.x = fmaf(a, x.x, acc.x); acc.y = fmaf(a, x.y, acc.y); acc.z = fmaf(a, x.z, acc.z); acc.w = fmaf(a, x.w, acc.w);
    }
    *reinterpret_cast<float4*>(p.step2 + (bh * m + l) * D + d0) = acc;
  }
}

// ------------------------------------------------------------------------------------------
// After the global-memory middle stage of the backward (num_landmarks > 64), what the tensor-core
// column pass and the in-place pass read: the 16-bit operand copies dO3 / 2^e (with 2^e >= max |dO3|)
// and qt_mul * Qt, padded to MP rows, and the per-landmark rows scale * dKt_tot / len.
struct MidPackParams {
  const float* dO3; const float* q_landmarks; const float* dkt_tot;   // [BH][m][D]
  void* do3n; float* do3_scale; void* qt16; float* rows_k;
  int m, D, MP, dtype;
  float qt_mul, scale;
  int64_t N;
};
// gridDim.y CTAs share a slice: each finds the scale for itself (the slice's dO3 comes from L2) and
// packs its share of the rows, four values per thread and step.
constexpr int kMidPackSplit = 8;
__global__ void __launch_bounds__(kThreads) mid_pack_kernel(MidPackParams p) {
  __shared__ float red[8];
  const int64_t bh = blockIdx.x;
  const int md = p.m * p.D, t = threadIdx.x;
  const float* dO3 = p.dO3 + bh * (int64_t)md;
  float amax = 0.f;
  for (int idx = t; idx < md / 4; idx += kThreads) {
    const float4 x = reinterpret_cast<const float4*>(dO3)[idx];
    amax = fmaxf(fmaxf(amax, fmaxf(fabsf(x.x), fabsf(x.y))), fmaxf(fabsf(x.z), fabsf(x.w)));
  }
  const float sc = pow2_scale(cta_max(amax, red)), inv_sc = 1.f / sc;
  if (t == 0 && blockIdx.y == 0) p.do3_scale[bh] = sc;
  const size_t ob = (size_t)bh * p.MP * p.D * 2;
  const float* qt = p.q_landmarks + bh * (int64_t)md;
  const float* dkt = p.dkt_tot + bh * (int64_t)md;
  Segments sg(p.N, p.m);
  const int groups = p.MP * p.D / 4;       // groups of four consecutive columns of the padded operands
  for (int g = blockIdx.y * kThreads + t; g < groups; g += gridDim.y * kThreads) {
    const int l = (g * 4) / p.D;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), q = a;
    if (l < p.m) {
      a = reinterpret_cast<const float4*>(dO3)[g];
      q = reinterpret_cast<const float4*>(qt)[g];
      const float4 k = reinterpret_cast<const float4*>(dkt)[g];
      const float f = p.scale / (float)sg.len(l);
      reinterpret_cast<float4*>(p.rows_k + bh * (int64_t)md)[g] = make_float4(k.x * f, k.y * f, k.z * f, k.w * f);
    }
    reinterpret_cast<uint2*>(reinterpret_cast<char*>(p.do3n) + ob)[g] =
        make_uint2(pack2x16(p.dtype, a.x * inv_sc, a.y * inv_sc), pack2x16(p.dtype, a.z * inv_sc, a.w * inv_sc));
    reinterpret_cast<uint2*>(reinterpret_cast<char*>(p.qt16) + ob)[g] =
        make_uint2(pack2x16(p.dtype, q.x * p.qt_mul, q.y * p.qt_mul), pack2x16(p.dtype, q.z * p.qt_mul, q.w * p.qt_mul));
  }
}

// ------------------------------------------------------------------------------------------
struct PackBwdAcParams {
  const float* k_landmarks; const float* step2;
  void* kt16;      // [BH][MP][D] = kt_mul * Kt
  void* ktT16;     // [BH][D][MP] = ktT_mul * Kt^T
  void* st16;      // [BH][MP][D] = step2 / st_scale
  float* st_scale;
  int m, D, MP, dtype;
  float kt_mul, ktT_mul;
};

__global__ void __launch_bounds__(kThreads) pack_bwd_ac_kernel(PackBwdAcParams p) {
  __shared__ float red[8];
  const int64_t bh = blockIdx.x;
  const int md = p.m * p.D;
  const size_t ob = (size_t)bh * p.MP * p.D * 2;
  const float* kt = p.k_landmarks + bh * (int64_t)md;
  const float* st = p.step2 + bh * (int64_t)md;
  float amax = 0.f;
  for (int idx = threadIdx.x; idx < md; idx += kThreads) amax = fmaxf(amax, fabsf(st[idx]));
  const float sc = pow2_scale(cta_max(amax, red));
  if (threadIdx.x == 0) p.st_scale[bh] = sc;
  pack_pair(st, reinterpret_cast<char*>(p.st16) + ob, nullptr, p.dtype, p.m, p.D, p.MP, 1.f / sc);
  pack_pair(kt, reinterpret_cast<char*>(p.kt16) + ob, nullptr, p.dtype, p.m, p.D, p.MP, p.kt_mul);
  if (p.ktT16) pack_pair(kt, nullptr, reinterpret_cast<char*>(p.ktT16) + ob, p.dtype, p.m, p.D, p.MP, p.ktT_mul);
}

// dqt_tot = dqt_ns + sum over chunks of the column-pass partials, summed in a fixed order.
// rows_q (optional) = scale * dqt_tot / len(landmark): the per-landmark row the dQ pass adds to
// every token of that landmark's segment.
__global__ void __launch_bounds__(kThreads)
dqt_reduce2_kernel(const float* partB, int nchunk, const float* dqt_ns, float* dqt_tot, float* rows_q, int m,
                   int D, int64_t N, float scale) {
  // 64 float4 columns x 4 chunk lanes per CTA: lane cl sums chunks cl, cl + 4, ...; the four
  // partial sums are then added in a fixed order through shared memory.
  __shared__ float4 part[3][64];
  pdl_trigger();
  pdl_wait();
  const int64_t bh = blockIdx.y;
  const int md = m * D;
  const int el = threadIdx.x & 63, cl = threadIdx.x >> 6;
  const int idx4 = (blockIdx.x * 64 + el) * 4;
  const bool in = idx4 < md;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (in) {
    const float* src = partB + bh * (size_t)nchunk * md + idx4;
#pragma unroll 5
    for (int c = cl; c < nchunk; c += 4) {
      const float4 x = *reinterpret_cast<const float4*>(src + (size_t)c * md);
      s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
    }
  }
  if (cl > 0) part[cl - 1][el] = s;
  __syncthreads();
  if (cl > 0 || !in) return;
  const float4 n0 = *reinterpret_cast<const float4*>(dqt_ns + bh * md + idx4);
#pragma unroll
  for (int k = 0; k < 3; ++k) { const float4 x = part[k][el]; s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w; }
  s.x += n0.x; s.y += n0.y; s.z += n0.z; s.w += n0.w;
  if (dqt_tot) *reinterpret_cast<float4*>(dqt_tot + bh * md + idx4) = s;
  if (rows_q) {
    Segments sg(N, m);
    const float f = scale / (float)sg.len(idx4 / D);
    *reinterpret_cast<float4*>(rows_q + bh * md + idx4) = make_float4(s.x * f, s.y * f, s.z * f, s.w * f);
  }
}

// Landmarks from the pooling pass's raw segment sums: qt / kt [BH][m][D] = scale * sum / len,
// plus the 16-bit copy of qt_mul * qt (rows m..MP-1 zero) for the tensor-core column pass.
// grid (BH, parts): the CTAs of a slice share its groups of four columns.
struct LandmarkFinalizeParams {
  const float* land_partial;  // [2][BH][m][C][D]
  int C;
  float* qt; float* kt;
  int64_t BH, N;
  int m, D;
  float scale;
  void* qt16; int dtype, MP; float qt16_mul;
};

__global__ void __launch_bounds__(kThreads) landmark_finalize_kernel(LandmarkFinalizeParams p) {
  const int64_t bh = blockIdx.x;
  const int m = p.m, D = p.D, rows = p.qt16 ? p.MP : m;
  Segments sg(p.N, m);
  // an item = four consecutive columns of one landmark row of Q~ or K~ (D is a multiple of 16)
  const int per_row = 2 * D / 4;
  for (int item = blockIdx.y * kThreads + threadIdx.x; item < rows * per_row; item += gridDim.y * kThreads) {
    const int l = item / per_row, r = item - l * per_row;
    const int which = r / (D / 4), d = (r - which * (D / 4)) * 4;
    float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
    if (l < m) {
      const float* src = p.land_partial + ((((size_t)which * p.BH + bh) * m + l) * p.C) * D + d;
      for (int c = 0; c < p.C; ++c) {
        const float4 x = *reinterpret_cast<const float4*>(src + (size_t)c * D);
        val.x += x.x; val.y += x.y; val.z += x.z; val.w += x.w;
      }
      const float f = p.scale / (float)sg.len(l);
      val = make_float4(val.x * f, val.y * f, val.z * f, val.w * f);
      *reinterpret_cast<float4*>((which ? p.kt : p.qt) + (bh * m + l) * D + d) = val;
    }
    if (which == 0 && p.qt16)
      *reinterpret_cast<uint2*>(reinterpret_cast<char*>(p.qt16) + ((size_t)bh * p.MP * D + (size_t)l * D + d) * 2) =
          make_uint2(pack2x16(p.dtype, val.x * p.qt16_mul, val.y * p.qt16_mul),
                     pack2x16(p.dtype, val.z * p.qt16_mul, val.w * p.qt16_mul));
  }
}

// out[bh][e] = sum over chunks of in[bh][chunk][e], fixed order (e < elems, elems % 4 == 0).
__global__ void __launch_bounds__(kThreads)
reduce_chunks_kernel(const float* in, int nchunk, int elems, float* out) {
  // same split as dqt_reduce2_kernel: 64 float4 columns x 4 chunk lanes per CTA
  __shared__ float4 part[3][64];
  pdl_trigger();
  pdl_wait();
  const int64_t bh = blockIdx.y;
  const int el = threadIdx.x & 63, cl = threadIdx.x >> 6;
  const int idx4 = (blockIdx.x * 64 + el) * 4;
  const bool inr = idx4 < elems;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (inr) {
    const float* src = in + bh * (size_t)nchunk * elems + idx4;
#pragma unroll 5
    for (int c = cl; c < nchunk; c += 4) {
      const float4 x = *reinterpret_cast<const float4*>(src + (size_t)c * elems);
      s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
    }
  }
  if (cl > 0) part[cl - 1][el] = s;
  __syncthreads();
  if (cl > 0 || !inr) return;
#pragma unroll
  for (int k = 0; k < 3; ++k) { const float4 x = part[k][el]; s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w; }
  *reinterpret_cast<float4*>(out + bh * (size_t)elems + idx4) = s;
}

// ------------------------------------------------------------------------------------------
// What the tensor-core column pass of the backward needs from the middle stage, for head_dim 64 and
// m <= 64, when the pseudoinverse backward runs beside that pass instead of in front of it:
//   dO3 = K2inv^T dstep2  ->  D3[l] = sum_d dO3[l][d] Bmat[l][d],
//   do3n = dO3 / 2^e (16-bit, rows >= m zero) with 2^e >= max |dO3|,  qt16 = qt_mul * Qt (16-bit).
// One CTA per slice: the three 64 x 64 inputs are fetched with every load in flight at once, the
// product runs from shared memory on 4 x 4 register tiles (two 16-byte shared loads per 16 FMAs).
struct ColpassOperandParams {
  const float* dstep2;        // first [m][D] block of each slice; slices bh_stride floats apart
  int64_t bh_stride;
  const float* k2inv;         // [BH][m][m]
  const float* bmat;          // [BH][m][D]
  const float* q_landmarks;   // [BH][m][D]
  float* D3;                  // [BH][m]
  void* do3n;                 // [BH][64][D] 16-bit
  float* do3_scale;           // [BH]
  void* qt16;                 // [BH][64][D] 16-bit
  float qt_mul;
  int m, dtype;
};
constexpr int kColpassOperandSmem = 3 * 64 * 64 * (int)sizeof(float);

__global__ void __launch_bounds__(kThreads) colpass_operands_kernel(ColpassOperandParams p) {
  constexpr int D = 64;
  extern __shared__ float sm[];
  __shared__ float red[8];
  float* Ki = sm;               // K2inv [k][l], later dO3 [l][d]
  float* Ds = sm + 64 * 64;     // dstep2 [k][d]
  float* Bm = sm + 2 * 64 * 64; // Bmat [l][d]
  pdl_trigger();
  pdl_wait();
  const int64_t bh = blockIdx.x;
  const int m = p.m, t = threadIdx.x;
  const float* k2inv = p.k2inv + bh * m * m;
  const float* ds = p.dstep2 + bh * p.bh_stride;
  const float* bm = p.bmat + bh * (int64_t)m * D;
  {
    float4 a[4], b[4], c[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = (t + kThreads * i) * 4, r = e >> 6, col = e & 63;
      a[i] = b[i] = c[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < m) {
        b[i] = *reinterpret_cast<const float4*>(ds + r * D + col);
        c[i] = *reinterpret_cast<const float4*>(bm + r * D + col);
        if (m == 64) {
          a[i] = *reinterpret_cast<const float4*>(k2inv + r * 64 + col);
        } else {
          a[i].x = col + 0 < m ? k2inv[r * m + col + 0] : 0.f;
          a[i].y = col + 1 < m ? k2inv[r * m + col + 1] : 0.f;
          a[i].z = col + 2 < m ? k2inv[r * m + col + 2] : 0.f;
          a[i].w = col + 3 < m ? k2inv[r * m + col + 3] : 0.f;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = (t + kThreads * i) * 4;
      *reinterpret_cast<float4*>(Ki + e) = a[i];
      *reinterpret_cast<float4*>(Ds + e) = b[i];
      *reinterpret_cast<float4*>(Bm + e) = c[i];
    }
  }
  __syncthreads();
  // dO3[l0..l0+3][d0..d0+3] = sum_k K2inv[k][l0..] dstep2[k][d0..]
  const int l0 = (t >> 4) * 4, d0 = (t & 15) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 8
  for (int k = 0; k < 64; ++k) {
    const float4 a = *reinterpret_cast<const float4*>(Ki + k * 64 + l0);
    const float4 b = *reinterpret_cast<const float4*>(Ds + k * 64 + d0);
    const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
  }
  float amax = 0.f, d3[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 x = *reinterpret_cast<const float4*>(Bm + (l0 + i) * 64 + d0);
    d3[i] = acc[i][0] * x.x + acc[i][1] * x.y + acc[i][2] * x.z + acc[i][3] * x.w;
#pragma unroll
    for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(acc[i][j]));
    // the 16 threads that share l0 are 16 consecutive lanes
    for (int o = 8; o > 0; o >>= 1) d3[i] += __shfl_xor_sync(0xffffffffu, d3[i], o);
  }
  if ((t & 15) == 0)
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (l0 + i < m) p.D3[bh * m + l0 + i] = d3[i];
  const float sc = pow2_scale(cta_max(amax, red));   // barriers inside: every read of Ki is done
  const float inv_sc = 1.f / sc;
  if (t == 0) p.do3_scale[bh] = sc;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<float4*>(Ki + (l0 + i) * 64 + d0) =
        make_float4(acc[i][0] * inv_sc, acc[i][1] * inv_sc, acc[i][2] * inv_sc, acc[i][3] * inv_sc);
  __syncthreads();
  // 16-bit copies: thread t packs row t >> 2, columns 16 (t & 3) .. +15 of both matrices
  const int r = t >> 2, c0 = (t & 3) * 16;
  const float* qrow = p.q_landmarks + bh * (int64_t)m * D + (int64_t)r * D + c0;
  uint32_t w0[8], w1[8];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float4 x = *reinterpret_cast<const float4*>(Ki + r * 64 + c0 + 4 * q);   // rows >= m are zero
    float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < m) y = *reinterpret_cast<const float4*>(qrow + 4 * q);
    w0[2 * q] = pack2x16(p.dtype, x.x, x.y); w0[2 * q + 1] = pack2x16(p.dtype, x.z, x.w);
    w1[2 * q] = pack2x16(p.dtype, y.x * p.qt_mul, y.y * p.qt_mul);
    w1[2 * q + 1] = pack2x16(p.dtype, y.z * p.qt_mul, y.w * p.qt_mul);
  }
  const size_t ob = ((size_t)bh * 64 + r) * D + c0;
  uint4* o0 = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.do3n) + ob);
  uint4* o1 = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.qt16) + ob);
  o0[0] = make_uint4(w0[0], w0[1], w0[2], w0[3]); o0[1] = make_uint4(w0[4], w0[5], w0[6], w0[7]);
  o1[0] = make_uint4(w1[0], w1[1], w1[2], w1[3]); o1[1] = make_uint4(w1[4], w1[5], w1[6], w1[7]);
}

}  // namespace fnb
