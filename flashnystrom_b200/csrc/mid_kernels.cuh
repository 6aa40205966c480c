// The landmark-sized ("middle") stages: everything that works on (m x m) and (m x D) FP32
// matrices per (b,h) slice.  Operands live in global memory (they are a few hundred KB per slice
// and stay in L2), so the same code serves every m <= 128.  On the CUDA cores: one CTA of 256
// threads per slice, products staged through shared memory k-slab by k-slab.  On the tensor
// cores: 512 threads per CTA and, for mid_fwd_kernel / mid_bwd_kernel, a thread-block cluster of
// up to eight CTAs per slice that shares the products (by output columns; in the backward
// iterations also as two halves that take independent products side by side) and the element-wise
// phases, meeting at cluster barriers.
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
#include "tc_common.cuh"

namespace fnb {

// ---- products on the tensor cores ------------------------------------------------------------
// The (<= 128)^3 FP32 products of the middle stages, with FP32-equivalent arithmetic on tcgen05:
// each operand is copied from global memory into shared memory as three bf16 terms
// x = x0 + x1 + x2 (24 significant bits together), stored exactly as it is laid out in memory
// (rows x columns, 128-byte swizzle, two 64-column blocks of [128 rows x 128 B] per term), so that
// a transposed use only changes the shared-memory descriptor (K-major or MN-major).  The six
// partial products x_i y_j with i + j <= 2 accumulate into one 128 x 128 FP32 accumulator in
// tensor memory (48 MMAs of M = N = 128, K = 16 for a full 128^3 product), and the epilogue applies
// alpha, beta C and the diagonal term on the way back to global memory.  One CTA of 256 threads per
// slice; thread 0 issues the MMAs.  A kernel that wants this path gives its GemmWs the tile area
// (2 x 96 KB of dynamic shared memory, 1024-byte aligned), an mbarrier and 128 columns of tensor
// memory; with tiles == nullptr the products run on the CUDA cores (cta_gemm below).
constexpr int kTcGemmTerm = 128 * 256;            // one bf16 term of a 128 x 128 operand
constexpr int kTcGemmSet = 3 * kTcGemmTerm;       // the three terms
constexpr size_t kTcGemmSmem = 2 * (size_t)kTcGemmSet + 1024;
// CTA size of the kernels of this file when their products run on the tensor cores: every product is a
// chain of three latency-bound phases (operand copy and split, MMAs, epilogue) that all threads take
// part in, so twice the warps shorten the first and the last (the CUDA-core products keep 256 threads)
constexpr int kMidTcThreads = 512;

#ifdef FNB_TC_TRACE
__device__ unsigned long long g_gemm_cycles[8];
#define GEMM_T(i) do { if (blockIdx.x == 0 && threadIdx.x == 0) { long long now_ = clock64(); atomicAdd(&g_gemm_cycles[i], (unsigned long long)(now_ - t_)); t_ = now_; } } while (0)
#define GEMM_T0() long long t_ = clock64()
#else
#define GEMM_T(i) do {} while (0)
#define GEMM_T0() do {} while (0)
#endif

struct GemmWs {
  float* sm;            // staging / reduction scratch of the CUDA-core code (kGemmSmemFloats floats)
  uint8_t* tiles;       // null: CUDA-core products
  uint64_t* bar;
  uint32_t tmem;
  uint32_t phase;
  int* status;
  // A slice may be worked on by a thread-block cluster of cs CTAs (rank = this CTA's place in it):
  // every product is split by output columns, every element-wise phase by elements, and the phases
  // meet at a cluster barrier; operands and results live in global memory (L2) as before.
  int cs, rank;
  int gt, gn;           // thread index and thread count over the whole cluster
  int defer_sync;       // 1: a product ends without the cluster barrier (the caller places it)
};

__device__ __forceinline__ int cluster_size() {
  uint32_t n;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n));
  return (int)n;
}
__device__ __forceinline__ int cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return (int)r;
}
// End of a phase: what the CTAs of the cluster wrote to global memory is visible to all of them
// afterwards.  All threads of all CTAs of the cluster call (a hardware barrier: no spin-wait).
__device__ __forceinline__ void mid_sync(int cs) {
  if (cs > 1) {
    __threadfence();
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  } else {
    __syncthreads();
  }
}

// rows x cols FP32 matrix in global memory (leading dimension ld) -> three swizzled bf16 term tiles,
// zero beyond rows / cols.  All NT threads of the CTA.
template <int NT>
__device__ inline void tc_gemm_load(uint8_t* set, const float* src, int ld, int rows, int cols) {
  // 128 rows x 16 chunks of 8 columns = 2048 items, 2048 / NT per thread; all of a thread's global
  // loads are issued before the first value is used (one round trip to L2)
  constexpr int kItems = 128 * 16 / NT;
  const bool vec = (ld & 3) == 0 && (cols & 7) == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
  float v[kItems][8];
#pragma unroll
  for (int it = 0; it < kItems; ++it) {
    const int item = threadIdx.x + it * NT;
    const int r = item >> 4, c0 = (item & 15) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[it][i] = 0.f;
    if (r < rows && c0 < cols) {
      const float* g = src + (size_t)r * ld + c0;
      if (vec) {
        const float4 a = *reinterpret_cast<const float4*>(g), b = *reinterpret_cast<const float4*>(g + 4);
        v[it][0] = a.x; v[it][1] = a.y; v[it][2] = a.z; v[it][3] = a.w;
        v[it][4] = b.x; v[it][5] = b.y; v[it][6] = b.z; v[it][7] = b.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) if (c0 + i < cols) v[it][i] = g[i];
      }
    }
  }
#pragma unroll
  for (int it = 0; it < kItems; ++it) {
    const int item = threadIdx.x + it * NT;
    const int r = item >> 4, ch = item & 15;
    uint32_t w0[4], w1[4], w2[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      float a = v[it][2 * p], b = v[it][2 * p + 1];
      w0[p] = tc::pack2<__nv_bfloat16>(a, b);
      a -= __uint_as_float(w0[p] << 16);
      b -= __uint_as_float(w0[p] & 0xffff0000u);
      w1[p] = tc::pack2<__nv_bfloat16>(a, b);
      a -= __uint_as_float(w1[p] << 16);
      b -= __uint_as_float(w1[p] & 0xffff0000u);
      w2[p] = tc::pack2<__nv_bfloat16>(a, b);
    }
    const uint32_t off = (uint32_t)(ch >> 3) * (128 * 128) + tc::sw128_offset(r, ch & 7);
    *reinterpret_cast<uint4*>(set + off) = make_uint4(w0[0], w0[1], w0[2], w0[3]);
    *reinterpret_cast<uint4*>(set + kTcGemmTerm + off) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
    *reinterpret_cast<uint4*>(set + 2 * kTcGemmTerm + off) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
  }
}

// descriptor of k-step k (16 elements of the contraction) of a term tile.
//   along_rows: the contraction index runs along the tile's rows (MN-major operand), else along its
//   columns (K-major operand)
__device__ __forceinline__ uint64_t tc_gemm_desc(uint32_t tile, bool along_rows, int k) {
  return along_rows ? tc::smem_desc_sw128(tile + k * 2048, 128 * 128, 1024)
                    : tc::smem_desc_sw128(tile + (k >> 2) * (128 * 128) + (k & 3) * 32, 16, 1024);
}

template <bool TA, bool TB, int NT>
__device__ inline void cta_gemm_tc(float* C, int ldc, const float* A, int lda, const float* B, int ldb, int M, int N,
                                   int K, float alpha, float beta, float diag, GemmWs& ws, float* C2, float alpha2,
                                   float diag2) {
  uint8_t* setA = ws.tiles;
  uint8_t* setB = ws.tiles + kTcGemmSet;
  GEMM_T0();
  // operands exactly as stored: A is (M x K) or, transposed, (K x M); B is (K x N) or (N x K)
  tc_gemm_load<NT>(setA, A, lda, TA ? K : M, TA ? M : K);
  tc_gemm_load<NT>(setB, B, ldb, TB ? N : K, TB ? K : N);
  tc::fence_proxy_async();
  __syncthreads();
  GEMM_T(0);
  if (threadIdx.x == 0) {
    tc::tc_fence_after();
    // A operand: K-major unless stored transposed; B operand: MN-major unless stored transposed.
    // The descriptor of (term, k-step) is the descriptor of (0, 0) plus a compile-time offset in its
    // 16-byte address field (all tiles lie inside one 256 KB window).
    constexpr bool AR = TA, BR = !TB;    // contraction index along the tile's rows?
    const uint32_t idesc = tc::make_idesc<__nv_bfloat16>(128, 128, TA, !TB);
    const uint64_t da = tc_gemm_desc(tc::smem_u32(setA), AR, 0), db = tc_gemm_desc(tc::smem_u32(setB), BR, 0);
    const int ksteps = (K + 15) >> 4;
    uint32_t acc = 0;
#pragma unroll
    for (int t = 0; t < 6; ++t) {
      // partial products x_i y_j, small terms first: (1,1) (0,2) (2,0) (0,1) (1,0) (0,0)
      constexpr int oi[6] = {1, 0, 2, 0, 1, 0}, oj[6] = {1, 2, 0, 1, 0, 0};
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (k < ksteps) {
          const uint32_t offa = oi[t] * kTcGemmTerm + (AR ? k * 2048 : (k >> 2) * (128 * 128) + (k & 3) * 32);
          const uint32_t offb = oj[t] * kTcGemmTerm + (BR ? k * 2048 : (k >> 2) * (128 * 128) + (k & 3) * 32);
          tc::umma(ws.tmem, da + (offa >> 4), db + (offb >> 4), idesc, acc);
          acc = 1;
        }
      }
    }
    tc::umma_commit(ws.bar);
  }
  GEMM_T(1);
  {
    tc::Abort ab{reinterpret_cast<volatile int*>(ws.bar + 1), ws.status};
    tc::mbar_wait(ws.bar, ws.phase, ab, 0x5000);
    ws.phase ^= 1u;
  }
  tc::tc_fence_after();
  GEMM_T(2);
  // epilogue, step 1: accumulator rows -> FP32 staging in shared memory (the operand tiles are dead).
  // Warp w reads TMEM lanes 32 (w & 3) .. + 31 (= rows) and its share of the 128 columns.
  constexpr int kLdS = 132;
  constexpr int kColsPerWarp = 128 / (NT / 128);
  float* stage = reinterpret_cast<float*>(ws.tiles);
  {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (warp & 3) * 32 + lane, cbase = (warp >> 2) * kColsPerWarp;
    const uint32_t taddr = ws.tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)cbase;
#pragma unroll
    for (int half = 0; half < kColsPerWarp / 32; ++half) {
      float v[32];
      tc::tmem_ld32(taddr + half * 32, v);
      tc::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(stage + r * kLdS + cbase + half * 32 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  // step 2: coalesced rows to global memory with alpha, beta C and the diagonal
  if ((ldc & 3) == 0 && (N & 3) == 0 && (reinterpret_cast<uintptr_t>(C) & 15u) == 0 &&
      (!C2 || (reinterpret_cast<uintptr_t>(C2) & 15u) == 0)) {
    const int n4 = N >> 2;
#pragma unroll 4
    for (int f = threadIdx.x; f < M * n4; f += NT) {
      const int r = f / n4, c = (f - r * n4) * 4;
      const float4 x = *reinterpret_cast<const float4*>(stage + r * kLdS + c);
      float4 o = make_float4(alpha * x.x, alpha * x.y, alpha * x.z, alpha * x.w);
      float* dst = C + (size_t)r * ldc + c;
      if (beta != 0.f) {
        const float4 old = *reinterpret_cast<const float4*>(dst);
        o.x += beta * old.x; o.y += beta * old.y; o.z += beta * old.z; o.w += beta * old.w;
      }
      const int dg = r - c;   // position of the diagonal element inside this group of four, if any
      if (dg == 0) o.x += diag; else if (dg == 1) o.y += diag; else if (dg == 2) o.z += diag; else if (dg == 3) o.w += diag;
      *reinterpret_cast<float4*>(dst) = o;
      if (C2) {
        float4 o2 = make_float4(alpha2 * x.x, alpha2 * x.y, alpha2 * x.z, alpha2 * x.w);
        if (dg == 0) o2.x += diag2; else if (dg == 1) o2.y += diag2; else if (dg == 2) o2.z += diag2; else if (dg == 3) o2.w += diag2;
        *reinterpret_cast<float4*>(C2 + (size_t)r * ldc + c) = o2;
      }
    }
  } else {
    for (int idx = threadIdx.x; idx < M * N; idx += NT) {
      const int r = idx / N, c = idx - r * N;
      const float x = stage[r * kLdS + c];
      float val = alpha * x;
      if (beta != 0.f) val += beta * C[(size_t)r * ldc + c];
      if (r == c) val += diag;
      C[(size_t)r * ldc + c] = val;
      if (C2) C2[(size_t)r * ldc + c] = alpha2 * x + (r == c ? diag2 : 0.f);
    }
  }
  __syncthreads();
  GEMM_T(3);
#ifdef FNB_TC_TRACE
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&g_gemm_cycles[4], 1ull);
#endif
}


// One column block of op(B) for the product of a cluster: rows [n0, n0 + nrows) of the (N x K) operand
// (stored_nk) or columns [n0, n0 + nrows) of the (K x N) operand, always written as a K-major tile
// whose row is the output column (so the MMA needs no partial swizzle atom along N).
template <int NT>
__device__ inline void tc_gemm_load_nblock(uint8_t* set, const float* B, int ldb, bool stored_nk, int n0, int nrows,
                                           int NB, int K) {
  const bool vec = stored_nk && (ldb & 3) == 0 && (K & 7) == 0 && (reinterpret_cast<uintptr_t>(B) & 15u) == 0;
  for (int item = threadIdx.x; item < NB * 16; item += NT) {
    // lanes run along the contiguous direction of the stored operand
    const int r = stored_nk ? item >> 4 : item % NB;
    const int ch = stored_nk ? item & 15 : item / NB;
    const int c0 = ch * 8;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (r < nrows && c0 < K) {
      if (stored_nk) {
        const float* g = B + (size_t)(n0 + r) * ldb + c0;
        if (vec) {
          const float4 a = *reinterpret_cast<const float4*>(g), b = *reinterpret_cast<const float4*>(g + 4);
          v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) if (c0 + i < K) v[i] = g[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) if (c0 + i < K) v[i] = B[(size_t)(c0 + i) * ldb + n0 + r];
      }
    }
    uint32_t w0[4], w1[4], w2[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      float a = v[2 * p], b = v[2 * p + 1];
      w0[p] = tc::pack2<__nv_bfloat16>(a, b);
      a -= __uint_as_float(w0[p] << 16);
      b -= __uint_as_float(w0[p] & 0xffff0000u);
      w1[p] = tc::pack2<__nv_bfloat16>(a, b);
      a -= __uint_as_float(w1[p] << 16);
      b -= __uint_as_float(w1[p] & 0xffff0000u);
      w2[p] = tc::pack2<__nv_bfloat16>(a, b);
    }
    const uint32_t off = (uint32_t)(ch >> 3) * (128 * 128) + tc::sw128_offset(r, ch & 7);
    *reinterpret_cast<uint4*>(set + off) = make_uint4(w0[0], w0[1], w0[2], w0[3]);
    *reinterpret_cast<uint4*>(set + kTcGemmTerm + off) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
    *reinterpret_cast<uint4*>(set + 2 * kTcGemmTerm + off) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
  }
}

// The product of cta_gemm_tc shared by the ws.cs CTAs of a cluster: CTA `rank` forms the output columns
// [rank NB, rank NB + NB), NB = 128 / cs, from the whole of op(A) and its column block of op(B) (MMAs of
// M = 128, N = NB), and writes them to global memory straight from the accumulator rows; the cluster
// barrier at the end makes the whole result visible to every CTA.  C must not alias an operand.
template <bool TA, bool TB, int NT>
__device__ inline void cluster_gemm_tc(float* C, int ldc, const float* A, int lda, const float* B, int ldb, int M, int N,
                                       int K, float alpha, float beta, float diag, GemmWs& ws, float* C2, float alpha2,
                                       float diag2) {
  const int NB = 128 / ws.cs, n0 = ws.rank * NB;
  const int ncols = min(NB, N - n0);          // <= 0: this CTA has no column of the result
  uint8_t* setA = ws.tiles;
  uint8_t* setB = ws.tiles + kTcGemmSet;
  GEMM_T0();
  if (ncols > 0) {
    tc_gemm_load<NT>(setA, A, lda, TA ? K : M, TA ? M : K);
    tc_gemm_load_nblock<NT>(setB, B, ldb, TB, n0, ncols, NB, K);
    tc::fence_proxy_async();
    __syncthreads();
    GEMM_T(0);
    // warp 0 issues from warp-uniform code (one elected lane per MMA)
    if (__shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0) == 0) {
      tc::tc_fence_after();
      constexpr bool AR = TA;
      const uint32_t idesc = tc::make_idesc<__nv_bfloat16>(128, NB, TA, false);
      const uint64_t da = tc_gemm_desc(tc::smem_u32(setA), AR, 0), db = tc_gemm_desc(tc::smem_u32(setB), false, 0);
      const int ksteps = (K + 15) >> 4;
      uint32_t acc = 0;
#pragma unroll
      for (int t = 0; t < 6; ++t) {
        constexpr int oi[6] = {1, 0, 2, 0, 1, 0}, oj[6] = {1, 2, 0, 1, 0, 0};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (k < ksteps) {
            const uint32_t offa = oi[t] * kTcGemmTerm + (AR ? k * 2048 : (k >> 2) * (128 * 128) + (k & 3) * 32);
            const uint32_t offb = oj[t] * kTcGemmTerm + (k >> 2) * (128 * 128) + (k & 3) * 32;
            tc::umma_elect(ws.tmem, da + (offa >> 4), db + (offb >> 4), idesc, acc);
            acc = 1;
          }
        }
      }
      tc::umma_commit_elect(ws.bar);
      GEMM_T(1);
      // one thread alone waits for the MMAs; the others sleep at the barrier below instead of
      // polling beside it
      if (threadIdx.x == 0) {
        tc::Abort ab{reinterpret_cast<volatile int*>(ws.bar + 1), ws.status};
        tc::mbar_wait(ws.bar, ws.phase, ab, 0x5100);
      }
    }
    ws.phase ^= 1u;
    __syncthreads();
    tc::tc_fence_after();
    GEMM_T(2);
    // epilogue: warp w holds accumulator rows 32 (w & 3) .. + 31 and takes groups of 8 of the block's columns
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (warp & 3) * 32 + lane;
    const bool vec = (ldc & 3) == 0 && (N & 3) == 0 && (reinterpret_cast<uintptr_t>(C) & 15u) == 0 &&
                     (!C2 || (reinterpret_cast<uintptr_t>(C2) & 15u) == 0);
    // (a CTA moves about 14 bytes per clock to global memory: the fewer columns a CTA owns, the
    // shorter this phase)
    for (int cb = (warp >> 2) * 8; cb < NB; cb += (NT / 128) * 8) {
      float v[8];
      tc::tmem_ld8(ws.tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)cb, v);
      tc::tmem_ld_wait();
      const int c = n0 + cb;
      if (r < M && c < N) {
        float* dst = C + (size_t)r * ldc + c;
        float o[8], o2[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = alpha * v[j];
          o2[j] = alpha2 * v[j];
        }
        if (vec) {
          if (beta != 0.f) {
#pragma unroll
            for (int q = 0; q < 8; q += 4)
              if (c + q < N) {
                const float4 old = *reinterpret_cast<const float4*>(dst + q);
                o[q] += beta * old.x; o[q + 1] += beta * old.y; o[q + 2] += beta * old.z; o[q + 3] += beta * old.w;
              }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (c + j == r) { o[j] += diag; o2[j] += diag2; }
#pragma unroll
          for (int q = 0; q < 8; q += 4)
            if (c + q < N) {
              *reinterpret_cast<float4*>(dst + q) = make_float4(o[q], o[q + 1], o[q + 2], o[q + 3]);
              if (C2) *reinterpret_cast<float4*>(C2 + (size_t)r * ldc + c + q) = make_float4(o2[q], o2[q + 1], o2[q + 2], o2[q + 3]);
            }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (c + j < N) {
              float val = o[j];
              if (beta != 0.f) val += beta * dst[j];
              if (c + j == r) val += diag;
              dst[j] = val;
              if (C2) C2[(size_t)r * ldc + c + j] = o2[j] + (c + j == r ? diag2 : 0.f);
            }
        }
      }
    }
    tc::tc_fence_before();
  }
  GEMM_T(3);
  if (!ws.defer_sync) mid_sync(ws.cs);
  GEMM_T(5);
#ifdef FNB_TC_TRACE
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&g_gemm_cycles[4], 1ull);
#endif
}

// One half of a cluster of four or eight CTAs as the owner of a product: the halves take independent
// products side by side (each shared by the CTAs of the half by blocks of the output columns); the
// caller ends the step with mid_sync(ws.cs) and takes the mbarrier phase back (ws.phase = half.phase).
__device__ __forceinline__ bool gemm_halves(const GemmWs& ws) { return ws.tiles && ws.cs >= 4; }
__device__ __forceinline__ GemmWs gemm_half(const GemmWs& ws) {
  GemmWs pr = ws;
  pr.cs = ws.cs / 2; pr.rank = ws.rank % pr.cs; pr.defer_sync = 1;
  return pr;
}
__device__ __forceinline__ bool gemm_left_half(const GemmWs& ws) { return ws.rank < ws.cs / 2; }

// set-up / teardown of the tensor-core products inside a kernel of this file (all threads call)
__device__ inline void gemm_ws_open(GemmWs& ws, float* sm, uint8_t* dyn, bool use_tc, uint64_t* bar_and_flag,
                                    uint32_t* tmem_slot, int* status) {
  ws.sm = sm; ws.tiles = nullptr; ws.bar = bar_and_flag; ws.tmem = 0; ws.phase = 0; ws.status = status;
  ws.cs = cluster_size(); ws.rank = cluster_rank(); ws.defer_sync = 0;
  ws.gt = ws.rank * (int)blockDim.x + (int)threadIdx.x; ws.gn = ws.cs * (int)blockDim.x;
  if (!use_tc || blockDim.x != kMidTcThreads) return;   // the tensor-core products are written for kMidTcThreads threads
  ws.tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn) + 1023) & ~(uintptr_t)1023);
  if (threadIdx.x == 0) {
    tc::mbar_init(bar_and_flag, 1);
    *reinterpret_cast<volatile int*>(bar_and_flag + 1) = 0;   // abort flag of the bounded wait
    tc::fence_mbar_init();
  }
  if (threadIdx.x < 32) {
    tc::tmem_alloc(tmem_slot, 128);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  ws.tmem = *tmem_slot;
}
__device__ inline void gemm_ws_close(GemmWs& ws) {
  if (!ws.tiles) return;
  tc::tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tc::tmem_dealloc(ws.tmem, 128);
}

constexpr int kGemmKT = 16;            // k-slab depth
constexpr int kGemmLd = kMaxM + 4;     // shared row stride of a slab
constexpr int kGemmSmemFloats = 2 * kGemmKT * kGemmLd;

// C(MxN) = alpha * op(A) * op(B) + beta * C + diag * I,  M, N <= 128, any K.
//   TA == false: A is (M x K) row-major with leading dimension lda;  TA == true: A is (K x M).
//   TB == false: B is (K x N) row-major with leading dimension ldb;  TB == true: B is (N x K).
// C may alias A or B.  All 256 threads must call; ends with a barrier.
// Pointers are deliberately not __restrict__: operands are produced by this same CTA and must
// be read through the coherent path.
// Optional second output C2 = alpha2 * op(A) * op(B) + diag2 * I (same leading dimension as C, must
// not alias an operand).
template <bool TA, bool TB>
__device__ __noinline__ void cta_gemm(float* C, int ldc, const float* A, int lda, const float* B, int ldb,
                         int M, int N, int K, float alpha, float beta, float diag, GemmWs& ws,
                         float* C2 = nullptr, float alpha2 = 0.f, float diag2 = 0.f) {
  if (ws.tiles) {
    // (tiles are only handed out to CTAs of kMidTcThreads threads)
    if (ws.cs > 1)
      cluster_gemm_tc<TA, TB, kMidTcThreads>(C, ldc, A, lda, B, ldb, M, N, K, alpha, beta, diag, ws, C2, alpha2, diag2);
    else
      cta_gemm_tc<TA, TB, kMidTcThreads>(C, ldc, A, lda, B, ldb, M, N, K, alpha, beta, diag, ws, C2, alpha2, diag2);
    return;
  }
  // (the CUDA-core product below is written for 256 threads: kernels that take this branch are
  // launched with kThreads)
  float* sm = ws.sm;
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
        if (C2) C2[(size_t)r * ldc + c] = alpha2 * acc[i][j] + (r == c ? diag2 : 0.f);
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
  // one pass over A: warp w takes rows w, w + (number of warps), ...; a lane reads columns lane, lane + 32, ... of a
  // row (coalesced), keeps its column partial sums in registers and folds the row sum with shuffles
  const int t = threadIdx.x, w = t >> 5, lane = t & 31;
  float* rowsum = red;                       // [kMaxM]
  float* colpart = red + kMaxM;              // [warps][kMaxM]: up to 17 kMaxM floats of `red` in all
  float cs[kMaxM / 32];
#pragma unroll
  for (int q = 0; q < kMaxM / 32; ++q) cs[q] = 0.f;
  for (int r = w; r < m; r += ((int)blockDim.x >> 5)) {
    float x[kMaxM / 32];
#pragma unroll
    for (int q = 0; q < kMaxM / 32; ++q) {
      const int c = lane + 32 * q;
      x[q] = c < m ? fabsf(A[(size_t)r * m + c]) : 0.f;
    }
    float rs = 0.f;
#pragma unroll
    for (int q = 0; q < kMaxM / 32; ++q) { cs[q] += x[q]; rs += x[q]; }
    for (int o = 16; o > 0; o >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o);
    if (lane == 0) rowsum[r] = rs;
  }
#pragma unroll
  for (int q = 0; q < kMaxM / 32; ++q) colpart[w * kMaxM + lane + 32 * q] = cs[q];
  __syncthreads();
  __shared__ float out_n1, out_ninf;
  __shared__ int out_jc, out_ir;
  if (w == 0) {
    // column sums: fold the warps, then the first-occurrence argmax over columns
    float best = -1.f; int bi = 0;
    for (int c = lane; c < m; c += 32) {
      float s = 0.f;
      for (int ww = 0; ww < ((int)blockDim.x >> 5); ++ww) s += colpart[ww * kMaxM + c];
      if (s > best) { best = s; bi = c; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) { out_n1 = best; out_jc = bi; }
  } else if (w == 1) {
    float best = -1.f; int bi = 0;
    for (int r = lane; r < m; r += 32) {
      const float s = rowsum[r];
      if (s > best) { best = s; bi = r; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) { out_ninf = best; out_ir = bi; }
  }
  __syncthreads();
  Norms r{out_n1, out_ninf, out_jc, out_ir};
  __syncthreads();
  return r;
}

// dst = a*X + diag*I   (m x m, elementwise)
__device__ inline void cta_affine(float* dst, const float* X, float a, float diag, int m) {
  for (int idx = threadIdx.x; idx < m * m; idx += (int)blockDim.x) {
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
                                    float* scratch, int m, int J, float kappa, GemmWs& ws) {
  const int mm = m * m;
  float* Ab = scratch;            // ridge matrix (only with kappa > 0)
  float* Mb = scratch + mm;
  float* Ub = scratch + 2 * mm;
  float* Vb = scratch + 3 * mm;
  float* red = ws.sm;             // norms use the first 2*kMaxM floats of the gemm staging area
  const float* A = k2;
  if (kappa > 0.f) {
    Norms nk = cta_norms(k2, m, red);
    float lam = nk.n1 * nk.ninf / kappa;
    cta_gemm<true, false>(Ab, m, k2, m, k2, m, m, m, m, 1.f, 0.f, lam, ws);
    A = Ab;
  }
  Norms na = cta_norms(A, m, red);
  const float c = fmaxf(na.n1 * na.ninf, 1e-12f);
  for (int idx = ws.gt; idx < mm; idx += ws.gn) {
    int r = idx / m, cc = idx - r * m;
    iterates[idx] = A[cc * m + r] / c;
  }
  mid_sync(ws.cs);
  for (int j = 0; j < J; ++j) {
    const float* Z = iterates + (size_t)j * mm;
    float* Zn = iterates + (size_t)(j + 1) * mm;
    cta_gemm<false, false>(Mb, m, A, m, Z, m, m, m, m, 1.f, 0.f, 0.f, ws, Ub, -1.f, 7.f);   // M = A Z, U = 7I - M
    cta_gemm<false, false>(Vb, m, Mb, m, Ub, m, m, m, m, -1.f, 0.f, 15.f, ws);    // V = 15I - M U
    cta_gemm<false, false>(Ub, m, Mb, m, Vb, m, m, m, m, -1.f, 0.f, 13.f, ws);    // T = 13I - M V
    cta_gemm<false, false>(Zn, m, Z, m, Ub, m, m, m, m, 0.25f, 0.f, 0.f, ws);     // Z' = Z T / 4
  }
  const float* ZJ = iterates + (size_t)J * mm;
  if (kappa > 0.f) {
    cta_gemm<false, true>(k2inv, m, ZJ, m, k2, m, m, m, m, 1.f, 0.f, 0.f, ws);
  } else {
    for (int idx = ws.gt; idx < mm; idx += ws.gn) k2inv[idx] = ZJ[idx];
    mid_sync(ws.cs);
  }
}

// Scratch layout for the pseudoinverse backward: 12 (m x m) buffers.
constexpr int kPinvBwdBufs = 12;
// Gradient of the pseudoinverse w.r.t. the softmax matrix k2 (lambda detached).
//   G = dL/d k2inv  ->  dK2 = dL/d k2.
__device__ inline void pinv_backward(const float* k2, const float* iterates, const float* G,
                                     float* dK2, float* scratch, int m, int J, float kappa,
                                     GemmWs& ws) {
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
  float* red = ws.sm;
  const float* A = k2;
  const float* ZJ = iterates + (size_t)J * mm;
  if (kappa > 0.f) {
    Norms nk = cta_norms(k2, m, red);
    float lam = nk.n1 * nk.ninf / kappa;
    A = Ab;
    if (gemm_halves(ws)) {
      GemmWs pr = gemm_half(ws);
      if (gemm_left_half(ws)) {
        cta_gemm<true, false>(Ab, m, k2, m, k2, m, m, m, m, 1.f, 0.f, lam, pr);
        cta_gemm<false, false>(dZ, m, G, m, k2, m, m, m, m, 1.f, 0.f, 0.f, pr);    // G K2
      } else {
        cta_gemm<true, false>(dK2a, m, G, m, ZJ, m, m, m, m, 1.f, 0.f, 0.f, pr);   // G^T Z_J
      }
      ws.phase = pr.phase;
    } else {
      cta_gemm<true, false>(Ab, m, k2, m, k2, m, m, m, m, 1.f, 0.f, lam, ws);
      cta_gemm<true, false>(dK2a, m, G, m, ZJ, m, m, m, m, 1.f, 0.f, 0.f, ws);   // G^T Z_J
      cta_gemm<false, false>(dZ, m, G, m, k2, m, m, m, m, 1.f, 0.f, 0.f, ws);    // G K2
    }
  } else {
    for (int idx = ws.gt; idx < mm; idx += ws.gn) dZ[idx] = G[idx];
  }
  mid_sync(ws.cs);
  if (J == 0) {
    for (int idx = ws.gt; idx < mm; idx += ws.gn) dA[idx] = 0.f;
    mid_sync(ws.cs);
  }

  if (gemm_halves(ws)) {
    // A cluster of four or eight CTAs works as two halves: the eleven products of an iteration form four
    // steps of independent groups (as in the kernel for up to 64 landmarks), a half takes one group of a
    // step and shares each of its products by blocks of the output columns; a cluster barrier ends a step.
    // A half's accumulating products need no barrier in between: every CTA re-reads only its own columns.
    GemmWs pr = gemm_half(ws);
    const bool left = gemm_left_half(ws);
    for (int j = J - 1; j >= 0; --j) {
      const float* Z = iterates + (size_t)j * mm;
      if (left) cta_gemm<false, false>(Mb, m, A, m, Z, m, m, m, m, 1.f, 0.f, 0.f, pr, Ub, -1.f, 7.f);   // M and U = 7I - M
      else cta_gemm<true, false>(dT, m, Z, m, dZ, m, m, m, m, 0.25f, 0.f, 0.f, pr);                       // dT = Z^T dZ / 4
      mid_sync(ws.cs);
      if (left) cta_gemm<false, false>(Vb, m, Mb, m, Ub, m, m, m, m, -1.f, 0.f, 15.f, pr);                 // V = 15I - M U
      else cta_gemm<true, false>(dV, m, Mb, m, dT, m, m, m, m, -1.f, 0.f, 0.f, pr);                        // dV = -M^T dT
      mid_sync(ws.cs);
      if (left) {
        cta_gemm<false, true>(dM, m, dT, m, Vb, m, m, m, m, -1.f, 0.f, 0.f, pr);    // -dT V^T
        cta_gemm<false, true>(dM, m, dV, m, Ub, m, m, m, m, -1.f, 1.f, 0.f, pr);    // -= dV U^T
        cta_gemm<true, false>(dM, m, Mb, m, dV, m, m, m, m, 1.f, 1.f, 0.f, pr);     // += M^T dV
      } else {
        cta_gemm<false, false>(Tb, m, Mb, m, Vb, m, m, m, m, -1.f, 0.f, 13.f, pr);  // T = 13I - M V
      }
      mid_sync(ws.cs);
      if (left) {
        cta_gemm<false, true>(dZo, m, dZ, m, Tb, m, m, m, m, 0.25f, 0.f, 0.f, pr);  // dZ T^T / 4
        cta_gemm<true, false>(dZo, m, A, m, dM, m, m, m, m, 1.f, 1.f, 0.f, pr);     // dZ' = dZ T^T / 4 + A^T dM
      } else {
        cta_gemm<false, true>(dA, m, dM, m, Z, m, m, m, m, 1.f, j == J - 1 ? 0.f : 1.f, 0.f, pr);   // dA += dM Z^T
      }
      mid_sync(ws.cs);
      { float* tmp = dZ; dZ = dZo; dZo = tmp; }
    }
    ws.phase = pr.phase;   // (of this CTA's own mbarrier)
  } else
  for (int j = J - 1; j >= 0; --j) {
    const float* Z = iterates + (size_t)j * mm;
    cta_gemm<false, false>(Mb, m, A, m, Z, m, m, m, m, 1.f, 0.f, 0.f, ws, Ub, -1.f, 7.f);   // M and U = 7I - M
    cta_gemm<false, false>(Vb, m, Mb, m, Ub, m, m, m, m, -1.f, 0.f, 15.f, ws);
    cta_gemm<false, false>(Tb, m, Mb, m, Vb, m, m, m, m, -1.f, 0.f, 13.f, ws);
    cta_gemm<true, false>(dT, m, Z, m, dZ, m, m, m, m, 0.25f, 0.f, 0.f, ws);    // dT = Z^T dZ / 4
    cta_gemm<false, true>(dZo, m, dZ, m, Tb, m, m, m, m, 0.25f, 0.f, 0.f, ws);  // dZ T^T / 4
    cta_gemm<false, true>(dM, m, dT, m, Vb, m, m, m, m, -1.f, 0.f, 0.f, ws);    // -dT V^T
    cta_gemm<true, false>(dV, m, Mb, m, dT, m, m, m, m, -1.f, 0.f, 0.f, ws);    // dV = -M^T dT
    cta_gemm<false, true>(dM, m, dV, m, Ub, m, m, m, m, -1.f, 1.f, 0.f, ws);    // -= dV U^T
    cta_gemm<true, false>(dM, m, Mb, m, dV, m, m, m, m, 1.f, 1.f, 0.f, ws);     // += M^T dV
    cta_gemm<false, true>(dA, m, dM, m, Z, m, m, m, m, 1.f, j == J - 1 ? 0.f : 1.f, 0.f, ws);   // dA += dM Z^T
    cta_gemm<true, false>(dZo, m, A, m, dM, m, m, m, m, 1.f, 1.f, 0.f, ws);     // dZ' = dZ T^T / 4 + A^T dM
    { float* tmp = dZ; dZ = dZo; dZo = tmp; }
  }
  // Z0 = A^T / c with c = ||A||_1 ||A||_inf
  Norms na = cta_norms(A, m, red);
  const float craw = na.n1 * na.ninf;
  const float c = fmaxf(craw, 1e-12f);
  // S = sum_{a,b} dZ0[a,b] A[b,a]   (every CTA of a cluster forms the norms and this sum for itself)
  float part = 0.f;
  for (int idx = threadIdx.x; idx < mm; idx += (int)blockDim.x) {
    int a = idx / m, b = idx - a * m;
    part += dZ[idx] * A[b * m + a];
  }
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
  __syncthreads();
  float S = 0.f;
  for (int w = 0; w < ((int)blockDim.x >> 5); ++w) S += red[w];
  __syncthreads();
  const bool clamped = !(craw > 1e-12f);
  const float col_term = clamped ? 0.f : -S * na.ninf / (c * c);
  const float row_term = clamped ? 0.f : -S * na.n1 / (c * c);
  for (int idx = ws.gt; idx < mm; idx += ws.gn) {
    int r = idx / m, cc = idx - r * m;
    float a = A[idx];
    float sg = a > 0.f ? 1.f : (a < 0.f ? -1.f : 0.f);
    float g = dA[idx] + dZ[cc * m + r] / c;
    if (cc == na.jc) g += sg * col_term;
    if (r == na.ir) g += sg * row_term;
    dA[idx] = g;
  }
  mid_sync(ws.cs);
  if (kappa > 0.f) {
    // dK2 = dK2a + K2 (dA + dA^T)
    for (int idx = ws.gt; idx < mm; idx += ws.gn) {
      int r = idx / m, cc = idx - r * m;
      dM[idx] = dA[idx] + dA[cc * m + r];
    }
    mid_sync(ws.cs);
    cta_gemm<false, false>(dK2a, m, k2, m, dM, m, m, m, m, 1.f, 1.f, 0.f, ws);
    for (int idx = ws.gt; idx < mm; idx += ws.gn) dK2[idx] = dK2a[idx];
  } else {
    for (int idx = ws.gt; idx < mm; idx += ws.gn) dK2[idx] = dA[idx];
  }
  mid_sync(ws.cs);
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
  int use_tc;                 // products on the tensor cores (needs kTcGemmSmem bytes of dynamic shared memory)
  int* status;
};

__global__ void __launch_bounds__(kMidTcThreads) mid_fwd_kernel(MidFwdParams p) {
  __shared__ float sm[kGemmSmemFloats];
  __shared__ uint64_t gemm_bar[2];
  __shared__ uint32_t gemm_tmem;
  extern __shared__ uint8_t gemm_dyn[];
  const int cs = cluster_size(), rank = cluster_rank();
  const int64_t bh = blockIdx.x / cs;
  const int m = p.m, D = p.D, t = threadIdx.x;
  Segments sg(p.N, m);
  float* qt = p.qt + bh * m * D;
  float* kt = p.kt + bh * m * D;
  for (int idx = rank * (int)blockDim.x + t; idx < 2 * m * D; idx += cs * (int)blockDim.x) {
    int which = idx / (m * D), rem = idx - which * m * D;
    int l = rem / D, d = rem - l * D;
    const float* src = p.land_partial + ((((size_t)which * p.BH + bh) * m + l) * p.C) * D + d;
    float s = 0.f;
    for (int c = 0; c < p.C; ++c) s += src[(size_t)c * D];
    float val = s * (p.scale / (float)sg.len(l));
    (which ? kt : qt)[rem] = val;
  }
  mid_sync(cs);
  if (p.qt16 && rank == 0)
    pack_pair(qt, reinterpret_cast<char*>(p.qt16) + (size_t)bh * p.MP * D * 2, nullptr, p.dtype, m, D, p.MP,
              p.qt16_mul);
  if (p.landmarks_only) return;
  GemmWs ws;
  gemm_ws_open(ws, sm, gemm_dyn, p.use_tc != 0, gemm_bar, &gemm_tmem, p.status);
  float* k2 = p.k2 + bh * m * m;
  cta_gemm<false, true>(k2, m, qt, D, kt, D, m, m, D, 1.f, 0.f, 0.f, ws);
  // row softmax, one warp per row
  const int w = ws.gt >> 5, lane = t & 31;
  for (int r = w; r < m; r += (ws.gn >> 5)) {
    float mx = -INFINITY;
    for (int c = lane; c < m; c += 32) mx = fmaxf(mx, k2[r * m + c]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int c = lane; c < m; c += 32) sum += expf(k2[r * m + c] - mx);
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    for (int c = lane; c < m; c += 32) k2[r * m + c] = expf(k2[r * m + c] - mx) / sum;
    if (lane == 0) p.lse2[bh * m + r] = mx + logf(sum);
  }
  mid_sync(cs);
  pinv_forward(k2, p.iterates + bh * (size_t)(p.J + 1) * m * m, p.k2inv + bh * m * m,
               p.scratch + bh * (size_t)kPinvFwdBufs * m * m, m, p.J, p.kappa, ws);
  gemm_ws_close(ws);
}

__global__ void __launch_bounds__(kMidTcThreads)
pinv_fwd_debug_kernel(const float* k2, float* iterates, float* k2inv, float* scratch, int m,
                      int J, float kappa, int use_tc) {
  __shared__ float sm[kGemmSmemFloats];
  __shared__ uint64_t gemm_bar[2];
  __shared__ uint32_t gemm_tmem;
  extern __shared__ uint8_t gemm_dyn[];
  const int64_t bh = blockIdx.x / cluster_size();
  GemmWs ws;
  gemm_ws_open(ws, sm, gemm_dyn, use_tc != 0, gemm_bar, &gemm_tmem, nullptr);
  pinv_forward(k2 + bh * m * m, iterates + bh * (size_t)(J + 1) * m * m, k2inv + bh * m * m,
               scratch + bh * (size_t)kPinvFwdBufs * m * m, m, J, kappa, ws);
  gemm_ws_close(ws);
}

__global__ void __launch_bounds__(kMidTcThreads)
pinv_bwd_debug_kernel(const float* k2, const float* iterates, const float* G, float* dK2,
                      float* scratch, int m, int J, float kappa, int use_tc) {
  __shared__ float sm[kGemmSmemFloats];
  __shared__ uint64_t gemm_bar[2];
  __shared__ uint32_t gemm_tmem;
  extern __shared__ uint8_t gemm_dyn[];
  const int64_t bh = blockIdx.x / cluster_size();
  GemmWs ws;
  gemm_ws_open(ws, sm, gemm_dyn, use_tc != 0, gemm_bar, &gemm_tmem, nullptr);
  pinv_backward(k2 + bh * m * m, iterates + bh * (size_t)(J + 1) * m * m, G + bh * m * m,
                dK2 + bh * m * m, scratch + bh * (size_t)kPinvBwdBufs * m * m, m, J, kappa, ws);
  gemm_ws_close(ws);
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
  GemmWs ws;
  gemm_ws_open(ws, sm, nullptr, false, nullptr, nullptr, nullptr);
  cta_gemm<false, false>(p.step2 + bh * (size_t)total, D, p.k2inv + bh * m * m, m, bmat, D, m, D, m,
                         1.f, 0.f, 0.f, ws);
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
  int use_tc;                // products on the tensor cores (needs kTcGemmSmem bytes of dynamic shared memory)
  int* status;
};

__global__ void __launch_bounds__(kMidTcThreads) mid_bwd_kernel(MidBwdParams p) {
  __shared__ float sm[kGemmSmemFloats];
  __shared__ uint64_t gemm_bar[2];
  __shared__ uint32_t gemm_tmem;
  extern __shared__ uint8_t gemm_dyn[];
  GemmWs ws;
  gemm_ws_open(ws, sm, gemm_dyn, p.use_tc != 0 && !p.first_half_only, gemm_bar, &gemm_tmem, p.status);
  const int64_t bh = blockIdx.x / ws.cs;
  const int m = p.m, D = p.D, t = threadIdx.x, mm = m * m, md = m * D;
  float* dstep2 = p.dstep2 + bh * md;
  float* dkt_a = p.dkt_a + bh * md;
  const float* partA = p.partA + bh * (size_t)p.nchunk * 2 * md;
  for (int idx = ws.gt; idx < 2 * md; idx += ws.gn) {
    float s = 0.f;
    for (int c = 0; c < p.nchunk; ++c) s += partA[(size_t)c * 2 * md + idx];
    if (idx < md) dstep2[idx] = s; else dkt_a[idx - md] = s;
  }
  mid_sync(ws.cs);
  const float* k2inv = p.k2inv + bh * mm;
  const float* bmat = p.bmat + bh * md;
  const float* k2 = p.k2 + bh * mm;
  const float* qt = p.qt + bh * md;
  const float* kt = p.kt + bh * md;
  float* dO3 = p.dO3 + bh * md;
  float* G = p.G + bh * mm;
  float* dK2 = p.dK2 + bh * mm;
  if (gemm_halves(ws)) {
    GemmWs pr = gemm_half(ws);
    if (gemm_left_half(ws)) cta_gemm<true, false>(dO3, D, k2inv, m, dstep2, D, m, D, m, 1.f, 0.f, 0.f, pr);   // K2inv^T dstep2
    else cta_gemm<false, true>(G, m, dstep2, D, bmat, D, m, m, D, 1.f, 0.f, 0.f, pr);                         // dstep2 Bmat^T
    ws.phase = pr.phase;
    mid_sync(ws.cs);
  } else {
    cta_gemm<true, false>(dO3, D, k2inv, m, dstep2, D, m, D, m, 1.f, 0.f, 0.f, ws);   // K2inv^T dstep2
    cta_gemm<false, true>(G, m, dstep2, D, bmat, D, m, m, D, 1.f, 0.f, 0.f, ws);      // dstep2 Bmat^T
  }
  {
    const int w = ws.gt >> 5, lane = t & 31;
    for (int l = w; l < m; l += (ws.gn >> 5)) {
      float s = 0.f;
      for (int d = lane; d < D; d += 32) s += bmat[l * D + d] * dO3[l * D + d];
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) p.D3[bh * m + l] = s;
    }
  }
  if (p.first_half_only) return;
  pinv_backward(k2, p.iterates + bh * (size_t)(p.J + 1) * mm, G, dK2,
                p.scratch + bh * (size_t)kPinvBwdBufs * mm, m, p.J, p.kappa, ws);
  // softmax-2 Jacobian, in place: dS2 = K2 o (dK2 - rowsum(dK2 o K2))
  {
    const int w = ws.gt >> 5, lane = t & 31;
    for (int r = w; r < m; r += (ws.gn >> 5)) {
      float s = 0.f;
      for (int c = lane; c < m; c += 32) s += dK2[r * m + c] * k2[r * m + c];
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      for (int c = lane; c < m; c += 32) dK2[r * m + c] = k2[r * m + c] * (dK2[r * m + c] - s);
    }
  }
  mid_sync(ws.cs);
  float* dqt_ns = p.dqt_ns + bh * md;
  float* dkt_tot = p.dkt_tot + bh * md;
  for (int idx = ws.gt; idx < md; idx += ws.gn) dkt_tot[idx] = dkt_a[idx];
  mid_sync(ws.cs);
  if (gemm_halves(ws)) {
    GemmWs pr = gemm_half(ws);
    if (gemm_left_half(ws)) cta_gemm<false, false>(dqt_ns, D, dK2, m, kt, D, m, D, m, 1.f, 0.f, 0.f, pr);   // dS2 Kt
    else cta_gemm<true, false>(dkt_tot, D, dK2, m, qt, D, m, D, m, 1.f, 1.f, 0.f, pr);                      // += dS2^T Qt
    ws.phase = pr.phase;
    mid_sync(ws.cs);
  } else {
    cta_gemm<false, false>(dqt_ns, D, dK2, m, kt, D, m, D, m, 1.f, 0.f, 0.f, ws);      // dS2 Kt
    cta_gemm<true, false>(dkt_tot, D, dK2, m, qt, D, m, D, m, 1.f, 1.f, 0.f, ws);      // += dS2^T Qt
  }
  gemm_ws_close(ws);
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
