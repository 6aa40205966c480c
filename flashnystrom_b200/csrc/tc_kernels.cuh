// sm_100a tensor-core streaming kernels (fp16 / bf16 I/O, FP32 accumulation in TMEM).
//
// Common structure: a CTA of 6 warps owns a run of consecutive 128-row tiles of one (b,h)
// slice.  Warp 4 is the TMA producer, warp 5 issues tcgen05.mma (one thread), warps 0-3 are
// the softmax / epilogue warps: thread r owns tile row r, which is TMEM lane r, so every
// row-wise softmax quantity is thread-local.  Tiles of Q/K/V/dO are staged by TMA with the
// 128-byte swizzle; probabilities and softmax gradients go back to shared memory in the same
// swizzled [128 x 64] blocks and serve directly as UMMA operands.  The landmark-sized operands
// (m x D, padded to MP = 64 or 128 landmarks) are packed once per call into 16-bit copies by
// pack_kernel and stay resident in shared memory for the whole CTA.
#pragma once
#include "common.cuh"
#include "tc_common.cuh"

namespace fnb {
namespace tc {

constexpr int kTcThreads = 192;
constexpr int kTile = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// out[bh][r][c] (rows_out x cols_out, 16-bit) = scale * in[bh][r][c]  (or in[bh][c][r] when
// transpose), zero outside the (rows_in x cols_in) source.
template <class T>
__global__ void __launch_bounds__(kThreads)
pack_kernel(const float* __restrict__ in, T* __restrict__ out, int rows_in, int cols_in, int rows_out,
            int cols_out, int transpose, float scale) {
  const int64_t bh = blockIdx.x;
  const float* src = in + bh * (int64_t)rows_in * cols_in;
  T* dst = out + bh * (int64_t)rows_out * cols_out;
  for (int idx = threadIdx.x; idx < rows_out * cols_out; idx += kThreads) {
    int r = idx / cols_out, c = idx - r * cols_out;
    float x = 0.f;
    if (!transpose) { if (r < rows_in && c < cols_in) x = src[r * cols_in + c]; }
    else            { if (c < rows_in && r < cols_in) x = src[c * cols_in + r]; }
    dst[idx] = from_f<T>(x * scale);
  }
}

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~(uintptr_t)1023);
}

struct TcSched {
  int64_t N;
  int nchunk;            // CTAs per (b,h) slice
  int tiles_per_chunk;   // 128-row tiles per CTA
};

template <int D, int MP>
struct FwdCSmem {
  static constexpr int kKt = MP * D * 2, kSt = D * MP * 2, kQ = kTile * D * 2, kP = kTile * MP * 2,
                       kO = kTile * D * 2;
  static constexpr int kBytes = kKt + kSt + 2 * kQ + kP + kO + 256 + 1024;
};

// O = softmax(Q Kt^T) step2, lse1.   kt16 = s*log2e*Kt (MP x D), st16 = step2^T (D x MP).
template <class T, int D, int MP>
__global__ void __launch_bounds__(kTcThreads, 1)
tc_fwd_c_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_o,
                const __grid_constant__ CUtensorMap tm_kt, const __grid_constant__ CUtensorMap tm_st,
                float* __restrict__ lse1, TcSched sch, int m, int* status) {
  using L = FwdCSmem<D, MP>;
  constexpr int KBD = D / 64, KBM = MP / 64;
  constexpr uint32_t kTmemCols = (MP + D <= 128) ? 128 : 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = align1024(smem_raw);
  uint8_t* s_kt = base;
  uint8_t* s_st = s_kt + L::kKt;
  uint8_t* s_q = s_st + L::kSt;          // two stages
  uint8_t* s_p = s_q + 2 * L::kQ;
  uint8_t* s_o = s_p + L::kP;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_o + L::kO);
  uint64_t* small_full = bars + 0;
  uint64_t* q_full = bars + 1;           // [2]
  uint64_t* q_empty = bars + 3;          // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* o_full = bars + 7;
  uint64_t* o_free = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  int* abort_word = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t bh = blockIdx.x / sch.nchunk;
  const int chunk = (int)(blockIdx.x - bh * sch.nchunk);
  const int total_tiles = (int)((sch.N + kTile - 1) / kTile);
  const int tile0 = chunk * sch.tiles_per_chunk;
  const int count = min(sch.tiles_per_chunk, total_tiles - tile0);

  if (threadIdx.x == 0) {
    mbar_init(small_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(q_full + s, 1); mbar_init(q_empty + s, 1); }
    mbar_init(s_full, 1);
    mbar_init(p_full, kTile);
    mbar_init(o_full, 1);
    mbar_init(o_free, kTile);
    *abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + MP;
  Abort ab{abort_word, status};

  if (warp == 4) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_o);
      mbar_expect_tx(small_full, L::kKt + L::kSt);
      for (int kb = 0; kb < KBD; ++kb) tma_load_2d(s_kt + kb * (MP * 128), &tm_kt, small_full, kb * 64, (int)(bh * MP));
      for (int kb = 0; kb < KBM; ++kb) tma_load_2d(s_st + kb * (D * 128), &tm_st, small_full, kb * 64, (int)(bh * D));
      int armed = 0;
      for (int i = 0; i < count; ++i) {
        const int st = i & 1;
        if (!mbar_wait(q_empty + st, ((i >> 1) & 1) ^ 1, ab, 0x100 + i)) break;
        mbar_expect_tx(q_full + st, L::kQ);
        for (int kb = 0; kb < KBD; ++kb)
          tma_load_3d(s_q + st * L::kQ + kb * (kTile * 128), &tm_q, q_full + st, kb * 64, (tile0 + i) * kTile, (int)bh);
        armed = i + 1;
      }
      if (ab.raised()) {
        // let copies already in flight land before the CTA's shared memory is released
        for (int i = max(0, armed - 2); i < armed; ++i) mbar_drain(q_full + (i & 1), (i >> 1) & 1);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc1 = make_idesc<T>(kTile, MP, false, false);
      constexpr uint32_t idesc2 = make_idesc<T>(kTile, D, false, false);
      const uint32_t a_kt = smem_u32(s_kt), a_st = smem_u32(s_st), a_p = smem_u32(s_p);
      bool ok = mbar_wait(small_full, 0, ab, 0x200);
      for (int i = 0; ok && i < count; ++i) {
        const int st = i & 1;
        if (!mbar_wait(q_full + st, (i >> 1) & 1, ab, 0x300 + i)) break;
        tc_fence_after();
        const uint32_t a_q = smem_u32(s_q + st * L::kQ);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          uint64_t ad = smem_desc_sw128(a_q + (k >> 2) * (kTile * 128) + (k & 3) * 32, 16, 1024);
          uint64_t bd = smem_desc_sw128(a_kt + (k >> 2) * (MP * 128) + (k & 3) * 32, 16, 1024);
          umma(tmem_s, ad, bd, idesc1, k > 0);
        }
        umma_commit(q_empty + st);
        umma_commit(s_full);
        if (!mbar_wait(p_full, i & 1, ab, 0x400 + i)) break;
        if (!mbar_wait(o_free, (i & 1) ^ 1, ab, 0x500 + i)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < MP / 16; ++k) {
          uint64_t ad = smem_desc_sw128(a_p + (k >> 2) * (kTile * 128) + (k & 3) * 32, 16, 1024);
          uint64_t bd = smem_desc_sw128(a_st + (k >> 2) * (D * 128) + (k & 3) * 32, 16, 1024);
          umma(tmem_o, ad, bd, idesc2, k > 0);
        }
        umma_commit(o_full);
      }
    }
  } else {
    const int r = threadIdx.x;  // tile row == TMEM lane
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    for (int i = 0; i < count; ++i) {
      if (!mbar_wait(s_full, i & 1, ab, 0x600 + i)) break;
      __syncwarp();
      tc_fence_after();
      float s[MP];
#pragma unroll
      for (int c0 = 0; c0 < MP; c0 += 32) tmem_ld32(tmem_s + lane_base + c0, s + c0);
      tmem_ld_wait();
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < MP; ++j) if (j < m) mx = fmaxf(mx, s[j]);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < MP; ++j) {
        float e = (j < m) ? fast_exp2(s[j] - mx) : 0.f;
        s[j] = e;
        sum += e;
      }
      const float inv = 1.f / sum;
#pragma unroll
      for (int c = 0; c < MP / 8; ++c) {
        uint4 v;
        v.x = pack2<T>(s[8 * c + 0] * inv, s[8 * c + 1] * inv);
        v.y = pack2<T>(s[8 * c + 2] * inv, s[8 * c + 3] * inv);
        v.z = pack2<T>(s[8 * c + 4] * inv, s[8 * c + 5] * inv);
        v.w = pack2<T>(s[8 * c + 6] * inv, s[8 * c + 7] * inv);
        *reinterpret_cast<uint4*>(s_p + (c >> 3) * (kTile * 128) + sw128_offset(r, c & 7)) = v;
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(p_full);
      const int64_t row = (int64_t)(tile0 + i) * kTile + r;
      if (row < sch.N) lse1[bh * sch.N + row] = (mx + log2f(sum)) * kLn2;

      if (!mbar_wait(o_full, i & 1, ab, 0x700 + i)) break;
      __syncwarp();
      tc_fence_after();
      float o[D];
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) tmem_ld32(tmem_o + lane_base + c0, o + c0);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(o_free);
      if (r == 0) tma_store_wait_read();
      named_barrier(1, kTile);
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        uint4 v;
        v.x = pack2<T>(o[8 * c + 0], o[8 * c + 1]);
        v.y = pack2<T>(o[8 * c + 2], o[8 * c + 3]);
        v.z = pack2<T>(o[8 * c + 4], o[8 * c + 5]);
        v.w = pack2<T>(o[8 * c + 6], o[8 * c + 7]);
        *reinterpret_cast<uint4*>(s_o + (c >> 3) * (kTile * 128) + sw128_offset(r, c & 7)) = v;
      }
      fence_proxy_async();
      named_barrier(1, kTile);
      if (r == 0) {
        for (int kb = 0; kb < KBD; ++kb)
          tma_store_3d(&tm_o, s_o + kb * (kTile * 128), kb * 64, (tile0 + i) * kTile, (int)bh);
        tma_store_commit();
      }
    }
    if (r == 0) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace tc
}  // namespace fnb
