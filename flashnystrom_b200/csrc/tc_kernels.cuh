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

// Packs one FP32 (m x D) matrix per (b,h) into 16-bit UMMA operand copies:
//   out_n[bh][MP][D]  (row-major, rows m..MP-1 zero)       when out_n != nullptr
//   out_t[bh][D][MP]  (transposed, columns m..MP-1 zero)   when out_t != nullptr
// Values are multiplied by `premul`.  With normalize != 0 they are additionally divided by
// 2^e, e = ceil(log2(max|x|)), so that the copies lie in [-1, 1] whatever the magnitude of the
// source, and scales[bh] = 2^e is stored for the consumer to undo (exact: a power of two).
template <class T>
__global__ void __launch_bounds__(kThreads)
pack_kernel(const float* __restrict__ in, T* __restrict__ out_n, T* __restrict__ out_t, int m, int D, int MP,
            float premul, int normalize, float* __restrict__ scales) {
  __shared__ float red[kThreads / 32];
  __shared__ float sh_inv;
  const int64_t bh = blockIdx.x;
  const float* src = in + bh * (int64_t)m * D;
  float inv = 1.f;
  if (normalize) {
    float mx = 0.f;
    for (int idx = threadIdx.x; idx < m * D; idx += kThreads) mx = fmaxf(mx, fabsf(src[idx]));
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
      float a = 0.f;
      for (int w = 0; w < kThreads / 32; ++w) a = fmaxf(a, red[w]);
      a *= fabsf(premul);
      int e = 0;
      if (a > 0.f && isfinite(a)) { frexpf(a, &e); }   // a = f * 2^e, f in [0.5, 1)
      e = max(-100, min(100, e));
      sh_inv = ldexpf(1.f, -e);
      if (scales) scales[bh] = ldexpf(1.f, e);
    }
    __syncthreads();
    inv = sh_inv;
  }
  const float mul = premul * inv;
  if (out_n) {
    T* dst = out_n + bh * (int64_t)MP * D;
    for (int idx = threadIdx.x; idx < MP * D; idx += kThreads) {
      int r = idx / D;
      dst[idx] = from_f<T>(r < m ? src[idx] * mul : 0.f);
    }
  }
  if (out_t) {
    T* dst = out_t + bh * (int64_t)D * MP;
    for (int idx = threadIdx.x; idx < D * MP; idx += kThreads) {
      int d = idx / MP, l = idx - d * MP;
      dst[idx] = from_f<T>(l < m ? src[l * D + d] * mul : 0.f);
    }
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
  static constexpr int kBytes = kKt + kSt + 2 * kQ + 2 * kP + kO + 256 + 1024;
};

// O = softmax(Q Kt^T) step2, lse1.   kt16 = s*log2e*Kt (MP x D), st16 = step2^T (D x MP).
// Two-deep software pipeline: S and O are double-buffered in TMEM and P in shared memory, the
// MMA thread issues the score product two tiles ahead, and the compute warps run
// softmax(i) then epilogue(i-1), so they never wait for the tensor core.
template <class T, int D, int MP>
__global__ void __launch_bounds__(kTcThreads, 2)
tc_fwd_c_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_o,
                const __grid_constant__ CUtensorMap tm_kt, const __grid_constant__ CUtensorMap tm_st,
                float* __restrict__ lse1, const float* __restrict__ st_scale, TcSched sch, int m,
                int* status) {
  using L = FwdCSmem<D, MP>;
  constexpr int KBD = D / 64, KBM = MP / 64;
  constexpr uint32_t kCols = 2 * MP + 2 * D;
  constexpr uint32_t kTmemCols = kCols <= 256 ? 256 : 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = align1024(smem_raw);
  uint8_t* s_kt = base;
  uint8_t* s_st = s_kt + L::kKt;
  uint8_t* s_q = s_st + L::kSt;          // two stages
  uint8_t* s_p = s_q + 2 * L::kQ;        // two buffers
  uint8_t* s_o = s_p + 2 * L::kP;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_o + L::kO);
  uint64_t* small_full = bars + 0;
  uint64_t* q_full = bars + 1;           // [2]
  uint64_t* q_empty = bars + 3;          // [2]
  uint64_t* s_full = bars + 5;           // [2]
  uint64_t* p_full = bars + 7;           // [2]
  uint64_t* o_full = bars + 9;           // [2]
  uint64_t* o_free = bars + 11;          // [2]
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
    for (int s = 0; s < 2; ++s) {
      mbar_init(q_full + s, 1); mbar_init(q_empty + s, 1); mbar_init(s_full + s, 1);
      mbar_init(p_full + s, kTile); mbar_init(o_full + s, 1); mbar_init(o_free + s, kTile);
    }
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
      const uint32_t a_kt = smem_u32(s_kt), a_st = smem_u32(s_st);
      // score product of tile i into S[i & 1]; the buffer was released when the MMA thread
      // passed p_full of tile i-2, which precedes this call in program order
      auto front = [&](int i) -> bool {
        const int st = i & 1;
        if (!mbar_wait(q_full + st, (i >> 1) & 1, ab, 0x300 + i)) return false;
        tc_fence_after();
        const uint32_t a_q = smem_u32(s_q + st * L::kQ);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          uint64_t ad = smem_desc_sw128(a_q + (k >> 2) * (kTile * 128) + (k & 3) * 32, 16, 1024);
          uint64_t bd = smem_desc_sw128(a_kt + (k >> 2) * (MP * 128) + (k & 3) * 32, 16, 1024);
          umma(tmem_base + st * MP, ad, bd, idesc1, k > 0);
        }
        umma_commit(q_empty + st);
        umma_commit(s_full + st);
        return true;
      };
      bool ok = mbar_wait(small_full, 0, ab, 0x200);
      ok = ok && front(0);
      if (ok && count > 1) ok = front(1);
      for (int i = 0; ok && i < count; ++i) {
        const int st = i & 1;
        if (!mbar_wait(p_full + st, (i >> 1) & 1, ab, 0x400 + i)) break;
        if (!mbar_wait(o_free + st, ((i >> 1) & 1) ^ 1, ab, 0x500 + i)) break;
        tc_fence_after();
        const uint32_t a_p = smem_u32(s_p + st * L::kP);
#pragma unroll
        for (int k = 0; k < MP / 16; ++k) {
          uint64_t ad = smem_desc_sw128(a_p + (k >> 2) * (kTile * 128) + (k & 3) * 32, 16, 1024);
          uint64_t bd = smem_desc_sw128(a_st + (k >> 2) * (D * 128) + (k & 3) * 32, 16, 1024);
          umma(tmem_base + 2 * MP + st * D, ad, bd, idesc2, k > 0);
        }
        umma_commit(o_full + st);
        if (i + 2 < count) ok = front(i + 2);
      }
    }
  } else {
    const int r = threadIdx.x;  // tile row == TMEM lane
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const float osc = st_scale[bh];
    bool alive = true;
    // epilogue of tile j: O[j & 1] -> 16-bit -> staging -> TMA store
    auto epilogue = [&](int j) -> bool {
      const int st = j & 1;
      if (!mbar_wait(o_full + st, (j >> 1) & 1, ab, 0x700 + j)) return false;
      __syncwarp();
      tc_fence_after();
      float o[D];
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) tmem_ld32(tmem_base + 2 * MP + st * D + lane_base + c0, o + c0);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(o_free + st);
      if (r == 0) tma_store_wait_read();
      named_barrier(1, kTile);
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        uint4 v;
        v.x = pack2<T>(o[8 * c + 0] * osc, o[8 * c + 1] * osc);
        v.y = pack2<T>(o[8 * c + 2] * osc, o[8 * c + 3] * osc);
        v.z = pack2<T>(o[8 * c + 4] * osc, o[8 * c + 5] * osc);
        v.w = pack2<T>(o[8 * c + 6] * osc, o[8 * c + 7] * osc);
        *reinterpret_cast<uint4*>(s_o + (c >> 3) * (kTile * 128) + sw128_offset(r, c & 7)) = v;
      }
      fence_proxy_async();
      named_barrier(1, kTile);
      if (r == 0) {
        for (int kb = 0; kb < KBD; ++kb)
          tma_store_3d(&tm_o, s_o + kb * (kTile * 128), kb * 64, (tile0 + j) * kTile, (int)bh);
        tma_store_commit();
      }
      return true;
    };
    for (int i = 0; i < count; ++i) {
      const int st = i & 1;
      if (!mbar_wait(s_full + st, (i >> 1) & 1, ab, 0x600 + i)) { alive = false; break; }
      __syncwarp();
      tc_fence_after();
      float s[MP];
#pragma unroll
      for (int c0 = 0; c0 < MP; c0 += 32) tmem_ld32(tmem_base + st * MP + lane_base + c0, s + c0);
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
      // P[st] was last read by the output product of tile i-2, whose completion (o_full) the
      // epilogue of tile i-2 has already waited for
      uint8_t* pbuf = s_p + st * L::kP;
#pragma unroll
      for (int c = 0; c < MP / 8; ++c) {
        uint4 v;
        v.x = pack2<T>(s[8 * c + 0] * inv, s[8 * c + 1] * inv);
        v.y = pack2<T>(s[8 * c + 2] * inv, s[8 * c + 3] * inv);
        v.z = pack2<T>(s[8 * c + 4] * inv, s[8 * c + 5] * inv);
        v.w = pack2<T>(s[8 * c + 6] * inv, s[8 * c + 7] * inv);
        *reinterpret_cast<uint4*>(pbuf + (c >> 3) * (kTile * 128) + sw128_offset(r, c & 7)) = v;
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(p_full + st);
      const int64_t row = (int64_t)(tile0 + i) * kTile + r;
      if (row < sch.N) lse1[bh * sch.N + row] = (mx + log2f(sum)) * kLn2;
      if (i > 0 && !epilogue(i - 1)) { alive = false; break; }
    }
    if (alive) epilogue(count - 1);
    if (r == 0) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------------------------
// Softmax-1 backward, both row passes.  Per 128-row tile of Q and dO:
//   S1 = Q kt16^T (log2 domain), dP1 = dO st16^T (step2 normalised by 2^-e, undone by sc),
//   P1 = exp2(S1 - lse1*log2e), D1 = rowsum(P1 o dP1), dS1 = P1 o (dP1 - D1)        [FP32]
// kModeA: accumulate dstep2 += P1^T dO and dKt += dS1^T Q in TMEM over all of the CTA's tiles
//         (UMMA with both operands MN-major: the staged tiles are contracted over their rows)
//         and write one FP32 partial pair per CTA.
// kModeC: dQ = s (dS1 Kt + dQt_tot[l(n)] / len_l), written once through a TMA store.
constexpr int kModeA = 0, kModeC = 1;

template <int D, int MP, int MODE>
struct BwdAcSmem {
  static constexpr int kKt = MP * D * 2, kSt = MP * D * 2, kKtT = (MODE == kModeC) ? D * MP * 2 : 0,
                       kRows = (MODE == kModeC) ? MP * D * 4 : 0, kQ = kTile * D * 2, kG = kTile * D * 2,
                       kP = (MODE == kModeA) ? kTile * MP * 2 : 0, kDs = kTile * MP * 2,
                       kOut = (MODE == kModeC) ? kTile * D * 2 : 0;
  static constexpr int kBytes = kKt + kSt + kKtT + kRows + kQ + kG + kP + kDs + kOut + 256 + 1024;
};

template <class T, int D, int MP, int MODE>
__global__ void __launch_bounds__(kTcThreads, 2)
tc_bwd_ac_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_g,
                 const __grid_constant__ CUtensorMap tm_kt, const __grid_constant__ CUtensorMap tm_st,
                 const __grid_constant__ CUtensorMap tm_ktT, const __grid_constant__ CUtensorMap tm_dq,
                 const float* __restrict__ lse1, const float* __restrict__ st_scale,
                 const float* __restrict__ dqt_ns, const float* __restrict__ partB, int nchunk_b,
                 float* __restrict__ partA, TcSched sch, int m, float scale, int* status) {
  using L = BwdAcSmem<D, MP, MODE>;
  constexpr int KBD = D / 64, KBM = MP / 64;
  constexpr uint32_t kCols = (MODE == kModeA) ? 2 * MP + 2 * D : (2 * MP > D ? 2 * MP : D);
  constexpr uint32_t kTmemCols = kCols <= 128 ? 128 : (kCols <= 256 ? 256 : 512);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = align1024(smem_raw);
  uint8_t* s_kt = base;
  uint8_t* s_st = s_kt + L::kKt;
  uint8_t* s_ktT = s_st + L::kSt;
  float* s_rows = reinterpret_cast<float*>(s_ktT + L::kKtT);
  uint8_t* s_q = reinterpret_cast<uint8_t*>(s_rows) + L::kRows;
  uint8_t* s_g = s_q + L::kQ;
  uint8_t* s_p = s_g + L::kG;
  uint8_t* s_ds = s_p + L::kP;
  uint8_t* s_out = s_ds + L::kDs;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_out + L::kOut);
  uint64_t* small_full = bars + 0;
  uint64_t* in_full = bars + 1;
  uint64_t* in_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* pds_full = bars + 4;
  uint64_t* acc_done = bars + 5;    // mode A: MMA3/4 of a tile complete; mode C: dQ tile complete
  uint64_t* o_free = bars + 6;      // mode C: dQ accumulator read back
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
    mbar_init(in_full, 1);
    mbar_init(in_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, kTile);
    mbar_init(acc_done, 1);
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
  const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + MP;
  const uint32_t tmem_acc1 = tmem_base + 2 * MP, tmem_acc2 = tmem_base + 2 * MP + D;  // mode A
  const uint32_t tmem_dq = tmem_base;                                                 // mode C
  Abort ab{abort_word, status};

  if (warp == 4) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_g);
      mbar_expect_tx(small_full, L::kKt + L::kSt + L::kKtT);
      for (int kb = 0; kb < KBD; ++kb) {
        tma_load_2d(s_kt + kb * (MP * 128), &tm_kt, small_full, kb * 64, (int)(bh * MP));
        tma_load_2d(s_st + kb * (MP * 128), &tm_st, small_full, kb * 64, (int)(bh * MP));
      }
      if (MODE == kModeC)
        for (int kb = 0; kb < KBM; ++kb)
          tma_load_2d(s_ktT + kb * (D * 128), &tm_ktT, small_full, kb * 64, (int)(bh * D));
      int armed = 0;
      for (int i = 0; i < count; ++i) {
        if (!mbar_wait(in_empty, (i & 1) ^ 1, ab, 0x1100 + i)) break;
        mbar_expect_tx(in_full, L::kQ + L::kG);
        for (int kb = 0; kb < KBD; ++kb) {
          tma_load_3d(s_q + kb * (kTile * 128), &tm_q, in_full, kb * 64, (tile0 + i) * kTile, (int)bh);
          tma_load_3d(s_g + kb * (kTile * 128), &tm_g, in_full, kb * 64, (tile0 + i) * kTile, (int)bh);
        }
        armed = i + 1;
      }
      if (ab.raised() && armed > 0) mbar_drain(in_full, (armed - 1) & 1);
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc<T>(kTile, MP, false, false);
      constexpr uint32_t idesc_acc = make_idesc<T>(MP, D, true, true);
      constexpr uint32_t idesc_dq = make_idesc<T>(kTile, D, false, false);
      const uint32_t a_kt = smem_u32(s_kt), a_st = smem_u32(s_st), a_ktT = smem_u32(s_ktT);
      const uint32_t a_q = smem_u32(s_q), a_g = smem_u32(s_g), a_p = smem_u32(s_p), a_ds = smem_u32(s_ds);
      bool ok = mbar_wait(small_full, 0, ab, 0x1200);
      for (int i = 0; ok && i < count; ++i) {
        if (!mbar_wait(in_full, i & 1, ab, 0x1300 + i)) break;
        if (MODE == kModeC && !mbar_wait(o_free, (i & 1) ^ 1, ab, 0x1380 + i)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * (kTile * 128) + (k & 3) * 32, offb = (k >> 2) * (MP * 128) + (k & 3) * 32;
          umma(tmem_s, smem_desc_sw128(a_q + off, 16, 1024), smem_desc_sw128(a_kt + offb, 16, 1024), idesc_s, k > 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * (kTile * 128) + (k & 3) * 32, offb = (k >> 2) * (MP * 128) + (k & 3) * 32;
          umma(tmem_dp, smem_desc_sw128(a_g + off, 16, 1024), smem_desc_sw128(a_st + offb, 16, 1024), idesc_s, k > 0);
        }
        if (MODE == kModeC) umma_commit(in_empty);
        umma_commit(sdp_full);
        if (!mbar_wait(pds_full, i & 1, ab, 0x1400 + i)) break;
        tc_fence_after();
        if (MODE == kModeA) {
#pragma unroll
          for (int k = 0; k < kTile / 16; ++k)
            umma(tmem_acc1, smem_desc_sw128(a_p + k * 2048, kTile * 128, 1024),
                 smem_desc_sw128(a_g + k * 2048, kTile * 128, 1024), idesc_acc, (i > 0 || k > 0));
#pragma unroll
          for (int k = 0; k < kTile / 16; ++k)
            umma(tmem_acc2, smem_desc_sw128(a_ds + k * 2048, kTile * 128, 1024),
                 smem_desc_sw128(a_q + k * 2048, kTile * 128, 1024), idesc_acc, (i > 0 || k > 0));
          umma_commit(in_empty);
          umma_commit(acc_done);
        } else {
#pragma unroll
          for (int k = 0; k < MP / 16; ++k) {
            const uint32_t off = (k >> 2) * (kTile * 128) + (k & 3) * 32, offb = (k >> 2) * (D * 128) + (k & 3) * 32;
            umma(tmem_dq, smem_desc_sw128(a_ds + off, 16, 1024), smem_desc_sw128(a_ktT + offb, 16, 1024), idesc_dq, k > 0);
          }
          umma_commit(acc_done);
        }
      }
    }
  } else {
    const int r = threadIdx.x;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const float sc = st_scale[bh];
    Segments sg(sch.N, m);
    if (MODE == kModeC) {
      // Landmark rows of s * dQt_tot / len (FP32), resident for the whole CTA, for the landmarks
      // this CTA's rows belong to.  dQt_tot = Newton-Schulz part + the column pass's per-CTA
      // partials, summed here in a fixed order.
      const int64_t row_lo = (int64_t)tile0 * kTile;
      int64_t row_hi = (int64_t)(tile0 + count) * kTile - 1;
      if (row_hi > sch.N - 1) row_hi = sch.N - 1;
      const int l_lo = sg.landmark_of(row_lo), l_hi = sg.landmark_of(row_hi);
      const int md = m * D;
      const float* ns_part = dqt_ns + bh * (int64_t)md;
      const float* pb = partB + bh * (int64_t)nchunk_b * md;
      for (int idx = l_lo * D + r; idx < (l_hi + 1) * D; idx += kTile) {
        float acc = ns_part[idx];
        for (int c = 0; c < nchunk_b; ++c) acc += pb[(size_t)c * md + idx];
        s_rows[idx] = acc * (scale / (float)sg.len(idx / D));
      }
      named_barrier(1, kTile);
    }
    bool alive = true;
    for (int i = 0; i < count; ++i) {
      const int64_t row = (int64_t)(tile0 + i) * kTile + r;
      const bool valid = row < sch.N;
      const float lse = valid ? lse1[bh * sch.N + row] * kLog2e : 0.f;
      if (!mbar_wait(sdp_full, i & 1, ab, 0x1600 + i)) { alive = false; break; }
      __syncwarp();
      tc_fence_after();
      float p[MP];
#pragma unroll
      for (int c0 = 0; c0 < MP; c0 += 32) tmem_ld32(tmem_s + lane_base + c0, p + c0);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < MP; ++j) p[j] = (valid && j < m) ? fast_exp2(p[j] - lse) : 0.f;
      float d1 = 0.f;
#pragma unroll
      for (int c0 = 0; c0 < MP; c0 += 32) {
        float g[32];
        tmem_ld32(tmem_dp + lane_base + c0, g);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) d1 = fmaf(p[c0 + j], g[j], d1);
      }
      if (MODE == kModeA && i > 0) {
        // the previous tile's P / dS are still being read by its accumulation MMAs
        if (!mbar_wait(acc_done, (i - 1) & 1, ab, 0x1700 + i)) { alive = false; break; }
        __syncwarp();
      }
      if (MODE == kModeA) {
#pragma unroll
        for (int c = 0; c < MP / 8; ++c) {
          uint4 v;
          v.x = pack2<T>(p[8 * c + 0], p[8 * c + 1]);
          v.y = pack2<T>(p[8 * c + 2], p[8 * c + 3]);
          v.z = pack2<T>(p[8 * c + 4], p[8 * c + 5]);
          v.w = pack2<T>(p[8 * c + 6], p[8 * c + 7]);
          *reinterpret_cast<uint4*>(s_p + (c >> 3) * (kTile * 128) + sw128_offset(r, c & 7)) = v;
        }
      }
#pragma unroll
      for (int c0 = 0; c0 < MP; c0 += 32) {
        float g[32];
        tmem_ld32(tmem_dp + lane_base + c0, g);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) g[j] = p[c0 + j] * (g[j] - d1);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 v;
          v.x = pack2<T>(g[8 * c + 0], g[8 * c + 1]);
          v.y = pack2<T>(g[8 * c + 2], g[8 * c + 3]);
          v.z = pack2<T>(g[8 * c + 4], g[8 * c + 5]);
          v.w = pack2<T>(g[8 * c + 6], g[8 * c + 7]);
          const int cc = (c0 >> 3) + c;
          *reinterpret_cast<uint4*>(s_ds + (cc >> 3) * (kTile * 128) + sw128_offset(r, cc & 7)) = v;
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(pds_full);

      if (MODE == kModeC) {
        if (!mbar_wait(acc_done, i & 1, ab, 0x1800 + i)) { alive = false; break; }
        __syncwarp();
        tc_fence_after();
        if (r == 0) tma_store_wait_read();
        named_barrier(1, kTile);
        const int l = valid ? sg.landmark_of(row) : 0;
        const float* add = s_rows + l * D;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          float o[32];
          tmem_ld32(tmem_dq + lane_base + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = fmaf(o[j], sc, add[c0 + j]);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 v;
            v.x = pack2<T>(o[8 * c + 0], o[8 * c + 1]);
            v.y = pack2<T>(o[8 * c + 2], o[8 * c + 3]);
            v.z = pack2<T>(o[8 * c + 4], o[8 * c + 5]);
            v.w = pack2<T>(o[8 * c + 6], o[8 * c + 7]);
            const int cc = (c0 >> 3) + c;
            *reinterpret_cast<uint4*>(s_out + (cc >> 3) * (kTile * 128) + sw128_offset(r, cc & 7)) = v;
          }
        }
        tc_fence_before();
        mbar_arrive(o_free);
        fence_proxy_async();
        named_barrier(1, kTile);
        if (r == 0) {
          for (int kb = 0; kb < KBD; ++kb)
            tma_store_3d(&tm_dq, s_out + kb * (kTile * 128), kb * 64, (tile0 + i) * kTile, (int)bh);
          tma_store_commit();
        }
      }
    }
    if (MODE == kModeC) {
      if (r == 0) tma_store_wait_all();
    } else if (alive && mbar_wait(acc_done, (count - 1) & 1, ab, 0x1900)) {
      __syncwarp();
      tc_fence_after();
      // accumulator row -> TMEM lane: M = 128 uses lane = row; M = 64 keeps 16 rows per 32-lane
      // quarter in its lanes 0..15
      const int l = (MP == 128) ? r : (warp * 16 + lane);
      const bool owner = (MP == 128) ? true : (lane < 16);
      float* dst = partA + ((size_t)bh * sch.nchunk + chunk) * 2 * m * D;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const float mul = which ? sc * scale : 1.f;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          float o[32];
          tmem_ld32((which ? tmem_acc2 : tmem_acc1) + lane_base + c0, o);
          tmem_ld_wait();
          if (owner && l < m) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(dst + (size_t)which * m * D + l * D + c0 + j) =
                  make_float4(o[j] * mul, o[j + 1] * mul, o[j + 2] * mul, o[j + 3] * mul);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------------------------
// Softmax-3 backward (column pass).  Per 128-row tile of K and V (thread = row n):
//   S3^T = K qt16^T (log2 domain), dP3^T = V do3n^T (dO3 normalised by 2^-e, undone by dsc)
//   P' = 2^k exp(S3 - lse3) , dS' = P' o (dP3 - D3)     (2^k keeps the 16-bit operand copies of
//                                                         the ~1/N probabilities out of the
//                                                         subnormal range; undone in FP32)
//   dV = P'^T-tile * dO3          -> written once
//   dK = s (dS'^T-tile * Qt + dKt_tot[l(n)] / len_l) -> written once
//   dQt partial += dS' (sK)       -> TMEM accumulator over the CTA's tiles
template <int D, int MP>
struct BwdBSmem {
  static constexpr int kOp = MP * D * 2, kRows = MP * D * 4, kVec = 1024, kIn = kTile * D * 2,
                       kPd = kTile * (MP > D ? MP : D) * 2;
  static constexpr int kBytes = 4 * kOp + kRows + kVec + 2 * kIn + 2 * kPd + 256 + 1024;
};

template <class T, int D, int MP>
__global__ void __launch_bounds__(kTcThreads, 2)
tc_bwd_b_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                const __grid_constant__ CUtensorMap tm_qt, const __grid_constant__ CUtensorMap tm_do3,
                const __grid_constant__ CUtensorMap tm_do3T, const __grid_constant__ CUtensorMap tm_qtT,
                const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                const float* __restrict__ lse3, const float* __restrict__ D3,
                const float* __restrict__ do3_scale, const float* __restrict__ dkt_tot,
                float* __restrict__ partB, TcSched sch, int m, float scale, int kshift, int* status) {
  using L = BwdBSmem<D, MP>;
  constexpr int KBD = D / 64, KBM = MP / 64;
  constexpr int W = MP > D ? MP : D;
  constexpr uint32_t kCols = 2 * W + D;
  constexpr uint32_t kTmemCols = kCols <= 256 ? 256 : 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = align1024(smem_raw);
  uint8_t* s_qt = base;
  uint8_t* s_do3 = s_qt + L::kOp;
  uint8_t* s_do3T = s_do3 + L::kOp;
  uint8_t* s_qtT = s_do3T + L::kOp;
  float* s_rows = reinterpret_cast<float*>(s_qtT + L::kOp);
  float* s_c3 = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(s_rows) + L::kRows);
  float* s_d3 = s_c3 + MP;
  uint8_t* s_k = reinterpret_cast<uint8_t*>(s_c3) + L::kVec;
  uint8_t* s_v = s_k + L::kIn;
  uint8_t* s_p = s_v + L::kIn;      // P' tile, then staging of the dV tile
  uint8_t* s_ds = s_p + L::kPd;     // dS' tile, then staging of the dK tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_ds + L::kPd);
  uint64_t* small_full = bars + 0;
  uint64_t* in_full = bars + 1;
  uint64_t* in_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* pds_full = bars + 4;
  uint64_t* out_full = bars + 5;
  uint64_t* o_free = bars + 6;
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
    mbar_init(in_full, 1);
    mbar_init(in_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, kTile);
    mbar_init(out_full, 1);
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
  const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + W, tmem_acc = tmem_base + 2 * W;
  const uint32_t tmem_dv = tmem_s, tmem_dk = tmem_dp;
  Abort ab{abort_word, status};

  if (warp == 4) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_expect_tx(small_full, 4 * L::kOp);
      for (int kb = 0; kb < KBD; ++kb) {
        tma_load_2d(s_qt + kb * (MP * 128), &tm_qt, small_full, kb * 64, (int)(bh * MP));
        tma_load_2d(s_do3 + kb * (MP * 128), &tm_do3, small_full, kb * 64, (int)(bh * MP));
      }
      for (int kb = 0; kb < KBM; ++kb) {
        tma_load_2d(s_do3T + kb * (D * 128), &tm_do3T, small_full, kb * 64, (int)(bh * D));
        tma_load_2d(s_qtT + kb * (D * 128), &tm_qtT, small_full, kb * 64, (int)(bh * D));
      }
      int armed = 0;
      for (int i = 0; i < count; ++i) {
        if (!mbar_wait(in_empty, (i & 1) ^ 1, ab, 0x2100 + i)) break;
        mbar_expect_tx(in_full, 2 * L::kIn);
        for (int kb = 0; kb < KBD; ++kb) {
          tma_load_3d(s_k + kb * (kTile * 128), &tm_k, in_full, kb * 64, (tile0 + i) * kTile, (int)bh);
          tma_load_3d(s_v + kb * (kTile * 128), &tm_v, in_full, kb * 64, (tile0 + i) * kTile, (int)bh);
        }
        armed = i + 1;
      }
      if (ab.raised() && armed > 0) mbar_drain(in_full, (armed - 1) & 1);
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc<T>(kTile, MP, false, false);
      constexpr uint32_t idesc_o = make_idesc<T>(kTile, D, false, false);
      constexpr uint32_t idesc_acc = make_idesc<T>(MP, D, true, true);
      const uint32_t a_qt = smem_u32(s_qt), a_do3 = smem_u32(s_do3), a_do3T = smem_u32(s_do3T),
                     a_qtT = smem_u32(s_qtT), a_k = smem_u32(s_k), a_v = smem_u32(s_v), a_p = smem_u32(s_p),
                     a_ds = smem_u32(s_ds);
      bool ok = mbar_wait(small_full, 0, ab, 0x2200);
      for (int i = 0; ok && i < count; ++i) {
        if (!mbar_wait(in_full, i & 1, ab, 0x2300 + i)) break;
        if (!mbar_wait(o_free, (i & 1) ^ 1, ab, 0x2380 + i)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * (kTile * 128) + (k & 3) * 32, offb = (k >> 2) * (MP * 128) + (k & 3) * 32;
          umma(tmem_s, smem_desc_sw128(a_k + off, 16, 1024), smem_desc_sw128(a_qt + offb, 16, 1024), idesc_s, k > 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * (kTile * 128) + (k & 3) * 32, offb = (k >> 2) * (MP * 128) + (k & 3) * 32;
          umma(tmem_dp, smem_desc_sw128(a_v + off, 16, 1024), smem_desc_sw128(a_do3 + offb, 16, 1024), idesc_s, k > 0);
        }
        umma_commit(sdp_full);
        if (!mbar_wait(pds_full, i & 1, ab, 0x2400 + i)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < MP / 16; ++k) {
          const uint32_t off = (k >> 2) * (kTile * 128) + (k & 3) * 32, offb = (k >> 2) * (D * 128) + (k & 3) * 32;
          umma(tmem_dv, smem_desc_sw128(a_p + off, 16, 1024), smem_desc_sw128(a_do3T + offb, 16, 1024), idesc_o, k > 0);
        }
#pragma unroll
        for (int k = 0; k < MP / 16; ++k) {
          const uint32_t off = (k >> 2) * (kTile * 128) + (k & 3) * 32, offb = (k >> 2) * (D * 128) + (k & 3) * 32;
          umma(tmem_dk, smem_desc_sw128(a_ds + off, 16, 1024), smem_desc_sw128(a_qtT + offb, 16, 1024), idesc_o, k > 0);
        }
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)
          umma(tmem_acc, smem_desc_sw128(a_ds + k * 2048, kTile * 128, 1024),
               smem_desc_sw128(a_k + k * 2048, kTile * 128, 1024), idesc_acc, (i > 0 || k > 0));
        umma_commit(in_empty);
        umma_commit(out_full);
      }
    }
  } else {
    const int r = threadIdx.x;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const float dsc = do3_scale[bh];
    const float unshift = exp2f(-(float)kshift);
    Segments sg(sch.N, m);
    {
      const float* src = dkt_tot + bh * (int64_t)m * D;
      for (int idx = r; idx < m * D; idx += kTile) s_rows[idx] = src[idx] * (scale / (float)sg.len(idx / D));
      if (r < MP) {
        s_c3[r] = (r < m) ? lse3[bh * m + r] * kLog2e - (float)kshift : INFINITY;
        s_d3[r] = (r < m) ? D3[bh * m + r] : 0.f;
      }
      named_barrier(1, kTile);
    }
    bool alive = true;
    for (int i = 0; i < count; ++i) {
      const int64_t row = (int64_t)(tile0 + i) * kTile + r;
      const bool valid = row < sch.N;
      if (!mbar_wait(sdp_full, i & 1, ab, 0x2600 + i)) { alive = false; break; }
      __syncwarp();
      tc_fence_after();
      float p[MP];
#pragma unroll
      for (int c0 = 0; c0 < MP; c0 += 32) tmem_ld32(tmem_s + lane_base + c0, p + c0);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < MP; j += 4) {
        const float4 c = *reinterpret_cast<const float4*>(s_c3 + j);
        p[j + 0] = valid ? fast_exp2(p[j + 0] - c.x) : 0.f;
        p[j + 1] = valid ? fast_exp2(p[j + 1] - c.y) : 0.f;
        p[j + 2] = valid ? fast_exp2(p[j + 2] - c.z) : 0.f;
        p[j + 3] = valid ? fast_exp2(p[j + 3] - c.w) : 0.f;
      }
      // the staging copies of the previous tile's dV / dK share these buffers
      if (r == 0) tma_store_wait_read();
      named_barrier(1, kTile);
#pragma unroll
      for (int c = 0; c < MP / 8; ++c) {
        uint4 v;
        v.x = pack2<T>(p[8 * c + 0], p[8 * c + 1]);
        v.y = pack2<T>(p[8 * c + 2], p[8 * c + 3]);
        v.z = pack2<T>(p[8 * c + 4], p[8 * c + 5]);
        v.w = pack2<T>(p[8 * c + 6], p[8 * c + 7]);
        *reinterpret_cast<uint4*>(s_p + (c >> 3) * (kTile * 128) + sw128_offset(r, c & 7)) = v;
      }
#pragma unroll
      for (int c0 = 0; c0 < MP; c0 += 32) {
        float g[32];
        tmem_ld32(tmem_dp + lane_base + c0, g);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float ds = p[c0 + j] * (fmaf(g[j], dsc, -s_d3[c0 + j]));
          g[j] = fminf(fmaxf(ds, -60000.f), 60000.f);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 v;
          v.x = pack2<T>(g[8 * c + 0], g[8 * c + 1]);
          v.y = pack2<T>(g[8 * c + 2], g[8 * c + 3]);
          v.z = pack2<T>(g[8 * c + 4], g[8 * c + 5]);
          v.w = pack2<T>(g[8 * c + 6], g[8 * c + 7]);
          const int cc = (c0 >> 3) + c;
          *reinterpret_cast<uint4*>(s_ds + (cc >> 3) * (kTile * 128) + sw128_offset(r, cc & 7)) = v;
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(pds_full);

      if (!mbar_wait(out_full, i & 1, ab, 0x2800 + i)) { alive = false; break; }
      __syncwarp();
      tc_fence_after();
      const int l = valid ? sg.landmark_of(row) : 0;
      const float* add = s_rows + l * D;
      const float vmul = dsc * unshift;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        float o[32];
        tmem_ld32(tmem_dv + lane_base + c0, o);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 v;
          v.x = pack2<T>(o[8 * c + 0] * vmul, o[8 * c + 1] * vmul);
          v.y = pack2<T>(o[8 * c + 2] * vmul, o[8 * c + 3] * vmul);
          v.z = pack2<T>(o[8 * c + 4] * vmul, o[8 * c + 5] * vmul);
          v.w = pack2<T>(o[8 * c + 6] * vmul, o[8 * c + 7] * vmul);
          const int cc = (c0 >> 3) + c;
          *reinterpret_cast<uint4*>(s_p + (cc >> 3) * (kTile * 128) + sw128_offset(r, cc & 7)) = v;
        }
        tmem_ld32(tmem_dk + lane_base + c0, o);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] = fmaf(o[j], unshift, add[c0 + j]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 v;
          v.x = pack2<T>(o[8 * c + 0], o[8 * c + 1]);
          v.y = pack2<T>(o[8 * c + 2], o[8 * c + 3]);
          v.z = pack2<T>(o[8 * c + 4], o[8 * c + 5]);
          v.w = pack2<T>(o[8 * c + 6], o[8 * c + 7]);
          const int cc = (c0 >> 3) + c;
          *reinterpret_cast<uint4*>(s_ds + (cc >> 3) * (kTile * 128) + sw128_offset(r, cc & 7)) = v;
        }
      }
      tc_fence_before();
      mbar_arrive(o_free);
      fence_proxy_async();
      named_barrier(1, kTile);
      if (r == 0) {
        for (int kb = 0; kb < KBD; ++kb) {
          tma_store_3d(&tm_dv, s_p + kb * (kTile * 128), kb * 64, (tile0 + i) * kTile, (int)bh);
          tma_store_3d(&tm_dk, s_ds + kb * (kTile * 128), kb * 64, (tile0 + i) * kTile, (int)bh);
        }
        tma_store_commit();
      }
    }
    if (r == 0) tma_store_wait_all();
    if (alive) {
      // out_full of the last tile was waited above, so the accumulator is final
      const int l = (MP == 128) ? r : (warp * 16 + lane);
      const bool owner = (MP == 128) ? true : (lane < 16);
      float* dst = partB + ((size_t)bh * sch.nchunk + chunk) * m * D;
      const float mul = scale * unshift;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        float o[32];
        tmem_ld32(tmem_acc + lane_base + c0, o);
        tmem_ld_wait();
        if (owner && l < m) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + l * D + c0 + j) =
                make_float4(o[j] * mul, o[j + 1] * mul, o[j + 2] * mul, o[j + 3] * mul);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------------------------
// Softmax-3 forward (column pass): per-CTA partial of Bmat = softmax(Qt (sK)^T) V with a running
// reference exponent per landmark.  Thread = row n of the K/V tile, so the per-landmark maximum
// over the tile is a reduction across threads: 62 warp shuffles per thread fold the 32 rows of a
// warp, shared memory folds the 4 warps.  The reference only moves when a tile exceeds it by more
// than 2^8 (then the TMEM accumulators are rescaled in place), so probabilities stay <= 256 in
// the 16-bit operand copy and rescales are rare.  Row sums come from the tensor core too
// (P'^T times a block of ones).
template <int D, int MP>
struct FwdBSmem {
  static constexpr int kQt = MP * D * 2, kOnes = 2048, kIn = kTile * D * 2, kP = kTile * MP * 2,
                       kAux = (4 * MP + 3 * MP) * 4 + 64;
  static constexpr int kBytes = kQt + kOnes + 2 * kIn + kP + kAux + 256 + 1024;
};

template <class T, int D, int MP>
__global__ void __launch_bounds__(kTcThreads, 2)
tc_fwd_b_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                const __grid_constant__ CUtensorMap tm_qt, float* __restrict__ part_acc,
                float* __restrict__ part_max, float* __restrict__ part_sum, TcSched sch, int m,
                int* status) {
  using L = FwdBSmem<D, MP>;
  constexpr int KBD = D / 64;
  constexpr int CPL = MP / 32;                 // columns per lane after the warp fold
  constexpr uint32_t kTmemCols = 256 * ((MP + D + 32 + 255) / 256);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = align1024(smem_raw);
  uint8_t* s_qt = base;
  uint8_t* s_ones = s_qt + L::kQt;
  uint8_t* s_k = s_ones + L::kOnes;
  uint8_t* s_v = s_k + L::kIn;
  uint8_t* s_p = s_v + L::kIn;
  float* s_wmax = reinterpret_cast<float*>(s_p + L::kP);   // [4][MP]
  float* s_ref = s_wmax + 4 * MP;                          // [MP] running reference (log2 domain)
  float* s_fac = s_ref + MP;                               // [MP] rescale factor of this tile
  float* s_new = s_fac + MP;                               // [MP] scratch
  int* s_flag = reinterpret_cast<int*>(s_new + MP);        // [3], rotating
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(s_wmax) + L::kAux);
  uint64_t* small_full = bars + 0;
  uint64_t* in_full = bars + 1;
  uint64_t* in_empty = bars + 2;
  uint64_t* s_full = bars + 3;
  uint64_t* p_full = bars + 4;
  uint64_t* acc_done = bars + 5;
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
    mbar_init(in_full, 1);
    mbar_init(in_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, kTile);
    mbar_init(acc_done, 1);
    *abort_word = 0;
    s_flag[0] = 0;
    s_flag[1] = 0;
    s_flag[2] = 0;
    fence_mbar_init();
  }
  // block of 16-bit ones read by the row-sum MMA (any operand layout reads all-ones from it)
  for (int idx = threadIdx.x; idx < L::kOnes / 4; idx += kTcThreads)
    reinterpret_cast<uint32_t*>(s_ones)[idx] = pack2<T>(1.f, 1.f);
  fence_proxy_async();
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_acc = tmem_base + MP, tmem_sum = tmem_base + MP + D;
  Abort ab{abort_word, status};

  if (warp == 4) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_expect_tx(small_full, L::kQt);
      for (int kb = 0; kb < KBD; ++kb)
        tma_load_2d(s_qt + kb * (MP * 128), &tm_qt, small_full, kb * 64, (int)(bh * MP));
      int armed = 0;
      for (int i = 0; i < count; ++i) {
        if (!mbar_wait(in_empty, (i & 1) ^ 1, ab, 0x3100 + i)) break;
        mbar_expect_tx(in_full, 2 * L::kIn);
        for (int kb = 0; kb < KBD; ++kb) {
          tma_load_3d(s_k + kb * (kTile * 128), &tm_k, in_full, kb * 64, (tile0 + i) * kTile, (int)bh);
          tma_load_3d(s_v + kb * (kTile * 128), &tm_v, in_full, kb * 64, (tile0 + i) * kTile, (int)bh);
        }
        armed = i + 1;
      }
      if (ab.raised() && armed > 0) mbar_drain(in_full, (armed - 1) & 1);
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc<T>(kTile, MP, false, false);
      constexpr uint32_t idesc_acc = make_idesc<T>(MP, D, true, true);
      constexpr uint32_t idesc_sum = make_idesc<T>(MP, 16, true, false);
      const uint32_t a_qt = smem_u32(s_qt), a_k = smem_u32(s_k), a_v = smem_u32(s_v), a_p = smem_u32(s_p),
                     a_ones = smem_u32(s_ones);
      bool ok = mbar_wait(small_full, 0, ab, 0x3200);
      for (int i = 0; ok && i < count; ++i) {
        if (!mbar_wait(in_full, i & 1, ab, 0x3300 + i)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * (kTile * 128) + (k & 3) * 32, offb = (k >> 2) * (MP * 128) + (k & 3) * 32;
          umma(tmem_s, smem_desc_sw128(a_k + off, 16, 1024), smem_desc_sw128(a_qt + offb, 16, 1024), idesc_s, k > 0);
        }
        umma_commit(s_full);
        if (!mbar_wait(p_full, i & 1, ab, 0x3400 + i)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)
          umma(tmem_acc, smem_desc_sw128(a_p + k * 2048, kTile * 128, 1024),
               smem_desc_sw128(a_v + k * 2048, kTile * 128, 1024), idesc_acc, (i > 0 || k > 0));
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)
          umma(tmem_sum, smem_desc_sw128(a_p + k * 2048, kTile * 128, 1024),
               smem_desc_sw128(a_ones + (k & 3) * 32, 16, 1024), idesc_sum, (i > 0 || k > 0));
        umma_commit(in_empty);
        umma_commit(acc_done);
      }
    }
  } else {
    const int r = threadIdx.x;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const int lrow = (MP == 128) ? r : (warp * 16 + lane);          // accumulator row of this lane
    const bool owner = (MP == 128) ? true : (lane < 16);
    if (r < MP) s_ref[r] = -INFINITY;
    bool alive = true;
    for (int i = 0; i < count; ++i) {
      const int64_t row = (int64_t)(tile0 + i) * kTile + r;
      const bool valid = row < sch.N;
      if (!mbar_wait(s_full, i & 1, ab, 0x3600 + i)) { alive = false; break; }
      __syncwarp();
      tc_fence_after();
      float s[MP], v[MP];
#pragma unroll
      for (int c0 = 0; c0 < MP; c0 += 32) tmem_ld32(tmem_s + lane_base + c0, s + c0);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < MP; ++j) { s[j] = valid ? s[j] : -INFINITY; v[j] = s[j]; }
      // fold the 32 rows of this warp: afterwards lane L holds columns CPL*L .. CPL*L+CPL-1
#pragma unroll
      for (int off = 16, cnt = MP / 2; off >= 1; off >>= 1, cnt >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int j = 0; j < cnt; ++j) {
          const float send = upper ? v[j] : v[j + cnt];
          const float keep = upper ? v[j + cnt] : v[j];
          v[j] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, off));
        }
      }
#pragma unroll
      for (int j = 0; j < CPL; ++j) s_wmax[warp * MP + CPL * lane + j] = v[j];
      if (r == 0) s_flag[(i + 1) % 3] = 0;   // last read two tiles ago
      named_barrier(1, kTile);
      if (r < MP) {
        const float tmax = fmaxf(fmaxf(s_wmax[r], s_wmax[MP + r]), fmaxf(s_wmax[2 * MP + r], s_wmax[3 * MP + r]));
        const float old = s_ref[r];
        s_new[r] = fmaxf(old, tmax);
        if (r < m && tmax > old + 8.f) s_flag[i % 3] = 1;
      }
      named_barrier(1, kTile);
      const bool move = s_flag[i % 3] != 0;     // CTA-uniform
      if (i > 0) {
        // previous tile's accumulation still reads the P' tile and writes the accumulators
        if (!mbar_wait(acc_done, (i - 1) & 1, ab, 0x3700 + i)) { alive = false; break; }
        __syncwarp();
        tc_fence_after();
      }
      if (move) {
        if (r < MP) {
          const float old = s_ref[r], nw = s_new[r];
          s_fac[r] = (old == -INFINITY) ? 0.f : fast_exp2(old - nw);
          s_ref[r] = nw;
        }
        named_barrier(1, kTile);
        if (i > 0) {
          const float f = s_fac[owner ? lrow : 0];
#pragma unroll
          for (int c0 = 0; c0 < D + 32; c0 += 32) {
            float o[32];
            tmem_ld32(tmem_acc + lane_base + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= f;
            tmem_st32(tmem_acc + lane_base + c0, o);
          }
          tmem_st_wait();
        }
      }
#pragma unroll
      for (int j = 0; j < MP; j += 4) {
        const float4 c = *reinterpret_cast<const float4*>(s_ref + j);
        s[j + 0] = fast_exp2(s[j + 0] - c.x);
        s[j + 1] = fast_exp2(s[j + 1] - c.y);
        s[j + 2] = fast_exp2(s[j + 2] - c.z);
        s[j + 3] = fast_exp2(s[j + 3] - c.w);
      }
#pragma unroll
      for (int c = 0; c < MP / 8; ++c) {
        uint4 w4;
        w4.x = pack2<T>(s[8 * c + 0], s[8 * c + 1]);
        w4.y = pack2<T>(s[8 * c + 2], s[8 * c + 3]);
        w4.z = pack2<T>(s[8 * c + 4], s[8 * c + 5]);
        w4.w = pack2<T>(s[8 * c + 6], s[8 * c + 7]);
        *reinterpret_cast<uint4*>(s_p + (c >> 3) * (kTile * 128) + sw128_offset(r, c & 7)) = w4;
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (alive && mbar_wait(acc_done, (count - 1) & 1, ab, 0x3900)) {
      __syncwarp();
      tc_fence_after();
      const size_t slot = (size_t)bh * sch.nchunk + chunk;
      float* dst = part_acc + slot * m * D;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        float o[32];
        tmem_ld32(tmem_acc + lane_base + c0, o);
        tmem_ld_wait();
        if (owner && lrow < m) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + lrow * D + c0 + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
        }
      }
      float o[32];
      tmem_ld32(tmem_sum + lane_base, o);
      tmem_ld_wait();
      if (owner && lrow < m) {
        part_sum[slot * m + lrow] = o[0];
        part_max[slot * m + lrow] = s_ref[lrow] * kLn2;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace tc
}  // namespace fnb
