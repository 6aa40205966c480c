// sm_100a tensor-core streaming kernels (fp16 / bf16 I/O, FP32 accumulation in TMEM).
//
// Common structure: a CTA of 10 warps owns a run of consecutive 128-row tiles of one (b,h)
// slice.  Warp 8 is the TMA producer, warp 9 issues tcgen05.mma (one thread), warps 0-7 are
// the compute warps.  Compute thread t owns tile row r = t & 127 (= TMEM lane r) and column half
// h = t >> 7 of every per-row vector, so per-thread state is half a row and a row-wise reduction
// costs one exchange through shared memory between the two threads of a row.  Tiles of Q/K/V/dO
// are staged by TMA with the 128-byte swizzle; probabilities and softmax gradients go back to
// shared memory in the same swizzled [128 x 64] blocks and serve directly as UMMA operands
// (K-major when contracted over landmarks, MN-major when contracted over the tile's rows).  The
// landmark-sized operands (m x D, padded to MP = 64 or 128 landmarks) are packed once per call
// into 16-bit copies and stay resident in shared memory for the whole CTA.
#pragma once
#include <type_traits>
#include "common.cuh"
#include "small_kernels.cuh"
#include "tc_common.cuh"

namespace fnb {
namespace tc {

constexpr int kTile = 128;
constexpr int kComputeThreads = 256;
constexpr int kProducerWarp = 8, kMmaWarp = 9;
constexpr int kTcThreads = 320;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Optional per-tile timestamps of one CTA and per-CTA lifetimes (profiling builds only:
// -DFNB_TC_TRACE).  g_tc_trace_cta selects (kernel id << 16) | CTA; kernel ids: 0 forward column
// pass, 1 first backward row pass, 2 backward column pass, 3 in-place pass, 4 output pass.
#ifdef FNB_TC_TRACE
__device__ long long g_tc_trace[8][256];
__device__ int g_tc_trace_cta = 150;
__device__ unsigned long long g_tc_span[6 * 1024];   // per CTA: SM id, times (ns) of entry, exit, dependency wait over,
                                                     // first tile done, last tile done
__device__ __forceinline__ void tc_span(int which, int kid) {
  if (threadIdx.x == 0 && blockIdx.x < 1024 && (g_tc_trace_cta >> 16) == kid) {
    if (which == 0) {
      unsigned smid;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
      g_tc_span[6 * blockIdx.x] = smid;
    }
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_tc_span[6 * blockIdx.x + 1 + which] = t;
  }
}
#define TC_SPAN(which) tc_span(which, kTraceId)
#define TC_TRACE(role, idx)                                                                    \
  do {                                                                                         \
    if ((int)blockIdx.x + (kTraceId << 16) == g_tc_trace_cta && (idx) < 256) g_tc_trace[role][idx] = clock64(); \
  } while (0)
#else
#define TC_TRACE(role, idx) do {} while (0)
#define TC_SPAN(which) do {} while (0)
#endif

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~(uintptr_t)1023);
}

struct TcSched {
  int64_t N;             // rows of this rank's slice
  int nchunk;            // CTAs per (b,h) slice
  int tiles_per_chunk;   // 128-row tiles per CTA
  int64_t seg_N;         // sequence length the landmark segments are defined on (== N unless the
  int64_t row_offset;    //   sequence is sharded over ranks: then the global length and this
                         //   rank's first global row)
  // Order in which a CTA walks its tiles.  kOrderStrided: CTA c of a slice takes tiles c,
  // c + nchunk, c + 2 nchunk, ... (all CTAs of a slice sweep one moving window of the tensor, so
  // what the pass leaves in L2 is the end of every slice whatever nchunk is) instead of a
  // contiguous run.  kOrderDescending: last tile first (a pass that starts where its predecessor
  // in the stream ended finds that data still in L2).
  int order;
  int hint;              // L2 eviction hints, two bits per operand slot (tc_common.cuh: l2_policy_of)
  int H;                 // extent of the tensor maps' third dimension (heads; batch * heads for the plain layout):
                         //   slice bh sits at coordinates (bh % H, bh / H)
  int test_drop;         // test only: the output pass's first CTA never issues the load of its last tile,
                         //   so that a bounded wait runs out (FNB_FLAG_TEST_DROP_LOAD)
};
constexpr int kOrderStrided = 1, kOrderDescending = 2;

// NC consecutive FP32 TMEM columns of this thread's lane -> registers
template <int NC>
__device__ __forceinline__ void ld_cols(uint32_t taddr, float* v) {
#pragma unroll
  for (int c0 = 0; c0 < NC; c0 += 32) tmem_ld32(taddr + c0, v + c0);
}
// NC values (columns col0 .. col0+NC-1 of row r) -> 16-bit, into a swizzled tile made of
// [128 x 64] blocks
template <class T, int NC>
__device__ __forceinline__ void store_cols(uint8_t* tile, int r, int col0, const float* v) {
#pragma unroll
  for (int c = 0; c < NC / 8; ++c) {
    uint4 w;
    w.x = pack2<T>(v[8 * c + 0], v[8 * c + 1]);
    w.y = pack2<T>(v[8 * c + 2], v[8 * c + 3]);
    w.z = pack2<T>(v[8 * c + 4], v[8 * c + 5]);
    w.w = pack2<T>(v[8 * c + 6], v[8 * c + 7]);
    const int cc = (col0 >> 3) + c;
    *reinterpret_cast<uint4*>(tile + (cc >> 3) * (kTile * 128) + sw128_offset(r, cc & 7)) = w;
  }
}
// K-major operand: advance by k 16-element steps along K inside [rows x 64] blocks
__device__ __forceinline__ uint64_t kdesc(uint32_t base, int k, int rows) {
  return smem_desc_sw128(base + (k >> 2) * (rows * 128) + (k & 3) * 32, 16, 1024);
}
// MN-major operand staged as [128 rows(K) x 64] blocks: advance by k 16-row steps along K
__device__ __forceinline__ uint64_t mndesc(uint32_t base, int k) {
  return smem_desc_sw128(base + k * 2048, kTile * 128, 1024);
}

// Compute warps (256 threads): 16-bit swizzled operand tiles of two (m x D) landmark matrices of one
// slice straight from their FP32 originals (MP rows, rows >= m zero; D / 64 blocks of
// [MP rows x 128 B] each):
//   tile_a = mul_a * A,   tile_b = B / sc  with sc the power of two >= max |B|   (returned).
// 256 / MP threads share a row; each packs D MP / 256 consecutive columns, eight at a time.  scratch: 8 floats of shared memory; named barrier 3 is used once.
// The caller fences and signals the MMA thread.
template <class T, int D, int MP>
__device__ __forceinline__ float pack_landmark_operands(uint8_t* tile_a, uint8_t* tile_b, const float* A,
                                                        const float* B, int m, float mul_a, float* scratch) {
  constexpr int TPR = kComputeThreads / MP, CPT = D / TPR;
  const int t = threadIdx.x, r = t / TPR, c0 = (t % TPR) * CPT;
  // up to 32 columns per thread: both row segments stay in registers between the maximum and the
  // packing (one trip to the L2 instead of two); wider segments are read again
  constexpr bool kKeep = CPT <= 32;
  float4 xa[kKeep ? CPT / 4 : 1], yb[kKeep ? CPT / 4 : 1];
  float amax = 0.f;
  if (kKeep) {
#pragma unroll
    for (int q = 0; q < CPT / 4; ++q) {
      xa[q] = yb[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < m) {
        xa[q] = *reinterpret_cast<const float4*>(A + r * D + c0 + 4 * q);
        yb[q] = *reinterpret_cast<const float4*>(B + r * D + c0 + 4 * q);
      }
    }
#pragma unroll
    for (int q = 0; q < CPT / 4; ++q)
      amax = fmaxf(fmaxf(amax, fmaxf(fabsf(yb[q].x), fabsf(yb[q].y))), fmaxf(fabsf(yb[q].z), fabsf(yb[q].w)));
  } else if (r < m) {
#pragma unroll
    for (int q = 0; q < CPT / 4; ++q) {
      const float4 y = *reinterpret_cast<const float4*>(B + r * D + c0 + 4 * q);
      amax = fmaxf(fmaxf(amax, fmaxf(fabsf(y.x), fabsf(y.y))), fmaxf(fabsf(y.z), fabsf(y.w)));
    }
  }
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((t & 31) == 0) scratch[t >> 5] = amax;
  named_barrier(3, kComputeThreads);
  float cmax = scratch[0];
#pragma unroll
  for (int w = 1; w < kComputeThreads / 32; ++w) cmax = fmaxf(cmax, scratch[w]);
  const float sc = pow2_scale(cmax), inv = 1.f / sc;
#pragma unroll
  for (int c = 0; c < CPT / 8; ++c) {
    float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0, y0 = x0, y1 = x0;
    if (kKeep) {
      x0 = xa[kKeep ? 2 * c : 0]; x1 = xa[kKeep ? 2 * c + 1 : 0]; y0 = yb[kKeep ? 2 * c : 0]; y1 = yb[kKeep ? 2 * c + 1 : 0];
    } else if (r < m) {
      x0 = *reinterpret_cast<const float4*>(A + r * D + c0 + 8 * c);
      x1 = *reinterpret_cast<const float4*>(A + r * D + c0 + 8 * c + 4);
      y0 = *reinterpret_cast<const float4*>(B + r * D + c0 + 8 * c);
      y1 = *reinterpret_cast<const float4*>(B + r * D + c0 + 8 * c + 4);
    }
    uint4 wa, wb;
    wa.x = pack2<T>(x0.x * mul_a, x0.y * mul_a); wa.y = pack2<T>(x0.z * mul_a, x0.w * mul_a);
    wa.z = pack2<T>(x1.x * mul_a, x1.y * mul_a); wa.w = pack2<T>(x1.z * mul_a, x1.w * mul_a);
    wb.x = pack2<T>(y0.x * inv, y0.y * inv); wb.y = pack2<T>(y0.z * inv, y0.w * inv);
    wb.z = pack2<T>(y1.x * inv, y1.y * inv); wb.w = pack2<T>(y1.z * inv, y1.w * inv);
    const int cc = (c0 >> 3) + c;
    const uint32_t off = (uint32_t)(cc >> 3) * (MP * 128) + sw128_offset(r, cc & 7);
    *reinterpret_cast<uint4*>(tile_a + off) = wa;
    *reinterpret_cast<uint4*>(tile_b + off) = wb;
  }
  return sc;
}

struct TileRange {
  int64_t bh;
  int ch, cb;            // tensor-map coordinates of the slice: (bh % H, bh / H)
  int chunk, first, step, count;
  bool desc;
  // i-th tile this CTA works on
  __device__ __forceinline__ int tile(int i) const { return first + (desc ? count - 1 - i : i) * step; }
  __device__ __forceinline__ int lowest() const { return first; }
  __device__ __forceinline__ int highest() const { return first + (count - 1) * step; }
};
__device__ __forceinline__ TileRange tile_range(const TcSched& sch, int order) {
  TileRange t;
  const int bhi = (int)blockIdx.x / sch.nchunk;
  t.bh = bhi;
  t.ch = bhi % sch.H;
  t.cb = bhi / sch.H;
  t.chunk = (int)blockIdx.x - bhi * sch.nchunk;
  const int total_tiles = (int)((sch.N + kTile - 1) / kTile);
  if (order & kOrderStrided) {
    t.first = t.chunk;
    t.step = sch.nchunk;
    t.count = t.chunk < total_tiles ? (total_tiles - t.chunk + sch.nchunk - 1) / sch.nchunk : 0;
  } else {
    t.first = t.chunk * sch.tiles_per_chunk;
    t.step = 1;
    t.count = max(0, min(sch.tiles_per_chunk, total_tiles - t.first));
  }
  t.desc = (order & kOrderDescending) != 0;
  return t;
}
__device__ __forceinline__ TileRange tile_range(const TcSched& sch) { return tile_range(sch, sch.order); }

// ------------------------------------------------------------------------------------------
// Forward output pass:  O = softmax(Q Kt^T) step2, lse1.
//   kt16 = s*log2e*Kt (MP x D), st16 = step2^T / 2^e (D x MP), st_scale[bh] = 2^e.
// The eight compute warps form two groups of 128 threads (one thread per tile row, all landmark
// columns).  Group g owns tiles g, g+2, ... with its own S and O accumulators in TMEM and its own
// P buffer in shared memory, so two tiles are always in different phases (softmax of one while
// the products of the other run); the output tile is staged in the group's P buffer once the
// product that read it has completed.  The MMA thread issues the score product two tiles ahead.
template <int D, int MP>
struct FwdCSmem {
  static constexpr int kKt = MP * D * 2, kSt = D * MP * 2, kQ = kTile * D * 2, kP = kTile * MP * 2,
                       kO = kTile * D * 2;
  static constexpr int kPO = kP > kO ? kP : kO;   // the output tile is staged in the probability buffer
  static constexpr int kBytes = kKt + kSt + 2 * kQ + 2 * kPO + 256 + 1024;
};

template <class T, int D, int MP>
__global__ void __launch_bounds__(kTcThreads, (D == 64 ? 2 : 1))
tc_fwd_c_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_o,
                const float* __restrict__ k_landmarks, const float* __restrict__ step2,
                float* __restrict__ lse1, TcSched sch, int m, float scale, int* status) {
  using L = FwdCSmem<D, MP>;
  constexpr int kTraceId = 4; (void)kTraceId;
  TC_SPAN(0);
  static_assert((D == 64 && MP == 64) || (D == 128 && (MP == 64 || MP == 128)), "head_dim 64 with up to 64 landmarks, 128 with up to 128");
  constexpr int KBD = D / 64;
  constexpr int kGroup = kComputeThreads / 2;
  constexpr uint32_t kCols = 2 * MP + 2 * D;
  constexpr uint32_t kTmemCols = kCols <= 256 ? 256 : 512;
  extern __shared__ uint8_t smem_raw[];
  pdl_trigger();
  uint8_t* base = align1024(smem_raw);
  uint8_t* s_kt = base;
  uint8_t* s_st = s_kt + L::kKt;
  uint8_t* s_q = s_st + L::kSt;          // two stages
  uint8_t* s_p = s_q + 2 * L::kQ;        // one buffer per compute group
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_p + 2 * L::kPO);
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
  const TileRange tr = tile_range(sch);
  const int tr_ch = tr.ch, tr_cb = tr.cb;
  const int64_t bh = tr.bh;
  const int count = tr.count;

  if (threadIdx.x == 0) {
    mbar_init(small_full, kComputeThreads / 32);
    for (int s = 0; s < 2; ++s) {
      mbar_init(q_full + s, 1); mbar_init(q_empty + s, 1); mbar_init(s_full + s, 1);
      mbar_init(p_full + s, kGroup / 32); mbar_init(o_full + s, 1); mbar_init(o_free + s, kGroup / 32);
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
  pdl_wait();   // everything above overlaps the tail of the previous kernel of the stream
  TC_SPAN(2);
  const uint32_t tmem_base = *tmem_slot;
  Abort ab{abort_word, status};

  if (warp == kProducerWarp) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_o);
      const uint64_t pol_q = l2_policy_of(sch.hint, 0);
      int armed = 0;
      for (int i = 0; i < count; ++i) {
        const int st = i & 1;
        if (!mbar_wait(q_empty + st, ((i >> 1) & 1) ^ 1, ab, 0x100 + i)) break;
        if (sch.test_drop && blockIdx.x == 0 && i == count - 1) break;   // fault injection on the host's request
        mbar_expect_tx(q_full + st, L::kQ);
        for (int kb = 0; kb < KBD; ++kb)
          tma_load_4d_h(s_q + st * L::kQ + kb * (kTile * 128), &tm_q, q_full + st, kb * 64, tr.tile(i) * kTile, tr_ch, tr_cb, pol_q);
        armed = i + 1;
      }
      if (ab.raised())   // let copies already in flight land before the shared memory is released
        for (int i = max(0, armed - 2); i < armed; ++i) mbar_drain(q_full + (i & 1), (i >> 1) & 1);
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc1 = make_idesc<T>(kTile, MP, false, false);
      constexpr uint32_t idesc2 = make_idesc<T>(kTile, D, false, true);   // step2 (m x D) is read MN-major
      const uint32_t a_kt = smem_u32(s_kt), a_st = smem_u32(s_st);
      // Score product of tile i into S[i & 1].  That buffer was released when this thread passed
      // p_full of tile i-2, which precedes this call in program order.
      auto front = [&](int i) -> bool {
        const int st = i & 1;
        if (!mbar_wait(q_full + st, (i >> 1) & 1, ab, 0x300 + i)) return false;
        tc_fence_after();
        const uint32_t a_q = smem_u32(s_q + st * L::kQ);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma(tmem_base + st * MP, kdesc(a_q, k, kTile), kdesc(a_kt, k, MP), idesc1, k > 0);
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
        const uint32_t a_p = smem_u32(s_p + st * L::kPO);
#pragma unroll
        for (int k = 0; k < MP / 16; ++k)
          umma(tmem_base + 2 * MP + st * D, kdesc(a_p, k, kTile), smem_desc_sw128(a_st + k * 2048, MP * 128, 1024),
               idesc2, k > 0);
        umma_commit(o_full + st);
        if (i + 2 < count) ok = front(i + 2);
      }
    }
  } else {
    const int g = warp >> 2;                                  // compute group
    const int r = threadIdx.x & 127;                           // tile row = TMEM lane
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    // operand copies of Kt and step2 for this slice (the P buffers are free until the first tile)
    const float osc = pack_landmark_operands<T, D, MP>(s_kt, s_st, k_landmarks + bh * m * D, step2 + bh * m * D, m,
                                                   scale * kLog2e, reinterpret_cast<float*>(s_p));
    fence_proxy_async();
    mbar_arrive_warp(small_full);
    uint8_t* my_p = s_p + g * L::kPO;
    const bool leader = r == 0;
    const uint64_t pol_o = leader ? l2_policy_of(sch.hint, 2) : 0ull;
    const bool full_m = m == MP;
    for (int i = g; i < count; i += 2) {
      if (i == 2) TC_SPAN(3);
      const uint32_t par = (uint32_t)(i >> 1) & 1u;
      if (!mbar_wait(s_full + g, par, ab, 0x600 + i)) break;
      __syncwarp();
      tc_fence_after();
      float s[MP];
      ld_cols<MP>(tmem_base + g * MP + lane_base, s);
      tmem_ld_wait();
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      float sm4[4] = {0.f, 0.f, 0.f, 0.f};
      float mx;
      if (full_m) {
#pragma unroll
        for (int j = 0; j < MP; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], s[j]);
        mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
#pragma unroll
        for (int j = 0; j < MP; ++j) {
          s[j] = fast_exp2(s[j] - mx);
          sm4[j & 3] += s[j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < MP; ++j) if (j < m) mx4[j & 3] = fmaxf(mx4[j & 3], s[j]);
        mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
#pragma unroll
        for (int j = 0; j < MP; ++j) {
          s[j] = (j < m) ? fast_exp2(s[j] - mx) : 0.f;
          sm4[j & 3] += s[j];
        }
      }
      const float tot = (sm4[0] + sm4[1]) + (sm4[2] + sm4[3]);
      // this group's previous output tile was stored from my_p: wait until the copy has read it
      if (leader) tma_store_wait_read();
      named_barrier(1 + g, kGroup);
      store_cols<T, MP>(my_p, r, 0, s);
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive_warp(p_full + g);
      const float mul = osc / tot;
      const int64_t row = (int64_t)tr.tile(i) * kTile + r;
      if (row < sch.N) lse1[bh * sch.N + row] = (mx + log2f(tot)) * kLn2;
      // output product of the same tile
      if (!mbar_wait(o_full + g, par, ab, 0x700 + i)) break;
      __syncwarp();
      tc_fence_after();
      // (the product that read P from my_p has completed, so the output tile can be staged there)
#pragma unroll
      for (int oc = 0; oc < D / 64; ++oc) {
        float o[64];
        ld_cols<64>(tmem_base + 2 * MP + g * D + oc * 64 + lane_base, o);
        tmem_ld_wait();
        if (oc == D / 64 - 1) {
          tc_fence_before();
          mbar_arrive_warp(o_free + g);
        }
#pragma unroll
        for (int j = 0; j < 64; ++j) o[j] *= mul;
        store_cols<T, 64>(my_p, r, oc * 64, o);
      }
      fence_proxy_async();
      named_barrier(1 + g, kGroup);
      if (leader) {
        for (int kb = 0; kb < KBD; ++kb)
          tma_store_4d_h(&tm_o, my_p + kb * (kTile * 128), kb * 64, tr.tile(i) * kTile, tr_ch, tr_cb, pol_o);
        tma_store_commit();
      }
    }
    TC_SPAN(4);
    if (leader) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
  TC_SPAN(1);
}

// ------------------------------------------------------------------------------------------
// Softmax-1 backward, first row pass.  Per 128-row tile of Q and dO (thread = row n, half the
// landmark columns):
//   S1 = Q kt16^T (log2 domain), dP1 = dO st16^T (step2 normalised by 2^-e, undone by sc),
//   P1 = exp2(S1 - lse1*log2e), D1 = rowsum(P1 o dP1), dS1 = P1 o (dP1 - D1)        [FP32]
//   dstep2 += P1^T dO and dKt += dS1^T Q accumulate in TMEM over all of the CTA's tiles (UMMA with
//   both operands MN-major: the staged tiles are contracted over their rows); one FP32 partial
//   pair per CTA.  The 16-bit dS1 tile also goes to global memory as it is, into the dQ tile of
//   the same rows (same footprint), where the in-place pass finishes dQ.
template <int D, int MP>
struct BwdASmem {
  static constexpr int kKt = MP * D * 2, kSt = MP * D * 2, kIn = kTile * D * 2, kP = kTile * MP * 2,
                       kDs = kTile * MP * 2;
  // (Q, dO) stages: two, or one where 128 landmarks leave no room for the second
  static constexpr int kStages = MP == 128 ? 1 : 2;
  // relies on the dynamic shared window being 1024-byte aligned (checked at run time)
  static constexpr int kBytes = kKt + kSt + 2 * kStages * kIn + kP + kDs + 256;
};

template <class T, int D, int MP>
__global__ void __launch_bounds__(kTcThreads, (D == 64 ? 2 : 1))
tc_bwd_a_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_g,
                const __grid_constant__ CUtensorMap tm_dq,
                const float* __restrict__ k_landmarks, const float* __restrict__ step2,
                const float* __restrict__ lse1, float* __restrict__ partA, float* __restrict__ sc_out,
                TcSched sch, int m, float scale, int* status) {
  static_assert((D == 64 && MP == 64) || (D == 128 && (MP == 64 || MP == 128)), "head_dim 64 with up to 64 landmarks, 128 with up to 128");
  using L = BwdASmem<D, MP>;
  constexpr int kTraceId = 1; (void)kTraceId;
  TC_SPAN(0);
  constexpr int HC = MP / 2, HD = D / 2, NST = L::kStages;
  constexpr uint32_t kTmemCols = 2 * MP + 2 * D <= 256 ? 256 : 512;    // S, dP, and 2 D accumulator columns
  extern __shared__ uint8_t smem_raw[];
  pdl_trigger();
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, (2 << 24) | 0x1000);
    return;
  }
  uint8_t* s_kt = smem_raw;
  uint8_t* s_st = s_kt + L::kKt;
  uint8_t* s_q = s_st + L::kSt;          // NST stages of [Q tile | dO tile]
  uint8_t* s_g = s_q + L::kIn;
  uint8_t* s_p = s_q + 2 * NST * L::kIn; // P tile (its head doubles as the D1 exchange)
  uint8_t* s_ds = s_p + L::kP;           // dS tile
  float* s_x = reinterpret_cast<float*>(s_p);
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_ds + L::kDs);
  uint64_t* small_full = bars + 0;
  uint64_t* in_full = bars + 1;          // [2]
  uint64_t* in_empty = bars + 3;         // [2]
  uint64_t* sdp_full = bars + 5;
  uint64_t* pds_full = bars + 6;
  uint64_t* acc_done = bars + 7;         // accumulation of a tile complete, its dS copy read
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  int* abort_word = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileRange tr = tile_range(sch);
  const int tr_ch = tr.ch, tr_cb = tr.cb;
  const int64_t bh = tr.bh;
  const int count = tr.count;

  if (threadIdx.x == 0) {
    mbar_init(small_full, kComputeThreads / 32);
    for (int s = 0; s < 2; ++s) { mbar_init(in_full + s, 1); mbar_init(in_empty + s, 1); }
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, kComputeThreads / 32);
    mbar_init(acc_done, 1);
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
  pdl_wait();   // everything above overlaps the tail of the previous kernel of the stream
  TC_SPAN(2);
  const uint32_t tmem_base = *tmem_slot;
  Abort ab{abort_word, status};

  if (warp == kProducerWarp) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_g);
      const uint64_t pol_q = l2_policy_of(sch.hint, 0), pol_g = l2_policy_of(sch.hint, 1);
      int armed = 0;
      for (int i = 0; i < count; ++i) {
        const int st = i % NST;
        if (!mbar_wait(in_empty + st, ((i / NST) & 1) ^ 1, ab, 0x1100 + i)) break;
        mbar_expect_tx(in_full + st, 2 * L::kIn);
        for (int kb = 0; kb < D / 64; ++kb) {
          tma_load_4d_h(s_q + st * 2 * L::kIn + kb * (kTile * 128), &tm_q, in_full + st, kb * 64, tr.tile(i) * kTile, tr_ch, tr_cb, pol_q);
          tma_load_4d_h(s_g + st * 2 * L::kIn + kb * (kTile * 128), &tm_g, in_full + st, kb * 64, tr.tile(i) * kTile, tr_ch, tr_cb, pol_g);
        }
        TC_TRACE(0, i);
        armed = i + 1;
      }
      if (ab.raised())
        for (int i = max(0, armed - NST); i < armed; ++i) mbar_drain(in_full + (i % NST), (i / NST) & 1);
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc<T>(kTile, MP, false, false);
      constexpr uint32_t idesc_acc2 = make_idesc<T>(MP == 64 ? 128 : 128, MP == 64 ? 2 * D : D, true, true);
      const uint32_t a_kt = smem_u32(s_kt), a_st = smem_u32(s_st), a_p = smem_u32(s_p);
      const uint64_t pol_ds = l2_policy_of(sch.hint, 2);
      // S and dP of tile i
      auto front = [&](int i) -> bool {
        const int st = i % NST;
        if (!mbar_wait(in_full + st, (i / NST) & 1, ab, 0x1300 + i)) return false;
        TC_TRACE(1, i);
        tc_fence_after();
        const uint32_t a_q = smem_u32(s_q + st * 2 * L::kIn), a_g = smem_u32(s_g + st * 2 * L::kIn);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma(tmem_base, kdesc(a_q, k, kTile), kdesc(a_kt, k, MP), idesc_s, k > 0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma(tmem_base + MP, kdesc(a_g, k, kTile), kdesc(a_st, k, MP), idesc_s, k > 0);
        umma_commit(sdp_full);
        return true;
      };
      bool ok = mbar_wait(small_full, 0, ab, 0x1200);
      ok = ok && front(0);
      for (int i = 0; ok && i < count; ++i) {
        if (!mbar_wait(pds_full, i & 1, ab, 0x1400 + i)) break;
        TC_TRACE(2, i);
        tc_fence_after();
        const int st = i % NST;
        // One 128 x 2D accumulator for both sums: [P | dS]^T [Q | dO] (both operands MN-major; the
        // 64-wide blocks of each follow one another in shared memory, 16 KB apart).  Rows 0..63 x
        // columns D..2D-1 hold P^T dO, rows 64..127 x columns 0..D-1 hold dS^T Q; the other two
        // quadrants are not used.  An M = N = 128 MMA takes 35 ns against 2 x 25 ns for two 64 x 64 ones.
        if (MP == 64) {
#pragma unroll
          for (int k = 0; k < kTile / 16; ++k)
            umma(tmem_base + 2 * MP, smem_desc_sw128(a_p + k * 2048, L::kP, 1024),
                 smem_desc_sw128(smem_u32(s_q + st * 2 * L::kIn) + k * 2048, kTile * 128, 1024), idesc_acc2, (i > 0 || k > 0));
        } else {
          // 128 landmarks: M = 128 each, so the two sums take an accumulator of their own
          // (P^T dO in columns 2 MP .. + D - 1, dS^T Q in the D columns after them)
          const uint32_t a_ds = smem_u32(s_ds);
#pragma unroll
          for (int k = 0; k < kTile / 16; ++k)
            umma(tmem_base + 2 * MP, mndesc(a_p, k), mndesc(smem_u32(s_g + st * 2 * L::kIn), k), idesc_acc2, (i > 0 || k > 0));
#pragma unroll
          for (int k = 0; k < kTile / 16; ++k)
            umma(tmem_base + 2 * MP + D, mndesc(a_ds, k), mndesc(smem_u32(s_q + st * 2 * L::kIn), k), idesc_acc2, (i > 0 || k > 0));
        }
        // the accumulation goes first: its commit frees the (Q, dO) stage, and the pass is bound by
        // how early the next load is issued; then the scores of the next tile
        umma_commit(in_empty + st);
        // the dS tile as it is -> (the first MP columns of) the dQ tile of the same rows
        for (int kb = 0; kb < MP / 64; ++kb)
          tma_store_4d_h(&tm_dq, s_ds + kb * (kTile * 128), kb * 64, tr.tile(i) * kTile, tr_ch, tr_cb, pol_ds);
        tma_store_commit();
        TC_TRACE(3, i);
        if (i + 1 < count && !front(i + 1)) break;
        // acc_done lets the compute warps overwrite the dS tile: the copy must have read it
        tma_store_wait_read();
        umma_commit(acc_done);
      }
      tma_store_wait_all();
    }
  } else {
    const int r = threadIdx.x & 127, h = threadIdx.x >> 7;
    const int quarter = warp & 3;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    // operand copies of Kt and step2 for this slice (the dS tile is free until the first tile)
    const float sc = pack_landmark_operands<T, D, MP>(s_kt, s_st, k_landmarks + bh * m * D, step2 + bh * m * D, m,
                                                  scale * kLog2e, reinterpret_cast<float*>(s_ds));
    fence_proxy_async();
    mbar_arrive_warp(small_full);
    // the in-place dQ pass rescales the dS tiles by the same power of two
    if (sc_out && threadIdx.x == 0) sc_out[bh] = sc;
    const int c0 = h * HC;
    bool alive = true;
    for (int i = 0; i < count; ++i) {
      if (i == 1) TC_SPAN(3);
      const int64_t row = (int64_t)tr.tile(i) * kTile + r;
      const bool valid = row < sch.N;
      const float lse = valid ? lse1[bh * sch.N + row] * kLog2e : 0.f;
      if (!mbar_wait(sdp_full, i & 1, ab, 0x1600 + i)) { alive = false; break; }
      if (threadIdx.x == 0) TC_TRACE(4, i);
      __syncwarp();
      tc_fence_after();
      float p[HC], g[HC];
      const uint32_t t_s = tmem_base + lane_base;
      ld_cols<HC>(t_s + c0, p);
      ld_cols<HC>(t_s + MP + c0, g);
      tmem_ld_wait();
      float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < HC; ++j) {
        p[j] = (valid && c0 + j < m) ? fast_exp2(p[j] - lse) : 0.f;
        d4[j & 3] = fmaf(p[j], g[j], d4[j & 3]);
      }
      const float dpart = (d4[0] + d4[1]) + (d4[2] + d4[3]);
      if (threadIdx.x == 0) TC_TRACE(5, i);
      // the previous tile's P / dS are still being read by its accumulation MMAs and its dS copy
      if (i > 0 && !mbar_wait(acc_done, (i - 1) & 1, ab, 0x1700 + i)) { alive = false; break; }
      if (threadIdx.x == 0) TC_TRACE(6, i);
      __syncwarp();
      s_x[h * kTile + r] = dpart;
      named_barrier(1, kComputeThreads);
      const float d1 = dpart + s_x[(h ^ 1) * kTile + r];
      named_barrier(1, kComputeThreads);   // exchange words live in the head of the P tile
      store_cols<T, HC>(s_p, r, c0, p);
#pragma unroll
      for (int j = 0; j < HC; ++j) g[j] = p[j] * (g[j] - d1);
      // (dS1 / sc leaves the fp16 range only for |dO| of several hundred and more; it then becomes
      // inf and dQ comes back inf / NaN, which is what a loss scaler looks for)
      store_cols<T, HC>(s_ds, r, c0, g);
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive_warp(pds_full);
      if (threadIdx.x == 0) TC_TRACE(7, i);
    }
    TC_SPAN(4);
    if (alive && mbar_wait(acc_done, (count - 1) & 1, ab, 0x1900)) {
      __syncwarp();
      tc_fence_after();
      if (MP == 64) {
        // 128-row accumulator: TMEM lane = row.  Quarters 0, 1 hold the dstep2 rows (columns
        // D..2D-1), quarters 2, 3 the dKt rows (columns 0..D-1); this thread takes half the columns.
        const int which = quarter >> 1;
        const int l = (quarter & 1) * 32 + lane;
        float* dst = partA + ((size_t)bh * sch.nchunk + tr.chunk) * 2 * m * D + (size_t)which * m * D;
        const float mul = which ? sc * scale : 1.f;
        float o[HD];
        ld_cols<HD>(tmem_base + 2 * MP + (which ? 0 : D) + lane_base + h * HD, o);
        tmem_ld_wait();
        if (l < m) {
#pragma unroll
          for (int j = 0; j < HD; j += 4)
            *reinterpret_cast<float4*>(dst + l * D + h * HD + j) =
                make_float4(o[j] * mul, o[j + 1] * mul, o[j + 2] * mul, o[j + 3] * mul);
        }
      } else {
        // two 128-row accumulators (lane = landmark): dstep2 first, then dKt
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          float* dst = partA + ((size_t)bh * sch.nchunk + tr.chunk) * 2 * m * D + (size_t)which * m * D;
          const float mul = which ? sc * scale : 1.f;
          float o[HD];
          ld_cols<HD>(tmem_base + 2 * MP + which * D + lane_base + h * HD, o);
          tmem_ld_wait();
          if (r < m) {
#pragma unroll
            for (int j = 0; j < HD; j += 4)
              *reinterpret_cast<float4*>(dst + r * D + h * HD + j) =
                  make_float4(o[j] * mul, o[j + 1] * mul, o[j + 2] * mul, o[j + 3] * mul);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
  TC_SPAN(1);
}

// ------------------------------------------------------------------------------------------
// Last backward pass: dQ and dK in place.  The first row pass leaves its 16-bit dS1 tiles
// (dS1 = P1 o (dP1 - D1), scaled by 1/sc with sc the power-of-two scale of step2) in the dQ buffer
// and the column pass its dS3' tiles in the dK buffer: with 64 landmark columns and head_dim 64
// such a tile has exactly the footprint of the gradient tile of the same rows.  Each tile becomes
//   side 0:  dQ = (sc ln2)  dS1  (s log2e Kt) + rows_q[l(n)]
//   side 1:  dK = (2^-k ln2) dS3' (s log2e Qt) + rows_k[l(n)]
// with one TMA load, one product and one TMA store; no exponentials, and Q, K, dO are not read
// again.  A CTA takes its run of tiles on side 0, then the same run on side 1.  Four input stages
// (released by the product's commit), four accumulators, compute groups of 128 threads (one thread
// per tile row; two groups, or four for head_dim 128 with up to 64 landmarks) that take the tiles in
// turn and stage their output tile in a buffer of their own.
struct RowsSide {
  const float* landmarks;   // [BH][m][D] FP32: the landmark matrix the tile is multiplied by
  float* rows;              // [BH][m][D] FP32: per-landmark term added to every row of its segment
  const float* out_scale;   // [BH] or null: per-slice factor of the product
  float out_mul;            // constant factor of the product
  // Optional: the CTA first forms the rows its own tiles need,
  //   rows[l] = rows_scale / len(l) * (base[l] + sum over chunks of part[chunk][l]),
  // (chunks in ascending order) and stores them into `rows`; CTAs that share a landmark store
  // identical values.  part == null: `rows` is complete on entry.
  const float* part;        // [BH][nchunk][m][D]
  const float* base;        // [BH][m][D]
  int nchunk;
  float rows_scale;
  int order;                // tile order of this side (kOrderStrided | kOrderDescending)
  const float* tile_scale;  // [BH][tiles] or null: extra factor of the product, per tile
};

template <int D, int MP>
struct RowsSmem {
  static constexpr int kStages = MP == 128 ? 2 : 4;   // 128-landmark tiles are twice as large
  // Compute groups of 128 threads (one thread per tile row) that take tiles in turn.  head_dim 128 with
  // up to 64 landmarks runs one CTA per SM, whose epilogue per tile is twice that of head_dim 64: four
  // groups (one per stage) instead of two keep as many tiles in flight as two CTAs of head_dim 64 do.
  static constexpr int kGroups = (D == 128 && MP == 64) ? 4 : 2;
  static constexpr int kThreads = (kGroups * 4 + 2) * 32;   // compute warps, TMA producer, MMA issuer
  static constexpr int kOp = MP * D * 2, kIn = kTile * MP * 2, kOut = kTile * D * 2;
  // relies on the dynamic shared window being 1024-byte aligned (checked at run time)
  static constexpr int kBytes = 2 * kOp + kStages * kIn + kGroups * kOut + 256;
  static_assert(kStages % kGroups == 0, "a group always works on the same stages");
  static_assert(kBytes <= 227 * 1024, "shared memory");
};

// 16-bit swizzled operand tile of one FP32 (m x D) landmark matrix (MP rows, rows >= m zero; D / 64
// blocks of [MP rows x 128 B]), times mul; compute warps (256 threads): 256 / MP threads share a row
template <class T, int D, int MP>
__device__ __forceinline__ void pack_landmark_operand(uint8_t* tile, const float* A, int m, float mul) {
  constexpr int TPR = kComputeThreads / MP, CPT = D / TPR;
  const int t = threadIdx.x, r = t / TPR, c0 = (t % TPR) * CPT;
#pragma unroll
  for (int c = 0; c < CPT / 8; ++c) {
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f), y = x;
    if (r < m) {
      x = *reinterpret_cast<const float4*>(A + r * D + c0 + 8 * c);
      y = *reinterpret_cast<const float4*>(A + r * D + c0 + 8 * c + 4);
    }
    uint4 w;
    w.x = pack2<T>(x.x * mul, x.y * mul); w.y = pack2<T>(x.z * mul, x.w * mul);
    w.z = pack2<T>(y.x * mul, y.y * mul); w.w = pack2<T>(y.z * mul, y.w * mul);
    const int cc = (c0 >> 3) + c;
    *reinterpret_cast<uint4*>(tile + (uint32_t)(cc >> 3) * (MP * 128) + sw128_offset(r, cc & 7)) = w;
  }
}

template <class T, int D, int MP>
__global__ void __launch_bounds__((RowsSmem<D, MP>::kThreads), (D == 64 ? 2 : 1))
tc_rows_inplace_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                       RowsSide side_a, RowsSide side_b, int nsides, float op_mul, TcSched sch, int m,
                       int* status) {
  using L = RowsSmem<D, MP>;
  constexpr int kTraceId = 3; (void)kTraceId;
  TC_SPAN(0);
  // a parked dS tile (MP columns) sits in the first MP columns of the gradient tile of its rows
  static_assert((D == 64 && MP == 64) || (D == 128 && (MP == 64 || MP == 128)), "head_dim 64 with up to 64 landmarks, 128 with up to 128");
  constexpr int kGroup = 128, kGroups = L::kGroups, kCompute = kGroups * kGroup;
  constexpr int kProducer = kGroups * 4, kIssuer = kGroups * 4 + 1;   // warp numbers of the two single-thread roles
  constexpr int kStages = L::kStages;
  constexpr uint32_t kTmemCols = kStages * D;
  static_assert(kTmemCols == 256 || kTmemCols == 512, "TMEM allocation must be a power of two");
  extern __shared__ uint8_t smem_raw[];
  pdl_trigger();
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, (2 << 24) | 0x2000);
    return;
  }
  uint8_t* s_op = smem_raw;                    // one operand tile per side
  uint8_t* s_in = s_op + 2 * L::kOp;           // kStages dS tiles
  uint8_t* s_out = s_in + kStages * L::kIn;    // one staging tile per group
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_out + kGroups * L::kOut);
  uint64_t* small_full = bars + 0;
  uint64_t* in_full = bars + 1;                // [kStages]
  uint64_t* in_empty = bars + 1 + kStages;     // [kStages]
  uint64_t* acc_done = bars + 1 + 2 * kStages; // [kStages]
  uint64_t* o_free = bars + 1 + 3 * kStages;   // [kStages]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1 + 4 * kStages);
  int* abort_word = reinterpret_cast<int*>(tmem_slot + 1);
  static_assert((1 + 4 * kStages) * 8 + 8 <= 256, "barrier area");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileRange tra = tile_range(sch, side_a.order), trb = tile_range(sch, side_b.order);
  const int tr_ch = tra.ch, tr_cb = tra.cb;
  const int64_t bh = tra.bh;
  const int count = tra.count, total = count + (nsides > 1 ? trb.count : 0);

  if (threadIdx.x == 0) {
    mbar_init(small_full, kComputeThreads / 32);   // the first eight warps pack the operands
    for (int s = 0; s < kStages; ++s) {
      mbar_init(in_full + s, 1); mbar_init(in_empty + s, 1);
      mbar_init(acc_done + s, 1); mbar_init(o_free + s, kGroup / 32);
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
  pdl_wait();   // everything above overlaps the tail of the previous kernel of the stream
  TC_SPAN(2);
  const uint32_t tmem_base = *tmem_slot;
  Abort ab{abort_word, status};

  if (warp == kProducer) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_a);
      if (nsides > 1) tma_prefetch_desc(&tm_b);
      const uint64_t pol_a = l2_policy_of(sch.hint, 0), pol_b = l2_policy_of(sch.hint, 1);
      int armed = 0;
      for (int i = 0; i < total; ++i) {
        const int s = i % kStages;
        const bool second = i >= count;
        if (!mbar_wait(in_empty + s, ((i / kStages) & 1) ^ 1, ab, 0x2100 + i)) break;
        mbar_expect_tx(in_full + s, L::kIn);
        for (int kb = 0; kb < MP / 64; ++kb)
          tma_load_4d_h(s_in + s * L::kIn + kb * (kTile * 128), second ? &tm_b : &tm_a, in_full + s, kb * 64,
                        (second ? trb.tile(i - count) : tra.tile(i)) * kTile, tr_ch, tr_cb, second ? pol_b : pol_a);
        armed = i + 1;
      }
      if (ab.raised())
        for (int i = max(0, armed - kStages); i < armed; ++i) mbar_drain(in_full + (i % kStages), (i / kStages) & 1);
    }
  } else if (warp == kIssuer) {
    if (lane == 0) {
      constexpr uint32_t idesc_o = make_idesc<T>(kTile, D, false, true);
      const uint32_t a_op = smem_u32(s_op);
      bool ok = mbar_wait(small_full, 0, ab, 0x2200);
      for (int i = 0; ok && i < total; ++i) {
        const int s = i % kStages;
        const uint32_t par = (uint32_t)(i / kStages) & 1u;
        const uint32_t a_b = a_op + (i >= count ? L::kOp : 0);
        // the accumulator of this stage was last read by tile i - kStages
        if (!mbar_wait(o_free + s, par ^ 1, ab, 0x2380 + i)) break;
        if (!mbar_wait(in_full + s, par, ab, 0x2300 + i)) break;
        tc_fence_after();
        const uint32_t a_ds = smem_u32(s_in + s * L::kIn);
        // (128 x MP, K-major) * (MP x D, MN-major view of the landmark operand)
#pragma unroll
        for (int k = 0; k < MP / 16; ++k)
          umma(tmem_base + s * D, kdesc(a_ds, k, kTile), smem_desc_sw128(a_b + k * 2048, MP * 128, 1024),
               idesc_o, k > 0);
        umma_commit(in_empty + s);
        umma_commit(acc_done + s);
      }
    }
  } else {
    const int g = warp >> 2;
    const int r = threadIdx.x & 127;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    if (threadIdx.x < kComputeThreads) {   // (uniform per warp)
      pack_landmark_operand<T, D, MP>(s_op, side_a.landmarks + bh * m * D, m, op_mul);
      if (nsides > 1) pack_landmark_operand<T, D, MP>(s_op + L::kOp, side_b.landmarks + bh * m * D, m, op_mul);
      fence_proxy_async();
      mbar_arrive_warp(small_full);
    }
    const float mul_a = (side_a.out_scale ? side_a.out_scale[bh] : 1.f) * side_a.out_mul;
    const float mul_b = nsides > 1 ? (side_b.out_scale ? side_b.out_scale[bh] : 1.f) * side_b.out_mul : 0.f;
    uint8_t* my_out = s_out + g * L::kOut;
    const bool leader = r == 0;
    const int64_t total_tiles = (sch.N + kTile - 1) / kTile;
    const uint64_t pol_oa = leader ? l2_policy_of(sch.hint, 2) : 0ull, pol_ob = leader ? l2_policy_of(sch.hint, 3) : 0ull;
    Segments sg(sch.seg_N, m);
    // the landmark rows of this CTA's tiles on a side whose rows still wait for the column-pass
    // partials (all landmarks between its lowest and its highest tile)
    auto presum = [&](const RowsSide& sd, const TileRange& t) {
      if (!sd.part || t.count <= 0) return;
      const int64_t first = sch.row_offset + (int64_t)t.lowest() * kTile;
      const int64_t last = sch.row_offset + min((int64_t)(t.highest() + 1) * kTile, sch.N) - 1;
      const int l_lo = sg.landmark_of(first), nl = sg.landmark_of(last) - l_lo + 1;
      const int md = m * D;
      for (int item = threadIdx.x; item < nl * (D / 4); item += kCompute) {
        const int l = l_lo + item / (D / 4), d = (item % (D / 4)) * 4;
        const float* src = sd.part + bh * (int64_t)sd.nchunk * md + l * D + d;
        float4 acc = *reinterpret_cast<const float4*>(sd.base + bh * md + l * D + d);
        for (int c = 0; c < sd.nchunk; ++c) {
          const float4 x = *reinterpret_cast<const float4*>(src + (int64_t)c * md);
          acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        }
        const float f = sd.rows_scale / (float)sg.len(l);
        *reinterpret_cast<float4*>(sd.rows + bh * md + l * D + d) = make_float4(acc.x * f, acc.y * f, acc.z * f, acc.w * f);
      }
    };
    presum(side_a, tra);
    if (nsides > 1) presum(side_b, trb);
    if (side_a.part || (nsides > 1 && side_b.part))
      named_barrier(5, kCompute);   // the stores above are visible to the CTA's epilogue reads
    for (int i = g; i < total; i += kGroups) {
      if (i == kGroups) TC_SPAN(3);
      const int s = i % kStages;
      const uint32_t par = (uint32_t)(i / kStages) & 1u;
      const bool second = i >= count;
      const int tile = second ? trb.tile(i - count) : tra.tile(i);
      const int64_t row = (int64_t)tile * kTile + r;
      const bool valid = row < sch.N;
      const int l = valid ? sg.landmark_of(sch.row_offset + row) : 0;
      const float4* add = reinterpret_cast<const float4*>((second ? side_b.rows : side_a.rows) + (bh * m + l) * D);
      const float* tsc = second ? side_b.tile_scale : side_a.tile_scale;
      const float mul = (second ? mul_b : mul_a) * (tsc ? tsc[bh * total_tiles + tile] : 1.f);
      const uint32_t t_o = tmem_base + s * D + lane_base;
      if (!mbar_wait(acc_done + s, par, ab, 0x2800 + i)) break;
      __syncwarp();
      tc_fence_after();
      // the previous tile of this group was stored from my_out: wait until the copy has read it
      if (leader) tma_store_wait_read();
      named_barrier(1 + g, kGroup);
#pragma unroll
      for (int hf = 0; hf < D / 32; ++hf) {
        float o[32];
        tmem_ld32(t_o + hf * 32, o);
        tmem_ld_wait();
        if (hf == D / 32 - 1) {
          tc_fence_before();
          mbar_arrive_warp(o_free + s);
        }
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 a = add[(hf * 32 + j) >> 2];
          o[j + 0] = fmaf(o[j + 0], mul, a.x); o[j + 1] = fmaf(o[j + 1], mul, a.y);
          o[j + 2] = fmaf(o[j + 2], mul, a.z); o[j + 3] = fmaf(o[j + 3], mul, a.w);
        }
        store_cols<T, 32>(my_out, r, hf * 32, o);
      }
      fence_proxy_async();
      named_barrier(1 + g, kGroup);
      if (leader) {
        for (int kb = 0; kb < D / 64; ++kb)
          tma_store_4d_h(second ? &tm_b : &tm_a, my_out + kb * (kTile * 128), kb * 64, tile * kTile, tr_ch, tr_cb,
                         second ? pol_ob : pol_oa);
        tma_store_commit();
      }
    }
    TC_SPAN(4);
    if (leader) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
  TC_SPAN(1);
}

// ------------------------------------------------------------------------------------------
// Softmax-3 backward (column pass).  Per 128-row tile of K and V (thread = row n, half the
// landmark columns):
//   S3^T = K qt16^T (log2 domain), dP3^T = V do3n^T (dO3 normalised by 2^-e, undone by dsc)
//   P' = 2^k exp(S3 - lse3) , dS' = P' o (dP3 - D3)     (2^k keeps the 16-bit operand copies of
//                                                         the ~1/N probabilities out of the
//                                                         subnormal range; undone in FP32)
//   dV = P' dO3                     -> written once (dO3 read as the MN-major view of do3n)
//   dS' tile                        -> written as it is into the dK tile of the same rows (same
//                                      footprint); the in-place pass turns it into
//                                      dK = s dS' Qt + rows_k[l(n)] once the landmark gradients
//                                      are known, so this pass does not wait for the
//                                      pseudoinverse backward
//   dQt partial += dS'^T (sK)       -> TMEM accumulator over the CTA's tiles
// K is double-buffered (it is needed until the tile's last product), V single-buffered.
template <int D, int MP>
struct BwdBSmem {
  static constexpr int kOp = MP * D * 2, kVec = 1024, kIn = kTile * D * 2,
                       kPd = kTile * (MP > D ? MP : D) * 2;
  static constexpr int kBytes = 2 * kOp + kVec + 3 * kIn + 2 * kPd + 256 + 1024;
};

template <class T, int D, int MP>
__global__ void __launch_bounds__(kTcThreads, (D == 64 ? 2 : 1))
tc_bwd_b_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                const __grid_constant__ CUtensorMap tm_qt, const __grid_constant__ CUtensorMap tm_do3,
                const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                const float* __restrict__ lse3, const float* __restrict__ D3,
                const float* __restrict__ do3_scale,
                float* __restrict__ partB, float* __restrict__ tile_scale, TcSched sch, int m, float scale, int kshift,
                int* status) {
  using L = BwdBSmem<D, MP>;
  constexpr int kTraceId = 2; (void)kTraceId;
  TC_SPAN(0);
  constexpr int KBD = D / 64, HC = MP / 2, HD = D / 2;
  constexpr int W = MP > D ? MP : D;
  constexpr uint32_t kCols = 2 * W + 2 * D;   // S, dP, the dQt accumulator, dV
  constexpr uint32_t kTmemCols = kCols <= 256 ? 256 : 512;
  static_assert(kCols <= 512, "tensor memory");
  extern __shared__ uint8_t smem_raw[];
  pdl_trigger();
  uint8_t* base = align1024(smem_raw);
  uint8_t* s_qt = base;
  uint8_t* s_do3 = s_qt + L::kOp;
  float* s_c3 = reinterpret_cast<float*>(s_do3 + L::kOp);
  float* s_d3 = s_c3 + MP;
  uint8_t* s_k = reinterpret_cast<uint8_t*>(s_c3) + L::kVec;   // two stages
  uint8_t* s_v = s_k + 2 * L::kIn;
  uint8_t* s_p = s_v + L::kIn;      // P' tile, then staging of the dV tile
  uint8_t* s_ds = s_p + L::kPd;     // dS' tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_ds + L::kPd);
  uint64_t* small_full = bars + 0;
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 6;
  uint64_t* sdp_full = bars + 7;
  uint64_t* pds_full = bars + 8;
  uint64_t* out_full = bars + 9;    // the products of a tile are complete
  uint64_t* ds_free = bars + 10;    // the copy of a tile's dS' has read the shared-memory tile
  unsigned* s_tmax = reinterpret_cast<unsigned*>(bars + 12);   // [2]: largest |dS'| of a tile (float bits), by tile parity
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  int* abort_word = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileRange tr = tile_range(sch);
  const int tr_ch = tr.ch, tr_cb = tr.cb;
  const int64_t bh = tr.bh;
  const int count = tr.count;

  if (threadIdx.x == 0) {
    mbar_init(small_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); }
    mbar_init(v_full, 1); mbar_init(v_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, kComputeThreads / 32);
    mbar_init(out_full, 1);
    mbar_init(ds_free, 1);
    *abort_word = 0;
    s_tmax[0] = 0; s_tmax[1] = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();   // everything above overlaps the tail of the previous kernel of the stream
  TC_SPAN(2);
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + W, tmem_acc = tmem_base + 2 * W;
  const uint32_t tmem_dv = tmem_acc + D;   // columns of its own: the scores of the next tile are formed while dV is read
  Abort ab{abort_word, status};

  if (warp == kProducerWarp) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      const uint64_t pol_k = l2_policy_of(sch.hint, 0), pol_v = l2_policy_of(sch.hint, 1);
      mbar_expect_tx(small_full, 2 * L::kOp);
      for (int kb = 0; kb < KBD; ++kb) {
        tma_load_2d(s_qt + kb * (MP * 128), &tm_qt, small_full, kb * 64, (int)(bh * MP));
        tma_load_2d(s_do3 + kb * (MP * 128), &tm_do3, small_full, kb * 64, (int)(bh * MP));
      }
      int armed = 0;
      for (int i = 0; i < count; ++i) {
        const int st = i & 1;
        if (!mbar_wait(k_empty + st, ((i >> 1) & 1) ^ 1, ab, 0x2100 + i)) break;
        mbar_expect_tx(k_full + st, L::kIn);
        for (int kb = 0; kb < KBD; ++kb)
          tma_load_4d_h(s_k + st * L::kIn + kb * (kTile * 128), &tm_k, k_full + st, kb * 64, tr.tile(i) * kTile, tr_ch, tr_cb, pol_k);
        if (!mbar_wait(v_empty, (i & 1) ^ 1, ab, 0x2180 + i)) { armed = -(i + 1); break; }
        mbar_expect_tx(v_full, L::kIn);
        for (int kb = 0; kb < KBD; ++kb)
          tma_load_4d_h(s_v + kb * (kTile * 128), &tm_v, v_full, kb * 64, tr.tile(i) * kTile, tr_ch, tr_cb, pol_v);
        armed = i + 1;
      }
      if (ab.raised()) {
        const int nk = armed < 0 ? -armed : armed, nv = armed < 0 ? -armed - 1 : armed;
        for (int i = max(0, nk - 2); i < nk; ++i) mbar_drain(k_full + (i & 1), (i >> 1) & 1);
        if (nv > 0) mbar_drain(v_full, (nv - 1) & 1);
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc<T>(kTile, MP, false, false);
      constexpr uint32_t idesc_o = make_idesc<T>(kTile, D, false, true);
      constexpr uint32_t idesc_acc = make_idesc<T>(MP, D, true, true);
      const uint32_t a_qt = smem_u32(s_qt), a_do3 = smem_u32(s_do3), a_v = smem_u32(s_v), a_p = smem_u32(s_p),
                     a_ds = smem_u32(s_ds);
      const uint64_t pol_ds = l2_policy_of(sch.hint, 2);
      // S and dP of tile i (their tensor-memory columns are free once the compute warps have read
      // those of tile i - 1, which they have when they hand over its P' and dS')
      auto front = [&](int i) -> bool {
        const int st = i & 1;
        if (!mbar_wait(k_full + st, (i >> 1) & 1, ab, 0x2300 + i)) return false;
        if (!mbar_wait(v_full, i & 1, ab, 0x2340 + i)) return false;
        TC_TRACE(1, i);
        tc_fence_after();
        const uint32_t a_k = smem_u32(s_k + st * L::kIn);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma(tmem_s, kdesc(a_k, k, kTile), kdesc(a_qt, k, MP), idesc_s, k > 0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma(tmem_dp, kdesc(a_v, k, kTile), kdesc(a_do3, k, MP), idesc_s, k > 0);
        umma_commit(v_empty);
        umma_commit(sdp_full);
        return true;
      };
      bool ok = mbar_wait(small_full, 0, ab, 0x2200);
      ok = ok && front(0);
      for (int i = 0; ok && i < count; ++i) {
        const int st = i & 1;
        const uint32_t a_k = smem_u32(s_k + st * L::kIn);
        if (!mbar_wait(pds_full, i & 1, ab, 0x2400 + i)) break;
        TC_TRACE(2, i);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < MP / 16; ++k)
          umma(tmem_dv, kdesc(a_p, k, kTile), smem_desc_sw128(a_do3 + k * 2048, MP * 128, 1024), idesc_o, k > 0);
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)
          umma(tmem_acc, mndesc(a_ds, k), mndesc(a_k, k), idesc_acc, (i > 0 || k > 0));
        umma_commit(k_empty + st);
        umma_commit(out_full);
        // the dS' tile as it is -> dK tile of the same rows
        for (int kb = 0; kb < MP / 64; ++kb)
          tma_store_4d_h(&tm_dk, s_ds + kb * (kTile * 128), kb * 64, tr.tile(i) * kTile, tr_ch, tr_cb, pol_ds);
        tma_store_commit();
        // the scores of the next tile run while the compute warps take this tile's dV out
        if (i + 1 < count && !front(i + 1)) break;
        // ds_free lets the compute warps write the next dS' tile: the copy must have read this one
        tma_store_wait_read();
        TC_TRACE(3, i);
        mbar_arrive(ds_free);
      }
      tma_store_wait_all();
    }
  } else {
    const int r = threadIdx.x & 127, h = threadIdx.x >> 7;
    const int quarter = warp & 3;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float dsc = do3_scale[bh];
    const float unshift = exp2f(-(float)kshift);
    const uint64_t pol_dv = threadIdx.x == 0 ? l2_policy_of(sch.hint, 3) : 0ull;
    const int c0 = h * HC;
    Segments sg(sch.seg_N, m);
    if (threadIdx.x < MP) {
      const int j = threadIdx.x;
      s_c3[j] = (j < m) ? lse3[bh * m + j] * kLog2e - (float)kshift : INFINITY;
      s_d3[j] = (j < m) ? D3[bh * m + j] : 0.f;   // times frun (below), which starts at 1
    }
    named_barrier(1, kComputeThreads);
    bool alive = true;
    // running power-of-two factor of the stored dS' tiles (fp16 only; see below), folded into the
    // two constants dS' is formed from
    float frun = 1.f, dscf = dsc;
    const int64_t total_tiles = (sch.N + kTile - 1) / kTile;
    for (int i = 0; i < count; ++i) {
      if (i == 1) TC_SPAN(3);
      const int64_t row = (int64_t)tr.tile(i) * kTile + r;
      const bool valid = row < sch.N;
      if (!mbar_wait(sdp_full, i & 1, ab, 0x2600 + i)) { alive = false; break; }
      if (threadIdx.x == 0) TC_TRACE(4, i);
      __syncwarp();
      tc_fence_after();
      float p[HC], g[HC];
      ld_cols<HC>(tmem_s + lane_base + c0, p);
      ld_cols<HC>(tmem_dp + lane_base + c0, g);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < HC; j += 4) {
        const float4 c = *reinterpret_cast<const float4*>(s_c3 + c0 + j);
        const float4 d = *reinterpret_cast<const float4*>(s_d3 + c0 + j);
        p[j + 0] = valid ? fast_exp2(p[j + 0] - c.x) : 0.f;
        p[j + 1] = valid ? fast_exp2(p[j + 1] - c.y) : 0.f;
        p[j + 2] = valid ? fast_exp2(p[j + 2] - c.z) : 0.f;
        p[j + 3] = valid ? fast_exp2(p[j + 3] - c.w) : 0.f;
        g[j + 0] = p[j + 0] * fmaf(g[j + 0], dscf, -d.x);
        g[j + 1] = p[j + 1] * fmaf(g[j + 1], dscf, -d.y);
        g[j + 2] = p[j + 2] * fmaf(g[j + 2], dscf, -d.z);
        g[j + 3] = p[j + 3] * fmaf(g[j + 3], dscf, -d.w);
      }
      // fp16 only: the 16-bit copy of dS' = f 2^k P3 (dP3 - D3) must stay inside the fp16 range whatever
      // the data (a peaked softmax-3 makes P3 ~ 1, an unnormalised dO makes dP3 large).  Every tile
      // finds its largest magnitude (one redux per warp, one shared atomic, the barrier that is
      // needed anyway); when it would pass 2^15 the CTA lowers its running power-of-two factor f,
      // rescales the dQt accumulator it has built so far by the same ratio and goes on.  f only
      // ever falls, so nothing overflows; the factor each tile was stored with goes to global
      // memory for the in-place pass that turns the tile into dK.
      if (std::is_same<T, __half>::value) {
        float big = 0.f;
#pragma unroll
        for (int j = 0; j < HC; j += 2) big = fmaxf(big, fmaxf(fabsf(g[j]), fabsf(g[j + 1])));
        const unsigned wb = __reduce_max_sync(0xffffffffu, __float_as_uint(big));
        if (lane == 0) atomicMax(s_tmax + (i & 1), wb);
      }
      // the staging copies of the previous tile's dV / dK share these buffers
      if (threadIdx.x == 0) {
        TC_TRACE(0, i);
        tma_store_wait_read();
        s_tmax[(i + 1) & 1] = 0;   // read for the last time before the previous tile's second barrier
      }
      // ... and the copy of the previous dS' tile must have read it
      if (i > 0 && !mbar_wait(ds_free, (i - 1) & 1, ab, 0x2700 + i)) { alive = false; break; }
      named_barrier(1, kComputeThreads);
      if (std::is_same<T, __half>::value) {
        const float tmax = __uint_as_float(s_tmax[i & 1]);   // CTA-uniform, already times frun
        if (!(tmax <= 32768.f)) {
          // non-finite input: reported; the values go through as they are
          if (!(tmax < 1e30f) && status) atomicCAS(status, 0, (kStatusRange << 24) | 0x2b00);
          // tmax = 1.x * 2^(E - 127) < 2^(E - 126): ratio = 2^(15 - (E - 126)) brings it below 2^15
          const uint32_t E = (s_tmax[i & 1] >> 23) & 0xffu;
          const float ratio = __uint_as_float((268u - E) << 23);   // < 1: new factor = ratio * frun
#pragma unroll
          for (int j = 0; j < HC; ++j) g[j] *= ratio;
          if (i > 0) {
            for (int cc = 0; cc < HD; cc += 8) {    // eight columns at a time: this path is rare, registers are not
              float o[8];
              tmem_ld8(tmem_acc + lane_base + h * HD + cc, o);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 8; ++j) o[j] *= ratio;
              tmem_st8(tmem_acc + lane_base + h * HD + cc, o);
            }
            tmem_st_wait();
          }
          // every thread has read s_d3 for this tile (barrier above); the next read comes after the
          // barrier that ends this tile
          if (threadIdx.x < MP) s_d3[threadIdx.x] *= ratio;
          frun *= ratio;
          dscf *= ratio;
        }
      }
      if (threadIdx.x == 0 && tile_scale) tile_scale[bh * total_tiles + tr.tile(i)] = 1.f / frun;
      if (threadIdx.x == 0) TC_TRACE(5, i);
      store_cols<T, HC>(s_p, r, c0, p);
      store_cols<T, HC>(s_ds, r, c0, g);
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive_warp(pds_full);

      if (!mbar_wait(out_full, i & 1, ab, 0x2800 + i)) { alive = false; break; }
      if (threadIdx.x == 0) TC_TRACE(6, i);
      __syncwarp();
      tc_fence_after();
      float o[HD];
      ld_cols<HD>(tmem_dv + lane_base + h * HD, o);
      tmem_ld_wait();
      const float vmul = dsc * unshift;
#pragma unroll
      for (int j = 0; j < HD; ++j) o[j] *= vmul;
      // out_full: every product that read the P' tile is complete, so it can hold the outgoing
      // dV tile now
      store_cols<T, HD>(s_p, r, h * HD, o);
      fence_proxy_async();
      named_barrier(1, kComputeThreads);
      if (threadIdx.x == 0) {
        for (int kb = 0; kb < KBD; ++kb)
          tma_store_4d_h(&tm_dv, s_p + kb * (kTile * 128), kb * 64, tr.tile(i) * kTile, tr_ch, tr_cb, pol_dv);
        tma_store_commit();
        TC_TRACE(7, i);
      }
    }
    TC_SPAN(4);
    if (threadIdx.x == 0) tma_store_wait_all();
    if (alive) {
      // out_full of the last tile was waited above, so the accumulator is final
      const int l = (MP == 128) ? r : (quarter * 16 + lane);
      const bool owner = (MP == 128) ? true : (lane < 16);
      float* dst = partB + ((size_t)bh * sch.nchunk + tr.chunk) * m * D;
      const float mul = scale * unshift / frun;
      float o[HD];
      ld_cols<HD>(tmem_acc + lane_base + h * HD, o);
      tmem_ld_wait();
      if (owner && l < m) {
#pragma unroll
        for (int j = 0; j < HD; j += 4)
          *reinterpret_cast<float4*>(dst + l * D + h * HD + j) =
              make_float4(o[j] * mul, o[j + 1] * mul, o[j + 2] * mul, o[j + 3] * mul);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
  TC_SPAN(1);
}

// ------------------------------------------------------------------------------------------
// Softmax-3 forward (column pass): per-CTA partial of Bmat = softmax(Qt (sK)^T) V with a running
// reference exponent per landmark.  Thread = row n of the K/V tile and half the landmark columns,
// so the per-landmark maximum over the tile is a reduction across threads (31 warp shuffles per
// thread fold the 32 rows of a warp, shared memory folds the 4 row quarters).  The reference only
// moves when a score exceeds it by more than 2^8 (then the TMEM accumulators are rescaled in
// place), so probabilities stay <= 256 in the 16-bit operand copy, and whether any score does is
// one compare per element and one barrier with an OR: the maximum is formed for those tiles only.  Row
// sums come from the tensor core too (P'^T times a block of ones).  S is double-buffered in
// TMEM and P' in shared memory (a tile's probabilities are written while the previous tile's
// accumulation still reads its own copy); K and V have separate two-stage rings (K is free
// after the score product, V after the accumulation).
template <int D, int MP>
struct FwdBSmem {
  static constexpr int kQt = MP * D * 2, kOnes = 2048, kIn = kTile * D * 2, kP = kTile * MP * 2,
                       kAux = 1024 * ((7 * MP * 4 + 64 + 1023) / 1024);
  // V is double-buffered unless 128 landmarks x head_dim 128 leave no room for the second stage
  static constexpr int kVStages = (MP == 128 && D == 128) ? 1 : 2;
  static constexpr int kBytes = kQt + kOnes + (2 + kVStages) * kIn + 2 * kP + kAux + 256 + 1024;
};

template <class T, int D, int MP>
__global__ void __launch_bounds__(kTcThreads, (D == 64 ? 2 : 1))
tc_fwd_b_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                const __grid_constant__ CUtensorMap tm_qt, const float* __restrict__ land, int land_chunks,
                int64_t land_bh, float scale, float* __restrict__ part_acc,
                float* __restrict__ part_max, float* __restrict__ part_sum, TcSched sch, int m,
                int* status) {
  using L = FwdBSmem<D, MP>;
  constexpr int kTraceId = 0; (void)kTraceId;
  TC_SPAN(0);
  constexpr int KBD = D / 64, HC = MP / 2;
  constexpr int CPL = HC / 32;                 // columns per lane after the warp fold
  constexpr int NCK = (D + 32) / 32;           // 32-column chunks of accumulator + row sums
  constexpr uint32_t kCols = 2 * MP + D + 32;
  constexpr uint32_t kTmemCols = kCols <= 256 ? 256 : 512;
  extern __shared__ uint8_t smem_raw[];
  pdl_trigger();
  uint8_t* base = align1024(smem_raw);
  uint8_t* s_qt = base;
  uint8_t* s_ones = s_qt + L::kQt;
  uint8_t* s_k = s_ones + L::kOnes;            // two stages
  constexpr int VS = L::kVStages;
  uint8_t* s_v = s_k + 2 * L::kIn;             // VS stages
  uint8_t* s_p = s_v + VS * L::kIn;            // two buffers, tile parity
  float* s_wmax = reinterpret_cast<float*>(s_p + 2 * L::kP);   // [4][MP]
  float* s_ref = s_wmax + 4 * MP;                          // [MP] running reference (log2 domain)
  float* s_fac = s_ref + MP;                               // [MP] rescale factor of this tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(s_wmax) + L::kAux);
  uint64_t* small_full = bars + 0;
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* v_full = bars + 5;      // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2]
  uint64_t* p_full = bars + 11;     // [2], tile parity
  uint64_t* acc_done = bars + 13;   // [2], tile parity
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  int* abort_word = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileRange tr = tile_range(sch);
  const int tr_ch = tr.ch, tr_cb = tr.cb;
  const int64_t bh = tr.bh;
  const int count = tr.count;

  if (threadIdx.x == 0) {
    mbar_init(small_full, land ? kComputeThreads / 32 : 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1);
      mbar_init(s_full + s, 1);
    }
    mbar_init(p_full, kComputeThreads / 32);
    mbar_init(p_full + 1, kComputeThreads / 32);
    mbar_init(acc_done, 1);
    mbar_init(acc_done + 1, 1);
    *abort_word = 0;
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
  pdl_wait();   // everything above overlaps the tail of the previous kernel of the stream
  TC_SPAN(2);
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_acc = tmem_base + 2 * MP;   // D accumulator columns, then 32 for the row sums
  Abort ab{abort_word, status};

  if (warp == kProducerWarp) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      const uint64_t pol_k = l2_policy_of(sch.hint, 0), pol_v = l2_policy_of(sch.hint, 1);
      if (!land) {
        mbar_expect_tx(small_full, L::kQt);
        for (int kb = 0; kb < KBD; ++kb)
          tma_load_2d(s_qt + kb * (MP * 128), &tm_qt, small_full, kb * 64, (int)(bh * MP));
      }
      int nk = 0, nv = 0;
      for (int i = 0; i < count; ++i) {
        const int st = i & 1;
        if (!mbar_wait(k_empty + st, ((i >> 1) & 1) ^ 1, ab, 0x3100 + i)) break;
        mbar_expect_tx(k_full + st, L::kIn);
        for (int kb = 0; kb < KBD; ++kb)
          tma_load_4d_h(s_k + st * L::kIn + kb * (kTile * 128), &tm_k, k_full + st, kb * 64, tr.tile(i) * kTile, tr_ch, tr_cb, pol_k);
        TC_TRACE(0, i);
        nk = i + 1;
        const int sv = i % VS;
        if (!mbar_wait(v_empty + sv, ((i / VS) & 1) ^ 1, ab, 0x3180 + i)) break;
        mbar_expect_tx(v_full + sv, L::kIn);
        for (int kb = 0; kb < KBD; ++kb)
          tma_load_4d_h(s_v + sv * L::kIn + kb * (kTile * 128), &tm_v, v_full + sv, kb * 64, tr.tile(i) * kTile, tr_ch, tr_cb, pol_v);
        TC_TRACE(1, i);
        nv = i + 1;
      }
      if (ab.raised()) {
        for (int i = max(0, nk - 2); i < nk; ++i) mbar_drain(k_full + (i & 1), (i >> 1) & 1);
        for (int i = max(0, nv - VS); i < nv; ++i) mbar_drain(v_full + (i % VS), (i / VS) & 1);
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc<T>(kTile, MP, false, false);
      constexpr uint32_t idesc_acc = make_idesc<T>(MP, D, true, true);
      constexpr uint32_t idesc_sum = make_idesc<T>(MP, 16, true, false);
      const uint32_t a_qt = smem_u32(s_qt), a_p = smem_u32(s_p), a_ones = smem_u32(s_ones);
      auto front = [&](int i) -> bool {
        const int st = i & 1;
        if (!mbar_wait(k_full + st, (i >> 1) & 1, ab, 0x3300 + i)) return false;
        TC_TRACE(2, i);
        tc_fence_after();
        const uint32_t a_k = smem_u32(s_k + st * L::kIn);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma(tmem_base + st * MP, kdesc(a_k, k, kTile), kdesc(a_qt, k, MP), idesc_s, k > 0);
        umma_commit(k_empty + st);
        umma_commit(s_full + st);
        return true;
      };
      bool ok = mbar_wait(small_full, 0, ab, 0x3200);
      ok = ok && front(0);
      if (ok && count > 1) ok = front(1);
      for (int i = 0; ok && i < count; ++i) {
        const int st = i & 1;
        if (!mbar_wait(p_full + st, (i >> 1) & 1, ab, 0x3400 + i)) break;
        TC_TRACE(3, i);
        const int sv = i % VS;
        if (!mbar_wait(v_full + sv, (i / VS) & 1, ab, 0x3480 + i)) break;
        TC_TRACE(4, i);
        tc_fence_after();
        const uint32_t a_v = smem_u32(s_v + sv * L::kIn);
        const uint32_t a_pi = a_p + st * L::kP;
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)
          umma(tmem_acc, mndesc(a_pi, k), mndesc(a_v, k), idesc_acc, (i > 0 || k > 0));
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)
          umma(tmem_acc + D, mndesc(a_pi, k), smem_desc_sw128(a_ones + (k & 3) * 32, 16, 1024), idesc_sum,
               (i > 0 || k > 0));
        umma_commit(v_empty + sv);
        umma_commit(acc_done + st);
        if (i + 2 < count) ok = front(i + 2);
      }
    }
  } else {
    const int r = threadIdx.x & 127, h = threadIdx.x >> 7;
    const int quarter = warp & 3;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int c0 = h * HC;
    const int lrow = (MP == 128) ? r : (quarter * 16 + lane);          // accumulator row of this lane
    const bool owner = (MP == 128) ? true : (lane < 16);
    if (threadIdx.x < MP) s_ref[threadIdx.x] = -INFINITY;
    if (land) {
      // 16-bit landmark operand s*log2e*Qt straight from the raw segment sums of the pooling pass
      float qv[16];
      pooled_row16(land, 0, land_bh, bh, m, land_chunks, sch.seg_N, scale, qv);
      const float mul = scale * kLog2e;
      const int pr = threadIdx.x >> 2, pc = (threadIdx.x & 3) * 2;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint4 wq;
        wq.x = pack2<T>(qv[8 * c + 0] * mul, qv[8 * c + 1] * mul); wq.y = pack2<T>(qv[8 * c + 2] * mul, qv[8 * c + 3] * mul);
        wq.z = pack2<T>(qv[8 * c + 4] * mul, qv[8 * c + 5] * mul); wq.w = pack2<T>(qv[8 * c + 6] * mul, qv[8 * c + 7] * mul);
        *reinterpret_cast<uint4*>(s_qt + sw128_offset(pr, pc + c)) = wq;
      }
      fence_proxy_async();
      mbar_arrive_warp(small_full);
    }
    named_barrier(1, kComputeThreads);   // s_ref is read before the first barrier of the loop
    bool alive = true;
    for (int i = 0; i < count; ++i) {
      if (i == 1) TC_SPAN(3);
      const int st = i & 1;
      const int64_t row = (int64_t)tr.tile(i) * kTile + r;
      const bool valid = row < sch.N;
      if (!mbar_wait(s_full + st, (i >> 1) & 1, ab, 0x3600 + i)) { alive = false; break; }
      if (threadIdx.x == 0) TC_TRACE(5, i);
      __syncwarp();
      tc_fence_after();
      float s[HC];
      ld_cols<HC>(tmem_base + st * MP + lane_base + c0, s);
      tmem_ld_wait();
      // s <- s - reference.  Does any difference exceed 8 (a score 2^8 above its landmark's
      // reference)?  One compare per element and one barrier with an OR; the tile maximum is only
      // formed when one does, from the scores read out of tensor memory again.
      bool over = false;
#pragma unroll
      for (int j = 0; j < HC; j += 4) {
        const float4 c = *reinterpret_cast<const float4*>(s_ref + c0 + j);
        s[j + 0] = (valid ? s[j + 0] : -INFINITY) - c.x; s[j + 1] = (valid ? s[j + 1] : -INFINITY) - c.y;
        s[j + 2] = (valid ? s[j + 2] : -INFINITY) - c.z; s[j + 3] = (valid ? s[j + 3] : -INFINITY) - c.w;
        over |= (s[j + 0] > 8.f) | (s[j + 1] > 8.f) | (s[j + 2] > 8.f) | (s[j + 3] > 8.f);
      }
      const bool move = named_barrier_or(1, kComputeThreads, over);     // CTA-uniform
      if (threadIdx.x == 0) TC_TRACE(6, i);
      if (i > 1) {
        // the accumulation of tile i-2 read the P' buffer this tile is about to fill
        if (!mbar_wait(acc_done + st, (uint32_t)((i - 2) >> 1) & 1u, ab, 0x3700 + i)) { alive = false; break; }
        __syncwarp();
      }
      if (move) {
        ld_cols<HC>(tmem_base + st * MP + lane_base + c0, s);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < HC; ++j) s[j] = valid ? s[j] : -INFINITY;
        // fold the 32 rows of this warp in place: afterwards lane L holds columns c0 + CPL*L .. +CPL-1
#pragma unroll
        for (int off = 16, cnt = HC / 2; off >= 1; off >>= 1, cnt >>= 1) {
          const bool upper = (lane & off) != 0;
#pragma unroll
          for (int j = 0; j < cnt; ++j) {
            const float send = upper ? s[j] : s[j + cnt];
            const float keep = upper ? s[j + cnt] : s[j];
            s[j] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, off));
          }
        }
#pragma unroll
        for (int j = 0; j < CPL; ++j) s_wmax[quarter * MP + c0 + CPL * lane + j] = s[j];
        if (i > 0) {
          // the accumulators are rescaled in place: every accumulation issued so far must be complete
          if (!mbar_wait(acc_done + (st ^ 1), (uint32_t)((i - 1) >> 1) & 1u, ab, 0x3780 + i)) { alive = false; break; }
          __syncwarp();
          tc_fence_after();
        }
        named_barrier(1, kComputeThreads);
        if (threadIdx.x < MP) {
          const int c = threadIdx.x;
          const float tmax = fmaxf(fmaxf(s_wmax[c], s_wmax[MP + c]), fmaxf(s_wmax[2 * MP + c], s_wmax[3 * MP + c]));
          const float old = s_ref[c], nw = fmaxf(old, tmax);
          s_fac[c] = (old == -INFINITY) ? 0.f : fast_exp2(old - nw);
          s_ref[c] = nw;
        }
        named_barrier(1, kComputeThreads);
        if (i > 0) {
          const float f = s_fac[owner ? lrow : 0];
#pragma unroll
          for (int ck = 0; ck < NCK; ++ck) {
            if ((ck & 1) == h) {
              float o[32];
              tmem_ld32(tmem_acc + lane_base + ck * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) o[j] *= f;
              tmem_st32(tmem_acc + lane_base + ck * 32, o);
            }
          }
          tmem_st_wait();
        }
        // the scores once more, against the new reference
        ld_cols<HC>(tmem_base + st * MP + lane_base + c0, s);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < HC; j += 4) {
          const float4 c = *reinterpret_cast<const float4*>(s_ref + c0 + j);
          s[j + 0] = (valid ? s[j + 0] : -INFINITY) - c.x; s[j + 1] = (valid ? s[j + 1] : -INFINITY) - c.y;
          s[j + 2] = (valid ? s[j + 2] : -INFINITY) - c.z; s[j + 3] = (valid ? s[j + 3] : -INFINITY) - c.w;
        }
      }
#pragma unroll
      for (int j = 0; j < HC; ++j) s[j] = fast_exp2(s[j]);
      store_cols<T, HC>(s_p + st * L::kP, r, c0, s);
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive_warp(p_full + st);
      if (threadIdx.x == 0) TC_TRACE(7, i);
    }
    TC_SPAN(4);
    if (alive && mbar_wait(acc_done + ((count - 1) & 1), (uint32_t)((count - 1) >> 1) & 1u, ab, 0x3900)) {
      __syncwarp();
      tc_fence_after();
      const size_t slot = (size_t)bh * sch.nchunk + tr.chunk;
      float* dst = part_acc + slot * m * D;
#pragma unroll
      for (int ck = 0; ck < NCK; ++ck) {
        if ((ck & 1) == h) {
          float o[32];
          tmem_ld32(tmem_acc + lane_base + ck * 32, o);
          tmem_ld_wait();
          if (owner && lrow < m) {
            if (ck < D / 32) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(dst + lrow * D + ck * 32 + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
            } else {
              part_sum[slot * m + lrow] = o[0];
              part_max[slot * m + lrow] = s_ref[lrow] * kLn2;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
  TC_SPAN(1);
}

}  // namespace tc
}  // namespace fnb
